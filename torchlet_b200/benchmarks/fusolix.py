"""Prefill and decode throughput of the Fusolix design at layer sizes that resemble a real model's, beside the
closest existing design of equal size: Numuzen (a recurrent mixer with a float32 state per head, a windowed softmax
attention, routed gated experts; same width, layers, heads, window and vocabulary).

    python -m torchlet_b200.benchmarks.fusolix [--size 2b|1b] [--layers N] [--prefill 2048] [--batch 8]
                                               [--context 2048] [--steps 32] [--kernels]

Random bfloat16 weights made on the GPU.  Prefill: one request's whole prompt in one step (CUDA events around the
step, best of three).  Decode: ``batch`` requests with ``context`` cached tokens, replayed from the captured decode
step.  ``--kernels`` also times the step of either model with each of its kernel classes replaced by nothing: the
difference is that class's cost in place, and the two models' like classes stand side by side.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import ops
from ..config import FusolixConfig, NumuzenConfig
from .dodonex import build, time_decode, time_prefill
from .numuzen import numuzen_config

SIZES = {
    # width, dense ff, vocabulary, (heads, KV heads, key size, value size) of the attention, (heads, key, value) of the retention
    "2b": (2048, 8192, 32768, (16, 4, 128, 128), (16, 64, 128)),
    "1b": (1024, 4096, 32768, (16, 4, 64, 64), (8, 64, 128)),
}


def fusolix_config(size: str, layers: int, experts: int = 8, top: int = 2, window: int = 1024, pool: int = 64,
                   streams: int = 4, taps: int = 4) -> dict:
    """Every layer: the attention over ``window`` tokens and blocks of ``pool`` beside the retention; the feed-forward
    alternates between the dense unit and ``experts`` experts of which a token uses ``top``, each 1 / top as wide."""
    width, ff, vocab, (H, G, d, dv), (RH, RD, RV) = SIZES[size]
    left = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": d ** -0.5, "mask": {"size": window, "pool": pool}}
    right = {"heads": RH, "dim": RD, "vdim": RV, "decay": [1.0 - 2.0 ** -(5 + h % 6) for h in range(RH)],
             "rot": {"base": 1000000.0, "dims": RD}}
    mixer = {"left": left, "right": right, "left_scale": 0.8, "right_scale": 0.9}
    dense = {"kind": "dense", "ff": ff, "limit": 7.0}
    routed = {"kind": "moe", "expert": {"ff": ff // top},
              "router": {"experts": experts, "top": top, "groups": {"count": experts // 2, "keep": max(top, experts // 4)}}}
    out = [{"type": "parallel", "mixer": mixer, "mlp": routed if i % 2 else dense} for i in range(layers)]
    return {"architecture": "Fusolix", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "canon": {"taps": taps}, "layers": out}


KERNEL_CLASSES = {
    "attention over window and blocks (cache write, scores and values)": ("pooled_store", "pooled_attention", "pooled_attention_mma"),
    "retention (rotation, scan, finish)": ("rotate_heads_f32", "gla_scan", "gla_finish"),
    "streams (read and norm, convolution, write)": ("hyper_read_norm", "hyper_conv", "hyper_conv_state", "hyper_write"),
    "routing (route, plan, scatter, combine)": ("moe_route", "moe_plan", "moe_scatter", "moe_combine"),
    "expert products": ("gemm_tc_grouped", "moe_gemm_simt"),
    "branch sums (zero, scaled add)": ("fill_zero", "scaled_add"),
}


NUMUZEN_CLASSES = {
    "attention (norm, rotation, cache write, scores and values)": ("normed_qk_store", "attention_tc", "attention_mma", "attention_generic"),
    "gla (decay, scan, finish)": ("gla_decay", "gla_scan", "gla_finish"),
    "side stream (zero, norm behind the sub-layer)": ("fill_zero", "rms_scaled_add"),
    "routing (route, plan, scatter, combine)": ("moe_route", "moe_plan", "moe_scatter", "moe_combine"),
    "expert products": ("gemm_tc_grouped", "moe_gemm_simt"),
}


def in_place_costs(model, classes: dict, ms: float, us: float, prefill: int, batch: int, context: int, steps: int) -> dict:
    costs = {}
    for label, names in classes.items():
        saved = {n: getattr(ops, n) for n in names if hasattr(ops, n)}
        for n in saved:
            setattr(ops, n, lambda *a, **k: None)
        try:
            costs[label] = {"prefill_ms": round(ms - time_prefill(model, prefill), 3),
                            "decode_us": round(us - time_decode(model, batch, context, steps), 1)}
        finally:
            for n, fn in saved.items():
                setattr(ops, n, fn)
    return costs


def run(size: str = "2b", layers: int = 8, prefill: int = 2048, batch: int = 8, context: int = 2048, steps: int = 32,
        kernels: bool = False, experts: int = 8, top: int = 2, window: int = 1024, pool: int = 64, streams: int = 4,
        taps: int = 4) -> dict:
    record = {"workload": "fusolix", "size": size, "layers": layers, "prefill_tokens": prefill, "batch": batch,
              "context": context, "experts": experts, "top": top, "window": window, "pool": pool, "streams": streams,
              "taps": taps}
    models = (("fusolix", FusolixConfig.from_dict(fusolix_config(size, layers, experts, top, window, pool, streams, taps)),
               KERNEL_CLASSES),
              ("numuzen_equal_size", NumuzenConfig.from_dict(numuzen_config(size, layers, experts, top, window)),
               NUMUZEN_CLASSES))
    for name, config, classes in models:
        model = build(config, seed=9)
        ms = time_prefill(model, prefill)
        us = time_decode(model, batch, context, steps)
        record[name] = {"prefill_ms": round(ms, 3), "prefill_tok_s": round(prefill / ms * 1e3, 1),
                        "decode_us": round(us, 1), "decode_tok_s": round(batch / us * 1e6, 1)}
        if kernels:
            record[name]["in_place_costs"] = in_place_costs(model, classes, ms, us, prefill, batch, context, steps)
        del model
        torch.cuda.empty_cache()
    record["value"] = record["fusolix"]["decode_tok_s"]
    record["unit"] = "tok/s"
    record["metric"] = f"decode tokens per second, batch {batch}, context {context}"
    return record


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--size", choices=sorted(SIZES), default="2b")
    parser.add_argument("--layers", type=int, default=8)
    parser.add_argument("--prefill", type=int, default=2048)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--experts", type=int, default=8)
    parser.add_argument("--top", type=int, default=2)
    parser.add_argument("--window", type=int, default=1024)
    parser.add_argument("--pool", type=int, default=64)
    parser.add_argument("--streams", type=int, default=4)
    parser.add_argument("--taps", type=int, default=4)
    parser.add_argument("--kernels", action="store_true")
    parser.add_argument("--only", choices=["prefill", "decode"], default=None,
                        help="one step of the Fusolix model alone, untimed (for a launch list)")
    args = parser.parse_args(argv)
    if args.only:
        config = FusolixConfig.from_dict(fusolix_config(args.size, args.layers, args.experts, args.top, args.window,
                                                        args.pool, args.streams, args.taps))
        model = build(config, seed=9)
        if args.only == "prefill":
            print(json.dumps({"prefill_ms": time_prefill(model, args.prefill, repeats=1)}))
        else:
            print(json.dumps({"decode_us": time_decode(model, args.batch, args.context, 2, warmup=1)}))
        return 0
    print(json.dumps(run(args.size, args.layers, args.prefill, args.batch, args.context, args.steps, args.kernels,
                         args.experts, args.top, args.window, args.pool, args.streams, args.taps)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
