"""Prefill and decode throughput of the Kilatar design at layer sizes that resemble a real model's, beside the
closest existing design of equal size: Fusolix (a softmax attention beside a linear attention with a constant decay
per head in every layer, dense and routed feed-forwards in turn; same width, layers, heads, span of the attention's mask
and vocabulary).

    python -m torchlet_b200.benchmarks.kilatar [--size 2b|1b] [--layers N] [--prefill 2048] [--batch 8]
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

from ..config import FusolixConfig, KilatarConfig
from .dodonex import build, time_decode, time_prefill
from .fusolix import KERNEL_CLASSES as FUSOLIX_CLASSES
from .fusolix import fusolix_config, in_place_costs

SIZES = {
    # width, dense ff, vocabulary, (heads, KV heads, key size, value size) of the chunked attention, (heads, key, value)
    # of the linear attention, (heads, unrotated, rotated, value, rank) of the latent attention, (heads, value size,
    # state, groups) of the state-space mixer
    "2b": (2048, 8192, 32768, (16, 4, 128, 128), (16, 64, 128), (16, 128, 64, 128, 512), (64, 64, 128, 1)),
    "1b": (1024, 4096, 32768, (16, 4, 64, 64), (8, 64, 128), (8, 64, 32, 64, 256), (32, 64, 128, 1)),
}


def kilatar_config(size: str, layers: int, experts: int = 8, top: int = 2, chunk: int = 1024, identity: int = 2,
                   taps: int = 4) -> dict:
    """The three kinds of layer in turn (state space, attention beside linear attention, latent attention); the
    feed-forward alternates between the dense unit and ``experts`` experts of which a token uses ``top``, each 1 / top as
    wide, with ``identity`` identity experts and a shared expert a quarter as wide as the dense unit."""
    width, ff, vocab, (H, G, d, dv), (RH, RD, RV), (LH, LD, LR, LV, rank), (MH, MV, MN, MG) = SIZES[size]
    pair = {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": d ** -0.5, "mask": {"size": chunk},
                     "rot": {"base": 500000.0, "dims": d // 2,
                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}},
            "right": {"heads": RH, "dim": RD, "vdim": RV, "decay": [1.0 - 2.0 ** -(5 + h % 6) for h in range(RH)]}}
    latent = {"heads": LH, "dim": LD, "rot_dim": LR, "vdim": LV, "kv_rank": rank, "scale": (LD + LR) ** -0.5,
              "rot": {"base": 10000.0, "dims": LR}}
    space = {"heads": MH, "vdim": MV, "state": MN, "groups": MG, "conv": taps, "norm_groups": 1}
    mixers = (("mamba2", space), ("parallel", pair), ("latent_attention", latent))
    dense = {"kind": "dense", "ff": ff}
    routed = {"kind": "moe", "expert": {"ff": ff // top}, "shared": {"ff": ff // 4},
              "router": {"experts": experts, "top": top, "identity": identity, "scale": 2.5}}
    out = [{"type": mixers[i % 3][0], "mixer": mixers[i % 3][1], "mlp": routed if i % 2 else dense} for i in range(layers)]
    return {"architecture": "Kilatar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": out}


KERNEL_CLASSES = {
    "chunked attention (norm-free projection, rotation, cache write, scores and values)":
        ("normed_qk_store", "attention_tc", "attention_mma", "attention_generic"),
    "linear attention (activation, scan, norm and gate)": ("activate_silu_", "gla_scan", "gated_norm"),
    "state space (convolution, step sizes, state rows)": ("ssm_conv", "ssm_conv_state"),
    "latent attention (prepare, absorb, scores and values, expand, gate)":
        ("latent_prepare", "latent_absorb_q", "latent_attention_mma", "latent_attention", "latent_expand_o", "gate_mul_"),
    "routing (route, plan, scatter, combine)": ("moe_route", "moe_plan", "moe_scatter", "moe_combine"),
    "expert products": ("gemm_tc_grouped", "moe_gemm_simt"),
    "dense and shared units' activation, token gate": ("glu_act", "token_gate"),
    "branch sums (zero, norm behind a branch, residual sum)": ("fill_zero", "rms_scaled_add", "rms_scaled_add_partials", "scaled_add"),
}


def run(size: str = "2b", layers: int = 8, prefill: int = 2048, batch: int = 8, context: int = 2048, steps: int = 32,
        kernels: bool = False, experts: int = 8, top: int = 2, chunk: int = 1024) -> dict:
    record = {"workload": "kilatar", "size": size, "layers": layers, "prefill_tokens": prefill, "batch": batch,
              "context": context, "experts": experts, "top": top, "chunk": chunk}
    models = (("kilatar", KilatarConfig.from_dict(kilatar_config(size, layers, experts, top, chunk)), KERNEL_CLASSES),
              ("fusolix_equal_size", FusolixConfig.from_dict(fusolix_config(size, layers, experts, top, chunk)), FUSOLIX_CLASSES))
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
    record["value"] = record["kilatar"]["decode_tok_s"]
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
    parser.add_argument("--chunk", type=int, default=1024)
    parser.add_argument("--kernels", action="store_true")
    parser.add_argument("--only", choices=["prefill", "decode"], default=None,
                        help="one step of the Kilatar model alone, untimed (for a launch list)")
    args = parser.parse_args(argv)
    if args.only:
        model = build(KilatarConfig.from_dict(kilatar_config(args.size, args.layers, args.experts, args.top, args.chunk)), seed=9)
        if args.only == "prefill":
            print(json.dumps({"prefill_ms": time_prefill(model, args.prefill, repeats=1)}))
        else:
            print(json.dumps({"decode_us": time_decode(model, args.batch, args.context, 2, warmup=1)}))
        return 0
    print(json.dumps(run(args.size, args.layers, args.prefill, args.batch, args.context, args.steps, args.kernels,
                         args.experts, args.top, args.chunk)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
