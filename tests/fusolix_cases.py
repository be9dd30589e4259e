"""Small Fusolix configurations of the tests, their random weights, and an engine around them.  No two agree in
any size: one stream and several, two to five taps, key and value sizes that differ and are no multiple of 32,
one head and several, one KV head and as many as query heads, a window of one token, of less than a page and of
several pages, blocks of one token, of a few and of more tokens than the window, a rotation over all entries and
over a few, a branch scale of one, one expert of one, every expert of three, groups of one expert, one group, a
layer without a feed-forward, either kind of feed-forward first."""
from __future__ import annotations

import copy
import functools

import torch

import plain_fusolix

# Largest allowed |engine - plain| of a position's logits as a fraction of that position's largest |logit|.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}


def left(heads, kv_heads, dim, vdim, scale, size, pool):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": size, "pool": pool}}


def right(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"base": base, "dims": rot_dims}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, count, keep):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(left_mixer, right_mixer, mlp, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left_mixer, "right": right_mixer, "left_scale": left_scale, "right_scale": right_scale}}


CASES = {
    # three streams, four taps; windows shorter than a page and of several; blocks of 5, 3 and (longer than its
    # window) 16 tokens; a rotation over a few entries; groups of two of which two of three are kept
    "P": {"architecture": "Fusolix", "vocab": 101, "width": 96, "streams": 3, "norm": {"eps": 1e-5},
          "embedding": {"scale": 1.7}, "canon": {"taps": 4},
          "layers": [
              layer(left(4, 2, 24, 16, 0.3, 13, 5), right(3, 12, 20, (0.9, 0.97, 0.99), 8, 500.0), dense(40, 1.0), 0.6, 1.3),
              layer(left(4, 2, 24, 16, 0.3, 37, 3), right(2, 24, 8, (0.95, 0.999), 6, 500.0), moe(6, 2, 24, 3, 2), 1.2, 0.7),
              layer(left(2, 1, 12, 40, 0.4, 7, 16), right(3, 12, 20, (0.5, 0.97, 1.0), 12, 500.0), None, 0.6, 1.3),
              layer(left(6, 3, 8, 8, 0.5, 20, 4), right(1, 40, 8, (0.98,), 8, 500.0), moe(4, 1, 56, 1, 1), 1.0, 0.5),
          ]},
    # one stream, two taps, one head, a window of ONE token, blocks of ONE token, full rotation, as many KV heads as
    # heads, every expert of three, one expert of one, groups of one expert, a branch scale of one, no embedding scale
    "Q": {"architecture": "Fusolix", "vocab": 67, "width": 64, "streams": 1, "norm": {"eps": 1e-6},
          "embedding": {"scale": 1.0}, "canon": {"taps": 2},
          "layers": [
              layer(left(1, 1, 40, 8, 0.2, 1, 1), right(1, 16, 24, (0.9,), 16, 100.0), moe(1, 1, 24, 1, 1), 1.0, 1.0),
              layer(left(2, 2, 16, 20, 0.25, 9, 2), right(5, 8, 16, (0.8, 0.9, 0.95, 0.99, 0.999), 2, 100.0),
                    moe(3, 3, 24, 3, 3), 1.0, 0.8),
              layer(left(3, 1, 20, 12, 0.2, 30, 30), right(2, 20, 12, (0.97, 0.99), 20, 100.0), dense(72, 0.7), 0.9, 1.0),
          ]},
    # head sizes of 64 and 128 (equal key and value sizes of these run on the tensor-core kernels: the first and the
    # last layer), windows and blocks over several pages, five taps
    "R": {"architecture": "Fusolix", "vocab": 211, "width": 128, "streams": 4, "norm": {"eps": 1e-6},
          "embedding": {"scale": 0.25}, "canon": {"taps": 5},
          "layers": [
              layer(left(4, 1, 64, 64, 0.125, 150, 16), right(2, 64, 64, (0.99, 0.995), 32, 50000.0),
                    moe(8, 2, 64, 4, 2), 0.7, 1.1),
              layer(left(6, 2, 128, 64, 0.09, 70, 24), right(1, 128, 32, (0.98,), 64, 50000.0), dense(192, 2.5), 1.1, 0.9),
              layer(left(2, 2, 64, 128, 0.125, 33, 8), right(4, 32, 64, (0.9, 0.95, 0.99, 0.999), 32, 50000.0),
                    moe(4, 2, 64, 2, 1), 0.8, 0.8),
              layer(left(8, 2, 128, 128, 0.09, 40, 8), right(2, 32, 32, (0.95, 0.99), 16, 50000.0), None, 0.9, 1.2),
          ]},
    # ONE tap (the convolution is a factor on the token itself and keeps nothing), two streams, one expert of two groups
    "S": {"architecture": "Fusolix", "vocab": 53, "width": 48, "streams": 2, "norm": {"eps": 1e-5},
          "embedding": {"scale": 2.0}, "canon": {"taps": 1},
          "layers": [
              layer(left(2, 1, 16, 24, 0.25, 11, 6), right(2, 8, 12, (0.9, 0.99), 4, 1000.0), moe(4, 1, 32, 2, 2), 0.5, 1.5),
              layer(left(3, 3, 8, 16, 0.35, 5, 2), right(1, 24, 16, (0.97,), 24, 1000.0), dense(64, 2.0), 1.5, 0.5),
          ]},
    # no convolution at all
    "T": {"architecture": "Fusolix", "vocab": 53, "width": 48, "streams": 2, "norm": {"eps": 1e-5},
          "embedding": {"scale": 2.0},
          "layers": [
              layer(left(2, 1, 16, 24, 0.25, 11, 6), right(2, 8, 12, (0.9, 0.99), 4, 1000.0), dense(64, 2.0), 0.5, 1.5),
              layer(left(3, 3, 8, 16, 0.35, 5, 2), right(1, 24, 16, (0.97,), 24, 1000.0), None, 1.5, 0.5),
          ]},
}


def _all_experts(case: dict) -> dict:
    case = copy.deepcopy(case)
    for entry in case["layers"]:
        if entry["mlp"] is not None and entry["mlp"]["kind"] == "moe":
            router = entry["mlp"]["router"]
            router["top"] = router["experts"]
            router["groups"]["keep"] = router["groups"]["count"]
    return case


# "Pa", "Qa", "Ra": the same models with EVERY expert chosen.  Random routers have close calls: where two experts'
# or two groups' scores lie within bfloat16 rounding of one another the bfloat16 engine may choose the other one, and
# that position, and through states and keys all behind it, then differs by a whole expert's output.  So the bfloat16
# engine is compared on these (same tensors, no discrete choice), the float32 engine on the true routing at every
# position, and the choice itself is tested on given inputs in test_fusolix_parts_gpu.py.
CASES.update({name + "a": _all_experts(case) for name, case in list(CASES.items())})


def variant(name: str, dtype: str) -> str:
    return name if dtype == "float32" else name + "a"


def config_for(name: str):
    from torchlet_b200.config import FusolixConfig

    return FusolixConfig.from_dict(CASES[name])


@functools.lru_cache(maxsize=None)
def weights_for(name: str, seed: int = 0):
    """bfloat16-rounded random weights as float32 tensors by name (so that both engines and the plain implementation
    hold the same numbers).  Routers are drawn wider, so that the experts' scores lie apart; the streams' vectors and
    matrices, the convolutions and the biases are drawn away from one, the identity and zero, so that each counts."""
    from torchlet_b200.weights import random_tensors

    tensors = random_tensors(config_for(name), seed=500 + seed, std=0.1, norm_std=0.1, dtype="bfloat16")
    g = torch.Generator().manual_seed(900 + seed)
    out = {}
    for k, v in tensors.items():
        v = v.float()
        if k.endswith(".router"):
            v = v * 4
        elif ".hc" in k:
            v = v + 0.3 * torch.randn(v.shape, generator=g)
        elif ".canon" in k:
            v = 0.4 * torch.randn(v.shape, generator=g)
        elif k.endswith(".b"):
            v = 0.2 * torch.randn(v.shape, generator=g)
        out[k] = v.to(torch.bfloat16).float()
    return out


def make_ids(name: str, length: int, seed: int):
    g = torch.Generator().manual_seed(4000 + seed)
    return torch.randint(0, CASES[name]["vocab"], (length,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int):
    ids = make_ids(name, length, seed)
    return ids, plain_fusolix.forward(CASES[name], weights_for(name), ids).float()


def make_model(name: str, dtype: str, weights=None):
    from torchlet_b200.engine.loading import build_model

    w = weights if weights is not None else weights_for(name)
    return build_model(config_for(name), {k: v.to(torch.bfloat16) for k, v in w.items()}, dtype)


def make_runner(name: str, dtype: str, num_pages: int = 64, slots: int = 4, page_size: int = 16, budget: int = 512,
                max_seq_len: int = 512, cuda_graph: bool = False, weights=None):
    from torchlet_b200.config import EngineConfig
    from torchlet_b200.engine import ModelRunner

    engine = EngineConfig(dtype=dtype, max_decode_slots=slots, kv_block_size=page_size, max_num_blocks=num_pages,
                          max_seq_len=max_seq_len, max_num_batched_tokens=budget, cuda_graph=cuda_graph)
    return ModelRunner(make_model(name, dtype, weights), engine)


def replay(runner, rid, ids, cuts, finish=True):
    """Feed ``ids`` of one request in portions of the given sizes, asking for every position's logits; returns
    [len(ids), vocab] on the CPU."""
    from torchlet_b200.engine import StepEntry

    assert sum(cuts) == len(ids)
    runner.admit(rid)
    out, start = [], 0
    for size in cuts:
        logits = runner.step([StepEntry(rid, ids[start:start + size], list(range(size)))])
        out.append(logits.cpu().clone())
        start += size
    if finish:
        runner.finish(rid)
        runner.cache.check()
    return torch.cat(out)


def assert_close(got, want, dtype: str, what: str = ""):
    assert got.shape == want.shape, f"{what}: shapes {tuple(got.shape)} and {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    got, want = got.reshape(-1, got.shape[-1]).double(), want.reshape(-1, want.shape[-1]).double()
    err = (got - want).abs().amax(dim=1)
    scale = want.abs().amax(dim=1)
    ratio = err / scale
    worst = int(ratio.argmax())
    if dtype == "bfloat16":
        # A retention head's output is divided by its root mean square, so it counts by its direction alone.  At the
        # first positions the state has rank one or two and a head's output is its first value vector times the
        # scalar k . q: where that scalar is within bfloat16 rounding of zero, its sign, and with it the whole head's
        # output, is a coin's toss.  Random weights have such positions; the float32 engine is held to its tolerance
        # at EVERY position of the same tests, the bfloat16 engine at nine in ten, and nowhere may it be off by more
        # than half of the largest logit.
        over = int((ratio > TOLERANCE[dtype]).sum())
        assert over <= max(1, ratio.numel() // 10) and ratio[worst] <= 0.5, (
            f"{what}: {over} of {ratio.numel()} rows over {TOLERANCE[dtype]:.1e}; worst row {worst}: {ratio[worst]:.3e}")
        return
    assert ratio[worst] <= TOLERANCE[dtype], (
        f"{what}: row {worst}: max |diff| {err[worst]:.3e} > {TOLERANCE[dtype]:.1e} * {scale[worst]:.3f}")
