"""Small Kilatar configurations of the tests, their random weights, and an engine around them.  No two agree in any
size: key and value sizes that differ and are no multiple of 8, one head and several, one key/value head and as many as
query heads, chunks of one token, of less than a page and of several pages, a rotation over all entries, over a few and
none, frequencies slowed down or not, state-space mixers with one group and several, one tap to four, one norm group
and several, routers with and without identity experts and a shared expert, one expert of two router outputs, every
expert of three, a layer without a feed-forward, a looped stretch at the start, in the middle, and no loop."""
from __future__ import annotations

import copy
import functools

import torch

import plain_kilatar

# Largest allowed |engine - plain| of a position's logits as a fraction of that position's largest |logit|.
TOLERANCE = {"float32": 1e-4, "bfloat16": 6e-2}


def rot(base, dims, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        factor, low, high, original = scaling
        out["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return out


def chunked(heads, kv_heads, dim, vdim, scale, size, rotation):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if rotation is not None:
        out["rot"] = rotation
    return out


def lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def parallel(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, rotation, mlp):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": rotation}}


def mamba(heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                      "norm_groups": norm_groups}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, scale=1.0, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity, "scale": scale}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


CASES = {
    # a looped stretch in the middle, three times; chunks of 13 and 5 tokens (less than a page, no power of two); a
    # rotation over 8 of 24 entries with slowed frequencies; two groups of B and C, two norm groups, four taps
    "P": {"architecture": "Kilatar", "vocab": 101, "width": 96, "norm": {"eps": 1e-5},
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [
              parallel(chunked(4, 2, 24, 16, 0.3, 13, rot(500.0, 8, (8.0, 1.0, 4.0, 64))),
                       lightning(3, 12, 20, (0.9, 0.97, 0.99)), moe(6, 2, 24, identity=2, scale=1.7, shared=40)),
              mamba(4, 12, 20, 2, 4, 2, dense(40)),
              latent(3, 20, 12, 28, 40, 0.2, rot(1000.0, 8), moe(5, 3, 24)),
              parallel(chunked(6, 3, 8, 12, 0.5, 5, rot(100.0, 8)), lightning(2, 24, 8, (0.5, 1.0)), None),
              mamba(2, 24, 8, 1, 2, 1, None),
          ]},
    # ones: one head everywhere, a chunk of ONE token, one tap, one expert beside one identity expert of which one is
    # chosen, every expert of three, no rotation in the attention, the loop at the very start, twice
    "Q": {"architecture": "Kilatar", "vocab": 67, "width": 64, "norm": {"eps": 1e-6},
          "loop": {"start": 0, "stop": 2, "times": 2},
          "layers": [
              latent(1, 8, 4, 8, 16, 0.35, rot(10000.0, 4), moe(1, 1, 24, identity=1, scale=2.0, shared=16)),
              parallel(chunked(1, 1, 40, 8, 0.2, 1, None), lightning(1, 16, 24, (0.9,)), moe(3, 3, 24)),
              mamba(1, 8, 4, 1, 1, 1, dense(72)),
          ]},
    # sizes the tensor-core kernels take: attention heads of 64 and 128 with chunks over several pages, a latent row of
    # 96 entries, experts of 64; no loop
    "R": {"architecture": "Kilatar", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
          "layers": [
              parallel(chunked(4, 1, 64, 64, 0.125, 48, rot(50000.0, 32, (4.0, 1.0, 2.0, 32))),
                       lightning(2, 64, 64, (0.99, 0.995)), moe(8, 2, 64, identity=2, scale=1.5, shared=64)),
              latent(4, 32, 32, 32, 64, 0.125, rot(20000.0, 32), dense(192)),
              parallel(chunked(4, 2, 128, 128, 0.09, 150, rot(50000.0, 128)), lightning(1, 128, 32, (0.98,)), moe(4, 2, 64)),
              mamba(4, 32, 64, 2, 4, 4, None),
          ]},
    # sizes that are no multiple of 8 (the products' and the attention's any-size kernels in both engines), a chunk longer
    # than every test sequence, five taps, three norm groups, three of four router outputs of which two are identity
    "S": {"architecture": "Kilatar", "vocab": 53, "width": 100, "norm": {"eps": 1e-5},
          "loop": {"start": 2, "stop": 3, "times": 2},
          "layers": [
              mamba(3, 10, 6, 3, 5, 3, moe(2, 3, 20, identity=2, scale=0.8, shared=12)),
              latent(2, 12, 6, 10, 20, 0.25, rot(300.0, 6), dense(36)),
              parallel(chunked(5, 5, 12, 12, 0.3, 1000, rot(300.0, 4, (2.0, 1.0, 3.0, 16))),
                       lightning(2, 10, 14, (0.8, 0.95)), dense(28)),
          ]},
}


def _all_experts(case: dict) -> dict:
    case = copy.deepcopy(case)
    for entry in case["layers"]:
        if entry["mlp"] is not None and entry["mlp"]["kind"] == "moe":
            router = entry["mlp"]["router"]
            router["top"] = router["experts"] + router.get("identity", 0)
    return case


# "Pa", "Qa", "Ra": the same models with EVERY expert chosen.  Random routers have close calls: where two experts'
# scores lie within bfloat16 rounding of one another the bfloat16 engine may choose the other one, and that position,
# and through states and keys all behind it, then differs by a whole expert's output.  So the bfloat16 engine is
# compared on these (same tensors, no discrete choice), the float32 engine on the true routing at every position, and
# the choice itself is tested on given inputs in test_kilatar_parts_gpu.py.
CASES.update({name + "a": _all_experts(case) for name, case in list(CASES.items())})


def variant(name: str, dtype: str) -> str:
    return name if dtype == "float32" else name + "a"


def config_for(name: str):
    from torchlet_b200.config import KilatarConfig

    return KilatarConfig.from_dict(CASES[name])


@functools.lru_cache(maxsize=None)
def weights_for(name: str, seed: int = 0):
    """bfloat16-rounded random weights as float32 tensors by name (so that both engines and the plain implementation
    hold the same numbers).  Routers are drawn wider, so that the experts' scores lie apart; corrections, biases,
    convolutions, step-size biases, rates and skips are drawn away from zero and one, so that each counts."""
    from torchlet_b200.weights import random_tensors

    tensors = random_tensors(config_for(name), seed=700 + seed, std=0.1, norm_std=0.1, dtype="bfloat16")
    g = torch.Generator().manual_seed(1100 + seed)
    out = {}
    for k, v in tensors.items():
        v = v.float()
        noise = torch.randn(v.shape, generator=g)
        if k.endswith(".router"):
            v = v * 4
        elif k.endswith(".correction"):
            v = 0.2 * noise
        elif k.endswith(".conv"):
            v = 0.4 * noise
        elif k.endswith(".b") or k.endswith(".dt_bias"):
            v = 0.3 * noise
        elif k.endswith(".A_log"):
            v = 0.7 * noise
        elif k.endswith(".D"):
            v = 1.0 + 0.5 * noise
        elif k.endswith(".sg"):
            v = v * 3
        out[k] = v.to(torch.bfloat16).float()
    return out


def make_ids(name: str, length: int, seed: int):
    g = torch.Generator().manual_seed(6000 + seed)
    return torch.randint(0, CASES[name]["vocab"], (length,), generator=g).tolist()


def _double(w: dict) -> dict:
    return {k: v.double() for k, v in w.items()}


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int):
    ids = make_ids(name, length, seed)
    return ids, plain_kilatar.forward(CASES[name], _double(weights_for(name)), ids).float()


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
        # Behind a norm a branch's output counts by its direction alone.  At the first positions a linear attention's
        # state has rank one or two and a head's output is its first value vector times the scalar k . q: where that
        # scalar is within bfloat16 rounding of zero its sign is a coin's toss.  Random weights have such positions; the
        # float32 engine is held to its tolerance at EVERY position of the same tests, the bfloat16 engine at nine in
        # ten, and nowhere may it be off by more than half of the largest logit.
        over = int((ratio > TOLERANCE[dtype]).sum())
        assert over <= max(1, ratio.numel() // 10) and ratio[worst] <= 0.5, (
            f"{what}: {over} of {ratio.numel()} rows over {TOLERANCE[dtype]:.1e}; worst row {worst}: {ratio[worst]:.3e}")
        return
    assert ratio[worst] <= TOLERANCE[dtype], (
        f"{what}: row {worst}: max |diff| {err[worst]:.3e} > {TOLERANCE[dtype]:.1e} * {scale[worst]:.3f}")
