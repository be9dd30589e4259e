"""Several mixers side by side: all read the same input, the result is the weighted sum of theirs,
sum_i scale_i mixer_i(x).

Parameters: ``branches``: a list of {"mixer": PartSpec, "prefix": tensor prefix below this mixer's, "scale": float,
"norm": PartSpec or None, "norm_prefix": its tensors' prefix below this mixer's}.  A branch with a ``norm`` adds
scale * norm(its output), the norm taken over the model width in float32 (``Norm.add_normed``).
Each branch keeps what its own kind keeps; at most one branch may keep paged history (the execution has one page
group), any number may keep per-request state (the execution's state is a dict by branch prefix).  A branch whose
scale is 1 adds straight into the stream; any other adds into a zeroed float32 stream of its own, and the scaled
sum into the stream is one float32 operation, so no weight is rescaled and nothing is rounded twice.
"""
from __future__ import annotations

import dataclasses

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, NORMS, Mixer, TensorSpec, build_part


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        branches = spec.params["branches"]
        if not branches:
            raise ValueError("a parallel mixer needs at least one branch")
        self.branches = [(str(b["prefix"]), build_part(MIXERS, b["mixer"]), float(b.get("scale", 1.0))) for b in branches]
        # the norm behind a branch, by the branch's prefix: (part, its tensors' prefix below this mixer's)
        self.norms = {str(b["prefix"]): (build_part(NORMS, b["norm"]), str(b.get("norm_prefix", b["prefix"])))
                      for b in branches if b.get("norm") is not None}
        if len({prefix for prefix, _, _ in self.branches}) != len(self.branches):
            raise ValueError("the branches of a parallel mixer need different prefixes")
        if sum(1 for _, part, _ in self.branches if part.kv_spec() is not None) > 1:
            raise ValueError("at most one branch of a parallel mixer may keep paged history")
        self.graph_safe = all(getattr(part, "graph_safe", False) for _, part, _ in self.branches)

    def kv_spec(self):
        for _, part, _ in self.branches:
            if part.kv_spec() is not None:
                return part.kv_spec()
        return None

    def state_spec(self):
        specs = {prefix: part.state_spec() for prefix, part, _ in self.branches if part.state_spec() is not None}
        return specs or None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        out = []
        for branch in spec.params["branches"]:
            out += MIXERS.get(branch["mixer"].kind).expected_tensors(branch["mixer"], prefix + branch["prefix"])
            if branch.get("norm") is not None:
                out += NORMS.get(branch["norm"].kind).expected_tensors(
                    branch["norm"], prefix + branch.get("norm_prefix", branch["prefix"]))
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        for name, part, _ in self.branches:
            part.load(tensors, prefix + name, device, dtype)
        for norm, norm_prefix in self.norms.values():
            norm.load(tensors, prefix + norm_prefix, device, dtype)

    def forward(self, ctx, x, acc, cache) -> None:
        states = cache.state or {}
        for name, part, scale in self.branches:
            mine = dataclasses.replace(cache, state=states.get(name))
            norm = self.norms.get(name)
            if scale == 1.0 and norm is None:
                part.forward(ctx, x, acc, mine)
                continue
            side = ctx.buffer("parallel_mixers.side", tuple(acc.shape), torch.float32)
            if ctx.plans.get("parallel_mixers.side.clean") != side.data_ptr():  # the step's first scaled branch
                ops.fill_zero(side)
                ctx.plans["parallel_mixers.side.clean"] = side.data_ptr()
            part.forward(ctx, x, side, mine)
            if norm is not None:  # takes over the branch's unfinished last sum, if it left one
                norm[0].add_normed(ctx, side, acc, scale, clear=True)
                continue
            ctx.flush_pending()
            ops.scaled_add(acc, side, scale, clear=True)  # zeroed again for the next branch to add into
