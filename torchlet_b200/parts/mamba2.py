"""A selective state-space mixer in its state-space-duality form ("Mamba-2"): a recurrent mixer whose per-request
state is one N x V float32 matrix per head plus the last inputs of a short causal convolution.

With inner = heads * V and G groups of N state channels, the input product gives [z (inner) | x (inner) | B (G N) |
C (G N) | dt (heads)].  x, B and C pass a causal convolution over time per channel (``conv`` [channels, taps], the last
column is the current token's; bias ``conv.b``) and silu.  dt = softplus(dt + dt_bias).  Per head h (group
h // (heads / G)):

    S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T        y_t = S_t^T C_t + D_h x_t

y, the heads concatenated, is multiplied by silu(z), RMS-normed in ``norm_groups`` equal parts, multiplied by
``norm`` and projected by ``o``.  The input product has float32 output; convolution, step sizes, decays, state,
recurrence, gate and norm are float32 in both engines (csrc/ssm.cu; the scan is csrc/gla.cu's with one decay number a
token and head and q/k heads shared by a group).

Parameters: ``hidden_size``, ``num_heads``, ``v_dim``, ``state_size`` (N), ``groups``, ``conv_taps``, ``norm_groups``,
``eps``.  Tensors below the prefix: in [2 inner + 2 G N + heads, hidden]; conv [inner + 2 G N, taps]; conv.b; dt_bias,
A_log, D [heads]; norm [inner]; o [hidden, inner].
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, Mixer, StateSpec, TensorSpec
from .linear import Linear


@MIXERS.register("mamba2")
class Mamba2(Mixer):
    graph_safe = True  # nothing is planned on the host: requests and slots are read on the device

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.v_dim = int(p["v_dim"])
        self.state_size = int(p["state_size"])
        self.groups = int(p.get("groups", 1))
        self.taps = int(p["conv_taps"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.eps = float(p["eps"])
        self.inner = self.num_heads * self.v_dim
        self.gn = self.groups * self.state_size
        self.channels = self.inner + 2 * self.gn
        if self.groups < 1 or self.num_heads % self.groups:
            raise ValueError(f"{self.num_heads} heads cannot share {self.groups} groups of B and C")
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels cannot be normed in {self.norm_groups} equal parts")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"a convolution of {self.taps} taps is not supported (1 to 8)")
        if self.state_size > 256 or self.v_dim > 256 or self.num_heads > 256:
            raise ValueError(f"state {self.state_size} x {self.v_dim} with {self.num_heads} heads is not supported by the "
                             "scan kernel (up to 256 each)")
        self.in_proj: Linear | None = None
        self.o_proj: Linear | None = None
        self.conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm_weight = None

    def state_spec(self):
        specs = {"ssm": StateSpec((self.num_heads, self.state_size, self.v_dim), "float32")}
        if self.taps > 1:
            specs["conv"] = StateSpec((self.taps - 1, self.channels), "float32")
        return specs

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, H = int(p["hidden_size"]), int(p["num_heads"])
        inner, gn = H * int(p["v_dim"]), int(p.get("groups", 1)) * int(p["state_size"])
        channels = inner + 2 * gn
        return [TensorSpec(prefix + "in", (2 * inner + 2 * gn + H, hidden)),
                TensorSpec(prefix + "conv", (channels, int(p["conv_taps"]))),
                TensorSpec(prefix + "conv.b", (channels,), init="zeros"),
                TensorSpec(prefix + "dt_bias", (H,), init="zeros"), TensorSpec(prefix + "A_log", (H,), init="zeros"),
                TensorSpec(prefix + "D", (H,), init="ones"), TensorSpec(prefix + "norm", (inner,), init="ones"),
                TensorSpec(prefix + "o", (hidden, inner))]

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        self.in_proj = Linear(tensors[prefix + "in"], None, device, dtype)
        self.o_proj = Linear(tensors[prefix + "o"], None, device, dtype)
        f32 = lambda name: tensors[prefix + name].to(device=device, dtype=torch.float32).contiguous()
        self.conv, self.conv_bias = f32("conv"), f32("conv.b")
        self.dt_bias, self.a_log, self.skip, self.norm_weight = f32("dt_bias"), f32("A_log"), f32("D"), f32("norm")

    def forward(self, ctx, x, acc, cache) -> None:
        tokens, H, V, N = x.shape[0], self.num_heads, self.v_dim, self.state_size
        inner, gn = self.inner, self.gn
        proj = ctx.buffer("mamba2.proj", (tokens, 2 * inner + 2 * gn + H), torch.float32)
        self.in_proj.forward(x, proj)
        scan_in = ctx.buffer("mamba2.scan_in", (tokens, 2 * gn + inner), torch.float32)
        xs = ctx.buffer("mamba2.x", (tokens, inner), torch.float32)
        decay = ctx.buffer("mamba2.decay", (tokens, H), torch.float32)
        conv_state = cache.state.get("conv") if self.taps > 1 else None
        ops.ssm_conv(proj, inner, 2 * inner + 2 * gn, self.conv, self.conv_bias, self.dt_bias, self.a_log, conv_state,
                     ctx.token_req, ctx.req_indptr, ctx.slots, scan_in, xs, decay, H, V, gn,
                     update_state=ctx.decode_only and conv_state is not None)
        if conv_state is not None and not ctx.decode_only:
            ops.ssm_conv_state(proj, inner, conv_state, ctx.req_indptr, ctx.slots, ctx.num_requests)
        o = ctx.buffer("mamba2.o", (tokens, inner), torch.float32)
        ops.gla_scan(scan_in, decay, ctx.req_indptr, ctx.slots, cache.state["ssm"], o, ctx.num_requests, H, N, V, 1.0,
                     token_decay=True, qk_heads=self.groups)
        out = ctx.buffer("mamba2.out", (tokens, inner), ctx.dtype)
        ops.gated_norm(o, proj[:, :inner], self.norm_weight, out, self.norm_groups, self.eps, gate_first=True,
                       gate_act="silu", x=xs, skip=self.skip, vdim=V)
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
