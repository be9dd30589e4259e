"""Retention: linear attention with a FIXED decay per head and no softmax or denominator; a recurrent mixer with
one D x V float32 state matrix per head and request, kept in the request's slot between steps.

q = W_q x, k = W_k x (heads x D), v = W_v x (heads x V); q and k are rotated by position (``positions``: a
``rotary_partial`` part, or None), k is multiplied by ``k_scale`` (default D^(-1/2)) after the rotation; per head

    S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

Each head's o is divided by its root mean square (no weight), the heads, concatenated, are multiplied by
silu(W_g x) and go through W_o into the stream.  The four input products run as ONE product with float32 output;
rotation, state and recurrence are float32 in both engines.  The scan is the gated-linear-attention scan with a
constant decay (csrc/gla.cu); the factor ``k_scale`` is applied to o instead of k, which is the same number.

Options (the "lightning" form of linear attention sets all three): ``activation`` "silu": q, k and v are
silu(W x) (None: as projected); ``norm`` "whole": the concatenated heads are RMS-normed together and multiplied by the
weight ``norm`` [H V] ("head", the default: each head by its own root mean square, no weight); ``gate`` "sigmoid": the
normed row is multiplied by sigmoid(W_g x) ("silu", the default).

Parameters: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_dim``, ``decay`` (one number a head), ``eps``,
``positions``, ``k_scale``, ``activation``, ``norm``, ``gate``.  Tensors below the prefix: q, k [H D, hidden]; v, g
[H V, hidden]; o [hidden, H V]; with ``norm`` "whole" also norm [H V].
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, POSITIONS, Mixer, StateSpec, TensorSpec, build_part
from .linear import Linear


@MIXERS.register("retention")
class Retention(Mixer):
    graph_safe = True  # nothing is planned on the host: requests and slots are read on the device

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p["v_dim"])
        self.decay_values = [float(a) for a in p["decay"]]
        self.eps = float(p["eps"])
        self.k_scale = float(p["k_scale"]) if p.get("k_scale") is not None else self.head_dim ** -0.5
        self.activation, self.norm, self.gate = p.get("activation"), p.get("norm", "head"), p.get("gate", "silu")
        if self.activation not in (None, "silu") or self.norm not in ("head", "whole") or self.gate not in ("silu", "sigmoid"):
            raise ValueError(f"unknown option: activation {self.activation!r} (silu, None), norm {self.norm!r} (head, whole), "
                             f"gate {self.gate!r} (silu, sigmoid)")
        if self.norm == "head" and self.gate != "silu":
            raise ValueError("the per-head norm is built with the silu gate only")
        if len(self.decay_values) != self.num_heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.num_heads} heads")
        if self.head_dim > 256 or self.v_dim > 256:
            raise ValueError(f"head sizes {self.head_dim} x {self.v_dim} are not supported by the scan kernel (up to 256)")
        self.positions = build_part(POSITIONS, p["positions"]) if p.get("positions") else None
        if self.positions is not None and not hasattr(self.positions, "inv_freq"):
            raise ValueError("this mixer rotates with its own kernel and needs a position part with a frequency table")
        if self.positions is not None and getattr(self.positions, "scaling", None):
            raise ValueError("frequency scaling is not built for this mixer")
        self.k_size = self.num_heads * self.head_dim
        self.v_size = self.num_heads * self.v_dim
        self.in_proj: Linear | None = None
        self.o_proj: Linear | None = None
        self.decay = self.norm_weight = None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_heads, self.head_dim, self.v_dim), "float32")

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden = int(p["hidden_size"])
        k_size, v_size = int(p["num_heads"]) * int(p["head_dim"]), int(p["num_heads"]) * int(p["v_dim"])
        out = [TensorSpec(prefix + "q", (k_size, hidden)), TensorSpec(prefix + "k", (k_size, hidden)),
               TensorSpec(prefix + "v", (v_size, hidden)), TensorSpec(prefix + "g", (v_size, hidden)),
               TensorSpec(prefix + "o", (hidden, v_size))]
        if p.get("norm", "head") == "whole":
            out.append(TensorSpec(prefix + "norm", (v_size,), init="ones"))
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        fused = torch.cat([tensors[prefix + name] for name in ("q", "k", "v", "g")], dim=0)
        self.in_proj = Linear(fused, None, device, dtype)
        self.o_proj = Linear(tensors[prefix + "o"], None, device, dtype)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)
        if self.positions is not None:
            self.positions.load(tensors, prefix, device, dtype)
        if self.norm == "whole":
            self.norm_weight = tensors[prefix + "norm"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, ctx, x, acc, cache) -> None:
        tokens, H, D, V = x.shape[0], self.num_heads, self.head_dim, self.v_dim
        proj = ctx.buffer("retention.proj", (tokens, 2 * self.k_size + 2 * self.v_size), torch.float32)
        self.in_proj.forward(x, proj)
        if self.activation == "silu":  # q, k and v: the first columns of the rows
            ops.activate_silu_(proj, 2 * self.k_size + self.v_size)
        if self.positions is not None:  # q and k are 2 H consecutive heads of D entries
            ops.rotate_heads_f32(proj, ctx.positions, self.positions.inv_freq, 2 * H, D, self.positions.dims)
        o = ctx.buffer("retention.o", (tokens, self.v_size), torch.float32)
        ops.gla_scan(proj, self.decay, ctx.req_indptr, ctx.slots, cache.state, o, ctx.num_requests, H, D, V, self.k_scale,
                     fixed_decay=True)
        out = ctx.buffer("retention.out", (tokens, self.v_size), ctx.dtype)
        if self.norm == "whole":
            ops.gated_norm(o, proj[:, 2 * self.k_size + self.v_size:], self.norm_weight, out, 1, self.eps, gate_first=False,
                           gate_act=self.gate)
        else:
            ops.gla_finish(o, proj, 2 * self.k_size + self.v_size, None, out, H, V, self.eps)
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
