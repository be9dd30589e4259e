"""A gated feed-forward with a choice of activation, optional biases and an optional gate of one number a token:

    y = W_down (act(W_gate x + b_gate) * (W_up x + b_up)) + b_down,        act = silu or the tanh form of gelu

With ``token_gate`` (the name of a [1, hidden] tensor below the prefix) the output is multiplied by
sigmoid(w_gate . x), one float32 number a token (an always-on expert beside routed ones); it is applied to the
activated rows before the down product, which is the same number.

In bfloat16 the gate and up products are ONE tcgen05 product over 16-interleaved rows with the biases, the activation
and the token's gate in its epilogue (``ops.gemm_tc_gated``); in float32, and at sizes that kernel does not take, one
product over [gate; up] and an activation kernel.

Parameters: ``hidden_size``, ``intermediate_size``, ``activation`` ("silu", "gelu_tanh"), ``bias`` (default False),
``token_gate`` (default None), and the tensors' names below the prefix: ``gate_name``, ``up_name``, ``down_name``
(defaults "gate", "up", "down"; a bias is the matrix's name + ``bias_suffix``, default ".b").
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import FEED_FORWARDS, FeedForward, TensorSpec
from .linear import Linear


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        self.activation = p.get("activation", "silu")
        self.bias = bool(p.get("bias", False))
        self.token_gate = p.get("token_gate")
        if self.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r} (known: {', '.join(ops.GLU_ACTIVATIONS)})")
        if self.bias and self.token_gate:
            raise ValueError("a gate of one number a token is not built together with biases")
        self.gate_up_proj: Linear | None = None
        self.gate_up_interleaved = None  # bfloat16 fused path: gate/up rows interleaved by 16
        self.gate_up_bias = None  # ... and their biases in the same order
        self.down_proj: Linear | None = None
        self.token_gate_weight = None

    @classmethod
    def _names(cls, spec: PartSpec, prefix: str):
        p = spec.params
        return tuple(prefix + p.get(key, default) for key, default in (("gate_name", "gate"), ("up_name", "up"), ("down_name", "down")))

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        gate, up, down = cls._names(spec, prefix)
        out = [TensorSpec(gate, (inter, hidden)), TensorSpec(up, (inter, hidden)), TensorSpec(down, (hidden, inter))]
        if p.get("bias", False):
            suffix = p.get("bias_suffix", ".b")
            out += [TensorSpec(gate + suffix, (inter,), init="zeros"), TensorSpec(up + suffix, (inter,), init="zeros"),
                    TensorSpec(down + suffix, (hidden,), init="zeros")]
        if p.get("token_gate"):
            out.append(TensorSpec(prefix + p["token_gate"], (1, hidden)))
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        from . import swiglu_bf16

        gate, up, down = self._names(self.spec, prefix)
        suffix = self.spec.params.get("bias_suffix", ".b")
        fused = dtype == torch.bfloat16 and swiglu_bf16.usable(self.hidden_size, self.intermediate_size)
        if fused:
            self.gate_up_interleaved = swiglu_bf16.interleave(
                tensors[gate].to(device=device, dtype=dtype), tensors[up].to(device=device, dtype=dtype))
            if self.bias:  # interleaved by 16 like the rows they belong to
                both = [tensors[name + suffix].to(device=device, dtype=torch.float32).view(-1, swiglu_bf16.BLOCK) for name in (gate, up)]
                self.gate_up_bias = torch.cat(both, dim=1).reshape(-1).contiguous()
        else:
            bias = torch.cat([tensors[gate + suffix].float(), tensors[up + suffix].float()]) if self.bias else None
            self.gate_up_proj = Linear(torch.cat([tensors[gate], tensors[up]], dim=0), bias, device, dtype)
        self.down_proj = Linear(tensors[down], tensors[down + suffix] if self.bias else None, device, dtype)
        if self.token_gate:
            self.token_gate_weight = tensors[prefix + self.token_gate].to(device=device, dtype=torch.float32).reshape(-1).contiguous()

    def forward(self, ctx, x, acc, row_scale=None) -> None:
        """``row_scale``: the token gate's numbers (float32 [tokens]) where the caller has computed them already (a router
        whose kernel takes ``token_gate_weight`` along)."""
        tokens = x.shape[0]
        if self.token_gate_weight is not None and row_scale is None:
            row_scale = ctx.buffer("gated_mlp.token_gate", (tokens,), torch.float32)
            ops.token_gate(x, self.token_gate_weight, row_scale)
        act = ctx.buffer("gated_mlp.act", (tokens, self.intermediate_size), ctx.dtype)
        if self.gate_up_interleaved is not None:
            ops.gemm_tc_gated(x, self.gate_up_interleaved, act, self.activation, self.gate_up_bias, row_scale)
        else:
            gate_up = ctx.buffer("gated_mlp.gate_up", (tokens, 2 * self.intermediate_size), ctx.dtype)
            self.gate_up_proj.forward(x, gate_up)
            ops.glu_act(gate_up, act, self.activation, row_scale)
        if not self.down_proj.accumulate_later(ctx, act, acc):
            self.down_proj.forward(act, acc, accumulate=True)
