"""Grouped-query softmax attention over a sliding window of tokens plus pooled blocks of older ones.

q = W_q x + b_q (heads x dim), k = W_k x + b_k (kv_heads x dim), v = W_v x + b_v (kv_heads x v_dim); no position
encoding.  The query at position i sees the tokens j with 0 <= i - j < ``window`` and, beside them, ONE key and
value for every block of ``pool`` consecutive tokens (block b: positions b pool .. b pool + pool - 1) that lies wholly
before its window (b pool + pool - 1 <= i - window): the mean of the block's cached keys and the mean of its values.
Tokens that have left the window while their block is not yet complete and passed are not seen.  Tokens and blocks
share one softmax of (q . k) * ``scale``; query head h reads KV head h // (heads / kv_heads); the heads,
concatenated, go through W_o (+ b_o) into the stream.

What the mixer keeps: a token's key and value per KV head in pages (one joined row [key | value]; a key plane and a
value plane where the two are equally wide and the tensor-core kernels take the size), held while the token is inside
the window or its block is incomplete (a windowed page group of max(window, pool) tokens), and the pooled rows,
float32, in the request's slot: one a block, written by the step that brings the block's last token
(csrc/pooled_attention.cu).

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_dim``, ``scale``, ``window``, ``pool``,
``bias`` (default True: q, k, v and o have biases).  Tensors below the prefix: q [H D, hidden], k [G D, hidden],
v [G V, hidden], o [hidden, H V], and ``<name>.b`` for the biases.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, KVSpec, Mixer, StateSpec, TensorSpec
from .linear import Linear


@MIXERS.register("pooled_window_attention")
class PooledWindowAttention(Mixer):
    graph_safe = True  # nothing is planned on the host

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.v_dim = int(p.get("v_dim", self.head_dim))
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.head_dim ** -0.5
        self.window = int(p["window"])
        self.pool = int(p["pool"])
        self.bias = bool(p.get("bias", True))
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if self.window <= 0 or self.pool <= 0:
            raise ValueError("window and pool must be positive")
        if self.head_dim > 256 or self.v_dim > 256:
            raise ValueError(f"head sizes {self.head_dim} x {self.v_dim} are not supported (up to 256)")
        self.q_size = self.num_heads * self.head_dim
        self.k_size = self.num_kv_heads * self.head_dim
        self.v_size = self.num_kv_heads * self.v_dim
        self.out_size = self.num_heads * self.v_dim
        self.in_proj: Linear | None = None
        self.o_proj: Linear | None = None

    def kv_spec(self) -> KVSpec:
        # a token's row is needed while it is in the window, and until the token that completes its block has come
        from .pooled_attention_bf16 import split_planes

        if split_planes(self.head_dim, self.v_dim):
            return KVSpec(self.num_kv_heads, self.head_dim, max(self.window, self.pool), planes=2)
        return KVSpec(self.num_kv_heads, self.head_dim + self.v_dim, max(self.window, self.pool), planes=1)

    def state_spec(self) -> StateSpec:
        return StateSpec((self.num_kv_heads, self.head_dim + self.v_dim), "float32", per_tokens=self.pool)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, d = int(p["hidden_size"]), int(p["head_dim"])
        dv = int(p.get("v_dim", d))
        H, G = int(p["num_heads"]), int(p["num_kv_heads"])
        out = []
        for name, shape in (("q", (H * d, hidden)), ("k", (G * d, hidden)), ("v", (G * dv, hidden)), ("o", (hidden, H * dv))):
            out.append(TensorSpec(prefix + name, shape))
            if p.get("bias", True):
                out.append(TensorSpec(prefix + name + ".b", (shape[0],)))
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        names = ("q", "k", "v")
        weight = torch.cat([tensors[prefix + n] for n in names], dim=0)
        bias = torch.cat([tensors[prefix + n + ".b"].float() for n in names], dim=0) if self.bias else None
        self.in_proj = Linear(weight, bias, device, dtype)
        self.o_proj = Linear(tensors[prefix + "o"], tensors[prefix + "o.b"] if self.bias else None, device, dtype)

    def forward(self, ctx, x, acc, cache) -> None:
        tokens = x.shape[0]
        H, G, d, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim
        qkv = ctx.buffer("pooled_attention.qkv", (tokens, self.q_size + self.k_size + self.v_size), ctx.dtype)
        self.in_proj.forward(x, qkv)
        pooled = cache.state
        if cache.writable:
            ops.pooled_store(qkv, self.q_size, self.q_size + self.k_size, cache.pages, cache.block_table, ctx.token_req,
                             ctx.positions, ctx.req_indptr, ctx.slots, pooled, G, d, dv, cache.page_size, self.pool)
        out = ctx.buffer("pooled_attention.out", (tokens, self.out_size), ctx.dtype)
        from . import pooled_attention_bf16

        if not (ctx.dtype == torch.bfloat16 and pooled_attention_bf16.forward(self, ctx, qkv, cache, out)):
            ops.pooled_attention(qkv, cache.pages, cache.block_table, ctx.token_req, ctx.positions, ctx.slots, pooled, out,
                                 H, G, d, dv, cache.page_size, self.window, self.pool, self.scale)
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
