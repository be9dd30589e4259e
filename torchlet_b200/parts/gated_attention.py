"""Grouped-query attention over a paged cache with the options newer designs combine:

* ``qk_norm`` "whole": q and k are RMS-normed over the WHOLE projection (all heads at once, plain
  weights ``q.norm`` / ``k.norm``) before the rotation; None: no norm;
* ``values_from_keys``: there is no value projection: the value of a token is its key AS PROJECTED
  (before norm and rotation);
* ``positions``: a ``rotary_partial`` part (the first ``dims`` entries of a head rotate) or None;
* ``softcap``: score <- softcap * tanh(score / softcap) after the scale; None: off;
* ``window``: a query at position i sees the keys j with 0 <= i - j < window; None: all before it;
* ``chunk``: a query at position i sees the keys j <= i of its own chunk, floor(j / chunk) = floor(i / chunk), chunks
  counted from position 0 of the sequence (not together with ``window``);
* ``v_dim``: the value size of a head where it differs from the key size (default ``head_dim``);
* ``sink``: one is added to the softmax's denominator, p_j = exp(s_j) / (1 + sum exp(s_j));
* ``gate`` "sigmoid": the concatenated heads are multiplied by sigmoid(W_g x) before the output
  projection; None: no gate.

Query head h reads KV head h // (heads / kv_heads).  The input products (q, k, the gate) run as ONE
product with float32 output, because norm and rotation are float32; one kernel then norms, rotates
and writes q and the cache rows (csrc/gated_attention.cu), and the paged attention kernels of the
plain attention mixer do the rest with softcap, sink and gate as arguments.

Heads whose key and value sizes differ are laid out at load time in rows of one padded size P (the larger of the two,
rounded up to a multiple of 8): zero rows in W_q, W_k and W_v, zero columns in W_o, so that scores and outputs are what they were and every paged
kernel sees heads of P entries.  A position part with ``pairing`` "interleaved" has the rows of W_q and W_k laid out
by its ``permutation()`` in the same pass.

Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``, ``eps`` and the
options above.  Tensors below the prefix: q [H D, hidden], k [G D, hidden], (v [G V, hidden]),
q.norm [H D], k.norm [G D], g [H V, hidden], o [hidden, H V].
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, POSITIONS, KVSpec, Mixer, TensorSpec, build_part
from .linear import Linear


@MIXERS.register("gated_attention")
class GatedAttentionMixer(Mixer):
    graph_safe = True  # nothing is planned on the host for single-token steps

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.qk_dim = int(p["head_dim"])
        self.v_dim = int(p["v_dim"]) if p.get("v_dim") is not None else self.qk_dim
        # the size of a head as the kernels and the pages see it: the larger of the two where they differ (then rounded up
        # to a multiple of 8, which the kernels' 16-byte loads want)
        self.head_dim = self.qk_dim if self.v_dim == self.qk_dim else -(-max(self.qk_dim, self.v_dim) // 8) * 8
        self.padded = self.head_dim != self.qk_dim or self.head_dim != self.v_dim
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.qk_dim ** -0.5
        self.softcap: Optional[float] = float(p["softcap"]) if p.get("softcap") else None
        self.chunk: Optional[int] = int(p["chunk"]) if p.get("chunk") else None
        if self.chunk is not None and p.get("window"):
            raise ValueError("a window and a chunked mask do not go together")
        # the mask code of the paged kernels: positive a sliding window, negative the chunk size, None neither
        self.window: Optional[int] = -self.chunk if self.chunk is not None else (int(p["window"]) if p.get("window") else None)
        self.sink = bool(p.get("sink", False))
        self.values_from_keys = bool(p.get("values_from_keys", False))
        self.qk_norm = p.get("qk_norm")
        self.gate = p.get("gate")
        self.eps = float(p.get("eps", 1e-6))
        if self.qk_norm not in (None, "whole"):
            raise ValueError(f"unknown qk_norm {self.qk_norm!r} (known: 'whole', None)")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"unknown gate {self.gate!r} (known: 'sigmoid', None)")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is not supported (up to 256)")
        if self.padded and (self.qk_norm is not None or self.values_from_keys):
            raise ValueError("heads whose key and value sizes differ are not built together with a norm over the whole "
                             "projection or with values taken from the keys")
        self.positions = build_part(POSITIONS, p["positions"]) if p.get("positions") else None
        if self.positions is not None and not hasattr(self.positions, "inv_freq"):
            raise ValueError("this mixer rotates inside its own kernel and needs a position part with a frequency table")
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.in_proj: Linear | None = None
        self.o_proj: Linear | None = None
        self.q_norm = self.k_norm = None

    def kv_spec(self) -> KVSpec:
        # a chunk's keys all lie within ``chunk`` positions of the query: pages are given back as for a window of that size
        return KVSpec(self.num_kv_heads, self.head_dim, self.chunk if self.chunk is not None else self.window)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, d = int(p["hidden_size"]), int(p["head_dim"])
        dv = int(p["v_dim"]) if p.get("v_dim") is not None else d
        q_size, kv_size = int(p["num_heads"]) * d, int(p["num_kv_heads"]) * d
        out = [TensorSpec(prefix + "q", (q_size, hidden)), TensorSpec(prefix + "k", (kv_size, hidden))]
        if not p.get("values_from_keys", False):
            out.append(TensorSpec(prefix + "v", (int(p["num_kv_heads"]) * dv, hidden)))
        if p.get("qk_norm") == "whole":
            out += [TensorSpec(prefix + "q.norm", (q_size,), init="ones"), TensorSpec(prefix + "k.norm", (kv_size,), init="ones")]
        if p.get("gate") == "sigmoid":
            out.append(TensorSpec(prefix + "g", (int(p["num_heads"]) * dv, hidden)))
        out.append(TensorSpec(prefix + "o", (hidden, int(p["num_heads"]) * dv)))
        if p.get("positions"):
            out += POSITIONS.get(p["positions"].kind).expected_tensors(p["positions"], prefix)
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        names = ["q", "k"] + ([] if self.values_from_keys else ["v"]) + (["g"] if self.gate else [])
        order = self.positions.permutation() if self.positions is not None and hasattr(self.positions, "permutation") else None
        P = self.head_dim

        def heads_of(name: str, size: int, permute: bool) -> torch.Tensor:
            """The projection ``name`` with every head's ``size`` rows in the kernels' order, padded to P rows."""
            w = tensors[prefix + name]
            if not self.padded and (order is None or not permute or order == list(range(size))):
                return w
            w = w.reshape(-1, size, w.shape[1])
            if permute and order is not None:
                w = w[:, order]
            if size != P:
                w = torch.cat([w, w.new_zeros(w.shape[0], P - size, w.shape[2])], dim=1)
            return w.reshape(-1, w.shape[2])

        sizes = {"q": (self.qk_dim, True), "k": (self.qk_dim, True), "v": (self.v_dim, False), "g": (self.v_dim, False)}
        self.in_proj = Linear(torch.cat([heads_of(n, *sizes[n]) for n in names], dim=0), None, device, dtype)
        w_o = tensors[prefix + "o"]
        if self.padded:  # zero columns where the heads' outputs are padded
            w_o = w_o.reshape(w_o.shape[0], self.num_heads, self.v_dim)
            w_o = torch.cat([w_o, w_o.new_zeros(w_o.shape[0], self.num_heads, P - self.v_dim)], dim=2).reshape(w_o.shape[0], -1)
        self.o_proj = Linear(w_o, None, device, dtype)
        if self.qk_norm == "whole":
            self.q_norm = tensors[prefix + "q.norm"].to(device=device, dtype=torch.float32).contiguous()
            self.k_norm = tensors[prefix + "k.norm"].to(device=device, dtype=torch.float32).contiguous()
        if self.positions is not None:
            self.positions.load(tensors, prefix, device, dtype)
        # where the projection rows hold the values and the gate
        self.v_offset = self.q_size if self.values_from_keys else self.q_size + self.kv_size
        self.gate_offset = self.q_size + self.kv_size * (1 if self.values_from_keys else 2)
        self.proj_size = self.gate_offset + (self.q_size if self.gate else 0)

    def forward(self, ctx, x, acc, cache) -> None:
        tokens = x.shape[0]
        proj = ctx.buffer("gated_attention.proj", (tokens, self.proj_size), torch.float32)
        self.in_proj.forward(x, proj)
        q = ctx.buffer("gated_attention.q", (tokens, self.q_size), ctx.dtype)
        positions = self.positions
        ops.normed_qk_store(
            proj, self.q_norm, self.k_norm, positions.inv_freq if positions is not None else None,
            positions.magnitude if positions is not None else 1.0, self.eps, ctx.positions, ctx.token_req,
            cache.block_table, cache.pages, cache.page_size, q, self.num_heads, self.num_kv_heads, self.head_dim,
            positions.dims if positions is not None else 0, self.v_offset, write_kv=cache.writable)
        out = ctx.buffer("gated_attention.out", (tokens, self.q_size), ctx.dtype)
        gate = proj[:, self.gate_offset:] if self.gate else None
        from . import attention_bf16

        # bfloat16 heads of 64 or 128: the tensor-core kernel (tiles of 16 packed rows for single tokens, of 64
        # for prompt portions); else, and in float32, one warp per (token, head)
        if not (ctx.dtype == torch.bfloat16 and attention_bf16.forward(self, ctx, q, cache, out, gate=gate)):
            ops.attention_generic(q, q.stride(0), cache.pages, cache.block_table, ctx.token_req, ctx.positions, out, tokens,
                                  self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size, self.window, self.scale,
                                  softcap=self.softcap, sink=self.sink, gate=gate)
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
