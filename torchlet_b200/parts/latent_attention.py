"""Latent attention: queries, keys and values come through low-rank latents, and a token's
cache row is [c (kv_rank) | k_rot (rot_dim)], shared by all heads.

    c_q = rmsnorm(W_dq x) * w_q            q[h] = W_uq,h c_q = [q_plain (dim) | q_rot (rot_dim)]
    [c', k'] = W_dkv x                     c = rmsnorm(c') * w_kv,   k_rot = rotate(k')
    key[h] = [W_uk,h c | k_rot]            value[h] = W_uv,h c
    score = scale (q_plain . W_uk,h c + rotate(q_rot) . k_rot),  causal softmax,  out = W_o [heads]

The attention itself runs in the latent space (csrc/latent_attention.cu): W_uk,h is folded into
the query and W_uv,h applied after the weighted sum of cached rows, so no key or value of a
cached token is ever expanded and prompt portions, single tokens and mixed batches are one code
path.  A layer with ``kv_from`` has no W_dkv and reads another layer's cache rows.

Options: ``q_rank`` None: there is no query latent, q = W_q x (tensor ``q`` instead of dq, dq.norm, uq);
``gate`` "sigmoid": the concatenated heads are multiplied by sigmoid(W_g x) (tensor ``g``) before W_o;
``pairing`` "interleaved": the checkpoint rotates entry 2i with 2i + 1; the rotated rows of W_q (or W_uq) and of W_dkv
are then laid out at load time so that the kernels' split-half rotation turns the same pairs (q and k alike, so every
score is what it was).

Parameters: ``hidden_size``, ``num_heads``, ``head_dim`` (unrotated), ``rot_dim``, ``v_dim``,
``q_rank``, ``kv_rank``, ``scale``, ``rot_base``, ``rot_dims`` (how many of the rot_dim entries
are rotated), ``eps``, ``own_kv``, ``gate``, ``pairing``.  Tensors below the prefix: dq, dq.norm, uq (or q),
[dkv, dkv.norm], uk, uv, [g], o.
"""
from __future__ import annotations

import functools

import numpy as np
import torch

from .. import ops
from ..config.spec import PartSpec
from .base import MIXERS, KVSpec, Mixer, TensorSpec
from .linear import Linear
from .rotary import pair_permutation


ROWS = 64  # packed (token, head) rows of a tile, as in csrc/latent_attention_mma.cu
MIN_KEYS_A_SPLIT = 128
MIN_TOKENS_FOR_HEAD_PRODUCTS = 256  # below: one kernel for all heads on the CUDA cores (a launch a head costs more)


@functools.lru_cache(maxsize=None)
def _sm_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def row_tiles(ctx, heads: int):
    """The row tiles of a step for the tensor-core kernel: (tile_req, tile_row, tiles, key splits),
    planned once a step for every layer with the same number of heads.  A step of single tokens
    plans nothing on the host (tile i is request i's) and splits each request's keys over as many
    CTAs as fill the GPU once, given the longest request the step may meet; the kernel decides on
    the device how many key tiles a split really has."""
    key = ("latent_attention.tiles", heads)
    plan = ctx.plans.get(key)
    if plan is None:
        if ctx.decode_only:
            tiles = ctx.num_requests * (-(-heads // ROWS))
            room = max(1, 2 * _sm_count(torch.cuda.current_device()) // tiles)
            splits = max(1, min(room, -(-ctx.max_kv_len // MIN_KEYS_A_SPLIT), 64))
            plan = (None, None, tiles, splits)
        else:
            indptr = ctx.req_indptr_host
            tile_req, tile_row = [], []
            for r in range(ctx.num_requests):
                rows = int(indptr[r + 1] - indptr[r]) * heads
                for row in range(0, rows, ROWS):
                    tile_req.append(r)
                    tile_row.append(row)
            both = ctx.upload(np.asarray(tile_req + tile_row, dtype=np.int32))
            plan = (both[:len(tile_req)], both[len(tile_req):], len(tile_req), 1)
        ctx.plans[key] = plan
    return plan


@MIXERS.register("latent_attention")
class LatentAttentionMixer(Mixer):
    graph_safe = True  # nothing is planned on the host for single-token steps

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.head_dim = int(p["head_dim"])
        self.rot_dim = int(p["rot_dim"])
        self.v_dim = int(p["v_dim"])
        self.q_rank, self.kv_rank = (int(p["q_rank"]) if p.get("q_rank") else 0), int(p["kv_rank"])
        self.gate = p.get("gate")
        self.pairing = p.get("pairing", "split_half")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"unknown gate {self.gate!r} (known: 'sigmoid', None)")
        self.scale = float(p["scale"])
        self.rot_base = float(p["rot_base"])
        self.rot_dims = int(p.get("rot_dims", self.rot_dim))
        self.eps = float(p["eps"])
        self.own_kv = bool(p.get("own_kv", True))
        if self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ValueError("rot_dims must be even and at most rot_dim")
        self.rot_order = pair_permutation(self.rot_dim, self.rot_dims, self.pairing)
        if self.q_rank == 0 and not p.get("own_kv", True):
            raise ValueError("a latent attention without a query latent that reads another layer's cache is not built")
        if self.kv_rank > 1024 or self.head_dim > 1024:
            raise ValueError(f"kv_rank {self.kv_rank} / head_dim {self.head_dim} are not supported by the latent "
                             "attention kernels (up to 1024)")
        self.row = self.kv_rank + self.rot_dim  # a token's cache row
        self.down_proj: Linear | None = None
        self.uq_proj: Linear | None = None
        self.o_proj: Linear | None = None
        self.uk = self.uv = self.uk_heads = self.q_norm = self.kv_norm = self.inv_freq = None

    def kv_spec(self) -> KVSpec:
        return KVSpec(1, self.row, None, planes=1)

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, H = int(p["hidden_size"]), int(p["num_heads"])
        D, R, V = int(p["head_dim"]), int(p["rot_dim"]), int(p["v_dim"])
        q_rank, kv_rank = (int(p["q_rank"]) if p.get("q_rank") else 0), int(p["kv_rank"])
        if q_rank:
            out = [TensorSpec(prefix + "dq", (q_rank, hidden)), TensorSpec(prefix + "dq.norm", (q_rank,), init="ones"),
                   TensorSpec(prefix + "uq", (H * (D + R), q_rank))]
        else:
            out = [TensorSpec(prefix + "q", (H * (D + R), hidden))]
        if p.get("own_kv", True):
            out += [TensorSpec(prefix + "dkv", (kv_rank + R, hidden)),
                    TensorSpec(prefix + "dkv.norm", (kv_rank,), init="ones")]
        out += [TensorSpec(prefix + "uk", (H * D, kv_rank)), TensorSpec(prefix + "uv", (H * V, kv_rank))]
        if p.get("gate") == "sigmoid":
            out.append(TensorSpec(prefix + "g", (H * V, hidden)))
        out.append(TensorSpec(prefix + "o", (hidden, H * V)))
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        H, D, R = self.num_heads, self.head_dim, self.rot_dim
        identity = self.rot_order == list(range(R))

        def query_rows(w: torch.Tensor) -> torch.Tensor:
            """The rotated rows of every head of a query projection in the kernels' order."""
            if identity:
                return w
            w = w.reshape(H, D + R, w.shape[1])
            return torch.cat([w[:, :D], w[:, D:][:, self.rot_order]], dim=1).reshape(H * (D + R), -1)

        dkv = tensors[prefix + "dkv"] if self.own_kv else None
        if dkv is not None and not identity:
            dkv = torch.cat([dkv[:self.kv_rank], dkv[self.kv_rank:][self.rot_order]], dim=0)
        # one product with float32 output for everything a norm, a rotation or a gate reads:
        # [dq (q_rank) | dkv (kv_rank + rot)] with a query latent, else [dkv | q (H (D + R))]; the gate's rows last
        if self.q_rank:
            down = [tensors[prefix + "dq"]] + ([dkv] if dkv is not None else [])
            self.uq_proj = Linear(query_rows(tensors[prefix + "uq"]), None, device, dtype)
        else:
            down = [dkv, query_rows(tensors[prefix + "q"])]
            self.uq_proj = None
        self.gate_offset = sum(w.shape[0] for w in down)
        if self.gate:
            down.append(tensors[prefix + "g"])
        self.down_proj = Linear(torch.cat(down, dim=0), None, device, dtype)
        self.o_proj = Linear(tensors[prefix + "o"], None, device, dtype)
        self.uk = tensors[prefix + "uk"].to(device=device, dtype=dtype).contiguous()
        self.uv = tensors[prefix + "uv"].to(device=device, dtype=dtype).contiguous()
        # for steps of many tokens in bfloat16: W_uk,h^T as a [kv_rank, dim] matrix a head, the operand
        # layout of the tensor-core product (sizes it takes: everything a multiple of 8)
        self.uk_heads = None
        sizes = (self.head_dim, self.kv_rank, self.rot_dim, self.v_dim)
        if dtype == torch.bfloat16 and all(n % 8 == 0 for n in sizes):
            self.uk_heads = self.uk.view(self.num_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        f32 = lambda name: tensors[prefix + name].to(device=device, dtype=torch.float32).contiguous()
        self.q_norm = f32("dq.norm") if self.q_rank else None
        self.kv_norm = f32("dkv.norm") if self.own_kv else None
        # base^(-2i/dims), taken in float64 and rounded once
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.inv_freq = (self.rot_base ** (-2.0 * i / max(self.rot_dims, 1))).to(torch.float32).to(device)

    def forward(self, ctx, x, acc, cache) -> None:
        tokens, H = x.shape[0], self.num_heads
        if self.own_kv != cache.writable:
            raise ValueError("a latent attention layer writes the cache exactly when it has a W_dkv of its own")
        down = ctx.buffer("latent.down", (tokens, self.down_proj.out_features), torch.float32)
        self.down_proj.forward(x, down)
        latent_width = self.q_rank + (self.kv_rank + self.rot_dim if self.own_kv else 0)
        c_q = ctx.buffer("latent.c_q", (tokens, self.q_rank), ctx.dtype) if self.q_rank else None
        ops.latent_prepare(down[:, :latent_width], self.q_rank, self.kv_rank, self.rot_dim, self.rot_dims, self.q_norm,
                           self.kv_norm, self.inv_freq, self.eps, ctx.positions, ctx.token_req, cache.block_table,
                           cache.pages, cache.page_size, c_q, write_kv=self.own_kv)
        if self.q_rank:
            q = ctx.buffer("latent.q", (tokens, H * (self.head_dim + self.rot_dim)), torch.float32)
            self.uq_proj.forward(c_q, q)
        else:  # the queries are rows of the first product
            q = down[:, latent_width:latent_width + H * (self.head_dim + self.rot_dim)]
        q_abs = ctx.buffer("latent.q_abs", (tokens, H * self.row), ctx.dtype)
        per_head_products = self.uk_heads is not None and tokens >= MIN_TOKENS_FOR_HEAD_PRODUCTS
        if per_head_products:  # many tokens: W_uk,h^T q_plain[h] of every head on the tensor cores
            D, rank = self.head_dim, self.kv_rank
            plain = ctx.buffer("latent.q_plain", (tokens, H * D), ctx.dtype)
            ops.latent_absorb_q(q, self.uk, self.inv_freq, ctx.positions, q_abs, H, D, self.rot_dim, self.rot_dims,
                                rank, fold=False, plain_out=plain)
            for h in range(H):
                ops.gemm_tc(plain[:, h * D:(h + 1) * D], self.uk_heads[h], q_abs[:, h * self.row:h * self.row + rank],
                            None, ops.EPI_STORE_BF16)
        else:
            ops.latent_absorb_q(q, self.uk, self.inv_freq, ctx.positions, q_abs, H, self.head_dim, self.rot_dim,
                                self.rot_dims, self.kv_rank)
        o_lat = ctx.buffer("latent.o_lat", (tokens, H * self.kv_rank), ctx.dtype)
        if ctx.dtype == torch.bfloat16 and ops.latent_attention_mma_supported(self.row, self.kv_rank):
            tile_req, tile_row, tiles, splits = row_tiles(ctx, H)
            ops.latent_attention_mma(q_abs, cache.pages, cache.block_table, ctx.req_indptr, ctx.kv_before, tile_req,
                                     tile_row, tiles, o_lat, tokens, H, self.row, self.kv_rank, cache.page_size,
                                     self.scale, splits)
        else:
            ops.latent_attention(q_abs, cache.pages, cache.block_table, ctx.token_req, ctx.positions, o_lat, tokens, H,
                                 self.row, self.kv_rank, cache.page_size, self.scale)
        out = ctx.buffer("latent.out", (tokens, H * self.v_dim), ctx.dtype)
        if per_head_products:
            V, rank = self.v_dim, self.kv_rank
            for h in range(H):
                ops.gemm_tc(o_lat[:, h * rank:(h + 1) * rank], self.uv[h * V:(h + 1) * V], out[:, h * V:(h + 1) * V],
                            None, ops.EPI_STORE_BF16)
        else:
            ops.latent_expand_o(o_lat, self.uv, out, H, self.v_dim, self.kv_rank,
                                gate=down[:, self.gate_offset:] if self.gate else None)
        if self.gate and per_head_products:
            ops.gate_mul_(out, down[:, self.gate_offset:])
        if not self.o_proj.accumulate_later(ctx, out, acc):
            self.o_proj.forward(out, acc, accumulate=True)
