"""Which kernels run the bfloat16 attention over a window and pooled blocks.

Where keys and values are equally wide and the tensor-core attention kernels take that size (64 or 128; the cache
then keeps a key plane and a value plane, as theirs does), the work is cut in two: ``pooled_prior`` leaves every
(token, head)'s softmax state over its pooled rows alone (a few rows a query: one a block of ``pool`` tokens), and the
paged kernels of the plain attention (tcgen05 for prompt portions, ``mma.sync`` tiles with split keys for single
tokens, csrc/attention_tc.cu and csrc/attention_mma.cu) walk the window's tokens and join that state where they
normalize a row.  Else (False) the one-warp-a-row kernel does both.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from . import attention_bf16


def split_planes(head_dim: int, v_dim: int) -> bool:
    """Whether the cache keeps a key plane and a value plane (the tensor-core kernels' layout) instead of joined rows."""
    return head_dim == v_dim and head_dim in (64, 128)


# TORCHLET_B200_POOLED_ATTENTION=plain: the one-warp-a-row kernel at every size (for measurements)
TENSOR_CORES = os.environ.get("TORCHLET_B200_POOLED_ATTENTION", "") != "plain"


def forward(mixer, ctx, qkv, cache, out) -> bool:
    d, nh, nkv = mixer.head_dim, mixer.num_heads, mixer.num_kv_heads
    if not TENSOR_CORES or cache.pages.shape[1] != 2 or not split_planes(d, mixer.v_dim) or nh // nkv > 16 or qkv.stride(0) % 8:
        return False
    tokens = qkv.shape[0]
    ml = ctx.buffer("pooled_attention.prior_ml", (tokens, nh, 2), torch.float32)
    acc = ctx.buffer("pooled_attention.prior_acc", (tokens, nh, d), torch.float32)
    ops.pooled_prior(qkv, ctx.token_req, ctx.positions, ctx.slots, cache.state, ml, acc, nh, nkv, d, d, mixer.window,
                     mixer.pool, mixer.scale)
    return attention_bf16.forward(mixer, ctx, qkv, cache, out, prior=(ml, acc))
