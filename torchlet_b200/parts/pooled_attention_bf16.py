"""Which kernel runs the bfloat16 attention over a window and pooled blocks: the tensor-core kernel where its
sizes fit, else (False) the one-warp-a-row kernel."""
from __future__ import annotations


def forward(mixer, ctx, qkv, cache, out) -> bool:
    return False
