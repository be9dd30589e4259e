"""Rotary position encoding, split-half pairing (element i with i + d/2):
y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin, angle = position * theta^(-2i/d),
angles and rotation in float32 (v10_triton_paged_gqa/layer/rope.py:18-69,
kernel/rope.py:21-41).

This encoding writes the k and v heads to the cache pages of each token in the same pass
(``stores_kv``): the encoded key never needs to exist anywhere else.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import POSITIONS, Positions


@POSITIONS.register("rotary_split_half")
class RotarySplitHalf(Positions):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for split-half rotation")
        self.inv_freq = None

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        # exactly the reference's table: 1 / theta ** (arange(0, d, 2) / d) in float32
        i = torch.arange(0, self.head_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (i / self.head_dim))).to(device)

    accepts_partials = True
    stores_kv = True

    def encode_and_store(self, ctx, qkv, num_heads, num_kv_heads, cache, partials=None) -> None:
        """``partials``: (float32 split sums, splits, bias) of the qkv product when the
        mixer left it unfinished; the sum, the bias, the rotation and the store then run as
        one kernel and ``qkv`` receives the encoded q."""
        if partials is not None:
            ops.finish_qkv_rope(partials[0], partials[1], partials[2], qkv, ctx.positions, ctx.token_req,
                                cache.block_table, cache.pages, self.inv_freq, num_heads, num_kv_heads,
                                self.head_dim, cache.page_size, write_kv=cache.writable)
            return
        ops.rope_kv(qkv, ctx.positions, ctx.token_req, cache.block_table, cache.pages, self.inv_freq,
                    num_heads, num_kv_heads, self.head_dim, cache.page_size, write_kv=cache.writable)


def scaled_frequencies(dims: int, base: float, scaling: dict | None) -> tuple:
    """The rotation frequencies of ``dims`` rotated entries (dims / 2 pairs), f_i = base^(-2 i / dims), and
    the magnitude both cos and sin are multiplied by.  With ``scaling`` (factor, original, fast, slow) the
    frequencies are blended between f_i (pairs that turn fast: more than ``fast`` turns over ``original``
    positions) and f_i / factor (pairs that turn slowly: fewer than ``slow`` turns): with
    pair(turns) = dims ln(original / (2 pi turns)) / (2 ln base), lo = max(floor(pair(fast)), 0),
    hi = min(ceil(pair(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    f_i <- f_i / factor * ramp_i + f_i (1 - ramp_i); the magnitude is 0.1 ln(factor) + 1.
    Taken in float64; returns (float64 tensor [dims / 2], float)."""
    import math

    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return freq, 1.0
    if "low" in scaling or "high" in scaling:
        return wavelength_scaled_frequencies(freq, scaling), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    freq = freq / factor * ramp + freq * (1.0 - ramp)
    return freq, 0.1 * math.log(factor) + 1.0


def wavelength_scaled_frequencies(freq: torch.Tensor, scaling: dict) -> torch.Tensor:
    """Frequencies slowed down by wavelength (``scaling``: factor, low, high, original).  With the wavelength
    l = 2 pi / f: f stays where l < original / high; becomes f / factor where l > original / low; and between the two,
    with s = (original / l - low) / (high - low), (1 - s) f / factor + s f.  float64 in, float64 out."""
    import math

    factor, original = float(scaling["factor"]), float(scaling["original"])
    low, high = float(scaling["low"]), float(scaling["high"])
    wavelength = 2.0 * math.pi / freq
    blend = (original / wavelength - low) / (high - low) if high != low else torch.ones_like(freq)
    mixed = (1.0 - blend) * freq / factor + blend * freq
    out = torch.where(wavelength > original / low, freq / factor, mixed)
    return torch.where(wavelength < original / high, freq, out)


def pair_permutation(head_dim: int, dims: int, pairing: str) -> list:
    """The order in which a head's projection rows are laid out so that the kernels' split-half rotation (entry i with
    i + dims / 2) turns the pairs the checkpoint means.  "split_half": as stored.  "interleaved": the checkpoint pairs
    entry 2i with 2i + 1, so the even entries of the first ``dims`` come first, then the odd ones.  q and k take the
    same order, which leaves every q . k as it was."""
    if pairing == "split_half":
        return list(range(head_dim))
    if pairing != "interleaved":
        raise ValueError(f"unknown pairing {pairing!r} (known: split_half, interleaved)")
    return list(range(0, dims, 2)) + list(range(1, dims, 2)) + list(range(dims, head_dim))


@POSITIONS.register("rotary_partial")
class RotaryPartial(Positions):
    """Split-half rotation of the FIRST ``dims`` entries of every head (entry i with i + dims / 2; the
    rest pass unchanged), with optional frequency scaling (``scaled_frequencies``).  Parameters:
    ``head_dim``, ``dims``, ``base``, ``scaling`` (None, or factor / original / fast / slow for frequencies blended by
    turns, or factor / original / low / high for frequencies slowed down by wavelength), ``pairing`` ("split_half", the
    default, or "interleaved": the checkpoint pairs entry 2i with 2i + 1, and the mixer lays the rows of its q and k
    projections out by ``permutation()`` when it loads them, after which the split-half kernels apply).  The part
    holds the table (``inv_freq``, float32) and the magnitude; the mixer that uses it rotates inside
    its own kernel between its norm and its cache write (``ops.normed_qk_store``)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.params["head_dim"])
        self.dims = int(spec.params["dims"])
        self.base = float(spec.params["base"])
        self.scaling = spec.params.get("scaling")
        self.pairing = spec.params.get("pairing", "split_half")
        if self.dims % 2 or not 0 < self.dims <= self.head_dim:
            raise ValueError(f"{self.dims} rotated entries do not fit a head of {self.head_dim}")
        self.inv_freq = None
        self.magnitude = 1.0
        pair_permutation(self.head_dim, self.dims, self.pairing)  # refuses an unknown pairing

    def permutation(self) -> list:
        return pair_permutation(self.head_dim, self.dims, self.pairing)

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        freq, self.magnitude = scaled_frequencies(self.dims, self.base, self.scaling)
        self.inv_freq = freq.to(torch.float32).to(device)
