"""Arrangements of a layer's parts around the residual stream.

"pre_norm": h = x + mixer(norm(x)); x' = h + feed_forward(norm(h))
(v10_triton_paged_gqa/layer/transformer_block.py:37-40).  The stream ``acc`` is
float32; mixer and feed-forward add into it.

"parallel_scaled": one norm, mixer and feed-forward side by side, a residual multiplier.

"sandwich": a norm before and behind each sub-layer: x += norm_b(f(norm_a(x))).

"hyper_connected": several residual streams a token, read and written through small learned vectors
and a matrix per sub-layer, with an optional causal convolution over time in front of each sub-layer.
"""
from __future__ import annotations

from .. import ops
from .base import BLOCKS, Block


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    norm_roles = ("mixer_norm", "feed_forward_norm")

    def forward(self, ctx, acc, cache) -> None:
        x = self.norms["mixer_norm"].apply(ctx, acc)
        self.mixer.forward(ctx, x, acc, cache)
        x = self.norms["feed_forward_norm"].apply(ctx, acc)
        self.feed_forward.forward(ctx, x, acc)


@BLOCKS.register("parallel_scaled")
class ParallelScaledBlock(Block):
    """h = norm(x); x' = x + m (mixer(h) + feed_forward(h)); then the layer's token input, if it
    has one, adds m * f(x', tokens).  One norm, both sub-layers read its output; ``m`` is the
    arrangement's parameter ``residual_mult`` (default 1).  The sub-layers add into a zeroed
    float32 stream of their own, so the scaled residual sum is one float32 operation."""

    norm_roles = ("shared_norm",)

    def forward(self, ctx, acc, cache) -> None:
        m = float(self.params.get("residual_mult", 1.0))
        x = self.norms["shared_norm"].apply(ctx, acc)
        delta = ctx.buffer("parallel.delta", tuple(acc.shape), acc.dtype)
        ops.fill_zero(delta)
        self.mixer.forward(ctx, x, delta, cache)
        if self.feed_forward is not None:
            self.feed_forward.forward(ctx, x, delta)
        ctx.flush_pending()
        token_input = self.token_input
        cast = token_input.wants_cast(ctx, acc) if token_input is not None else None
        ops.scaled_add(acc, delta, m, cast)
        if token_input is not None:
            token_input.forward(ctx, acc, m, cast=cast)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """x += post(mixer(pre(x))); then, if the layer has a feed-forward, x += post'(ff(pre'(x))).
    Each sub-layer adds its output into a zeroed float32 stream of its own, the norm behind it
    reads that stream and adds the normed rows into the residual stream (``Norm.add_normed``), so
    the sub-layer's output, its norm and the residual sum are all float32.  That norm's kernel also
    leaves the side stream zeroed again, so it is cleared by a kernel of its own once a step only."""

    norm_roles = ("mixer_norm", "mixer_post_norm")

    def __init__(self, mixer, feed_forward, norms, params=None, token_input=None):
        super().__init__(mixer, feed_forward, norms, params, token_input)
        if feed_forward is not None:
            missing = [role for role in ("feed_forward_norm", "feed_forward_post_norm") if role not in norms]
            if missing:
                raise ValueError(f"block arrangement {self.kind!r} with a feed-forward needs norms for the roles {missing}")

    def forward(self, ctx, acc, cache) -> None:
        side = ctx.buffer("sandwich.side", tuple(acc.shape), acc.dtype)
        x = self.norms["mixer_norm"].apply(ctx, acc)
        if ctx.plans.get("sandwich.side.clean") != side.data_ptr():  # the first sandwich block of the step
            ops.fill_zero(side)
            ctx.plans["sandwich.side.clean"] = side.data_ptr()
        self.mixer.forward(ctx, x, side, cache)
        self.norms["mixer_post_norm"].add_normed(ctx, side, acc, clear=True)
        if self.feed_forward is not None:
            x = self.norms["feed_forward_norm"].apply(ctx, acc)
            self.feed_forward.forward(ctx, x, side)
            self.norms["feed_forward_post_norm"].add_normed(ctx, side, acc, clear=True)


@BLOCKS.register("hyper_connected")
class HyperConnectedBlock(Block):
    """Several residual streams a token (the stream tensor is float32 ``[T, n, width]``) and, optionally, a causal
    convolution over time in front of every sub-layer.  Sub-layer q (the mixer, then the feed-forward if the layer
    has one) with its vectors a_q (in), b_q (out) and its matrix M_q (mix, indexed [from, to]):

        u = sum_s a_q[s] z_s;  h = norm_q(u);  x = h + conv_q(h);  y = sublayer_q(x);
        z_t <- sum_s M_q[s, t] z_s + b_q[t] y          (all streams at once from the old ones)

    conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j) on each channel, zeros before a sequence's start; the last
    taps - 1 rows of h are state of the request (``cache.block_state``), so prompts may be cut anywhere.
    The read, the norm (a layer norm or an RMS norm, by the norm part's ``centre``) and the weighted sum are one
    float32 kernel; the sub-layer adds into a zeroed float32 side stream which the write leaves zeroed again.
    A sub-layer's write is left to the next sub-layer's read (of this block or the next), which does both in one pass
    over the streams (``ctx.leave_write``; whoever needs the streams earlier calls ``ctx.flush_pending``).  In a step of
    single tokens that same kernel also convolves and moves the slots' rows: one launch a sub-layer.

    Parameters: ``streams`` (n), ``taps`` (None: no convolution), ``connections`` (the tensor prefixes of the two
    sub-layers' a, b, M below the layer's: ``<c>in`` [n], ``<c>out`` [n], ``<c>mix`` [n, n]), ``convolutions`` (the
    names of the two convolution weights, [width, taps])."""

    norm_roles = ("mixer_norm",)
    SUBLAYERS = ("mixer", "feed_forward")

    def __init__(self, mixer, feed_forward, norms, params=None, token_input=None):
        super().__init__(mixer, feed_forward, norms, params, token_input)
        if feed_forward is not None and "feed_forward_norm" not in norms:
            raise ValueError(f"block arrangement {self.kind!r} with a feed-forward needs a norm for the role 'feed_forward_norm'")
        self.streams = int(self.params.get("streams", 1))
        self.taps = int(self.params["taps"]) if self.params.get("taps") else None
        if self.taps is not None and not 1 <= self.taps <= 8:
            raise ValueError(f"a convolution of {self.taps} taps is not supported (1 to 8)")
        if not 1 <= self.streams <= 8:
            raise ValueError(f"{self.streams} streams are not supported (1 to 8)")
        for norm in norms.values():
            if not hasattr(norm, "weight") or not hasattr(norm, "centre") or getattr(norm, "groups", 1) != 1:
                raise ValueError(f"block arrangement {self.kind!r} norms inside its own kernel and takes layer_norm or "
                                 f"ungrouped rms_norm parts, not {norm.kind!r}")
        self.width = int(norms["mixer_norm"].size)
        self.a, self.b, self.mix, self.conv = {}, {}, {}, {}

    @classmethod
    def _names(cls, layer) -> list:
        """(sub-layer, connection prefix, convolution name or None) of the sub-layers the layer has."""
        params = layer.block_params
        connections = params.get("connections", ("hc1.", "hc2."))
        convolutions = params.get("convolutions", ("canon1", "canon2")) if params.get("taps") else (None, None)
        both = list(zip(cls.SUBLAYERS, connections, convolutions))
        return both if layer.feed_forward is not None else both[:1]

    @classmethod
    def expected_tensors(cls, layer) -> list:
        from .base import TensorSpec

        n, taps = int(layer.block_params.get("streams", 1)), layer.block_params.get("taps")
        width = int(layer.norm("mixer_norm").part.params["size"])
        out = []
        for _, connection, convolution in cls._names(layer):
            p = layer.prefix + connection
            out += [TensorSpec(p + "in", (n,), init="ones"), TensorSpec(p + "out", (n,), init="ones"),
                    TensorSpec(p + "mix", (n, n), init="eye")]
            if convolution is not None:
                out.append(TensorSpec(layer.prefix + convolution, (width, int(taps))))
        return out

    def load(self, tensors: dict, layer, device, dtype) -> None:
        import torch

        f32 = lambda name: tensors[name].to(device=device, dtype=torch.float32).contiguous()
        for which, connection, convolution in self._names(layer):
            p = layer.prefix + connection
            self.a[which], self.b[which], self.mix[which] = f32(p + "in"), f32(p + "out"), f32(p + "mix")
            self.conv[which] = f32(layer.prefix + convolution) if convolution is not None else None

    def state_spec(self):
        if self.taps is None or self.taps == 1:  # one tap reads the token itself: nothing to keep
            return None
        from .base import StateSpec

        which = self.SUBLAYERS if self.feed_forward is not None else self.SUBLAYERS[:1]
        return {name: StateSpec((self.taps - 1, self.width), "float32") for name in which}

    def _sublayer(self, ctx, z, cache, which: str, norm, run) -> None:
        import torch

        tokens, n, width = z.shape
        conv = self.conv[which]
        write = ctx.take_write(z)  # the write of the sub-layer before, if it was left to us
        ctx.flush_pending()
        state = cache.block_state[which] if conv is not None and self.taps > 1 else None
        if conv is not None and ctx.decode_only:  # a token's history is in its slot alone: one kernel
            x = ctx.buffer("hyper.x", (tokens, width), ctx.dtype)
            ops.hyper_read_norm(z, self.a[which], norm.weight, getattr(norm, "bias", None), norm.eps, x, centre=norm.centre,
                                write=write, conv=(conv, state, ctx.token_req, ctx.slots))
        else:
            h = ctx.buffer("hyper.h", (tokens, width), torch.float32 if conv is not None else ctx.dtype)
            ops.hyper_read_norm(z, self.a[which], norm.weight, getattr(norm, "bias", None), norm.eps, h, centre=norm.centre,
                                write=write)
            x = h
            if conv is not None:
                x = ctx.buffer("hyper.x", (tokens, width), ctx.dtype)
                ops.hyper_conv(h, conv, state, ctx.token_req, ctx.req_indptr, ctx.slots, x)
                if state is not None:
                    ops.hyper_conv_state(h, state, ctx.req_indptr, ctx.slots, ctx.num_requests)
        side = ctx.buffer("hyper.side", (tokens, width), torch.float32)
        if ctx.plans.get("hyper.side.clean") != side.data_ptr():  # the step's first sub-layer; the write kernel clears it after
            ops.fill_zero(side)
            ctx.plans["hyper.side.clean"] = side.data_ptr()
        run(x, side)
        ctx.flush_pending()
        ctx.leave_write(z, side, self.mix[which], self.b[which])

    def forward(self, ctx, acc, cache) -> None:
        if acc.dim() != 3 or acc.shape[1] != self.streams:
            raise ValueError(f"block arrangement {self.kind!r} works on [tokens, {self.streams}, width] streams "
                             "(ModelSpec.streams)")
        self._sublayer(ctx, acc, cache, "mixer", self.norms["mixer_norm"],
                       lambda x, side: self.mixer.forward(ctx, x, side, cache))
        if self.feed_forward is not None:
            self._sublayer(ctx, acc, cache, "feed_forward", self.norms["feed_forward_norm"],
                           lambda x, side: self.feed_forward.forward(ctx, x, side))
