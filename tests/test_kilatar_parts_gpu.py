"""Each mechanism of the Kilatar design alone: the kernels and parts against the plain functions of
tests/plain_kilatar.py, at sizes of their own, with inputs designed so that a fault shows (keys just inside and just
outside a chunk's edge, one far key among hundreds, keys at a page's border, stale pages full of NaN, states that must
carry over portions, slots and hundreds of steps, a correction that changes the choice and not the weight, identity
experts, a shared expert's gate)."""
import math

import pytest
import torch

import plain_kilatar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().double(), want.double()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} and {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    err = (got - want).abs().max()
    assert err <= tol * want.abs().max(), f"{what}: {err:.3e} > {tol:.1e} * {want.abs().max():.3f}"


class Ctx:
    """What a part reads of a step, for parts that are run alone: one or several requests' portions."""

    def __init__(self, td, lengths, before, slots, capacity=64):
        self.dtype, self.token_capacity = td, capacity
        self.buffers, self.plans = {}, {}
        i32 = lambda values: torch.tensor(list(values), dtype=torch.int32, device=DEV)
        indptr = [0]
        for n in lengths:
            indptr.append(indptr[-1] + n)
        self.req_indptr, self.slots, self.kv_before = i32(indptr), i32(slots), i32(before)
        self.token_req = i32(r for r, n in enumerate(lengths) for _ in range(n))
        self.positions = i32(before[r] + i for r, n in enumerate(lengths) for i in range(n))
        self.num_requests, self.num_tokens = len(lengths), indptr[-1]
        self.decode_only = all(n == 1 for n in lengths)

    def buffer(self, name, shape, dt):
        key = (name, tuple(shape[1:]), dt)
        if key not in self.buffers or self.buffers[key].shape[0] < shape[0]:
            self.buffers[key] = torch.full(shape, float("nan") if dt != torch.int32 else -7, dtype=dt, device=DEV)
        return self.buffers[key][:shape[0]]

    def leave_pending(self, *a):
        raise AssertionError("not used: accumulate_later is off in these tests")

    def flush_pending(self):
        pass


class Cache:
    def __init__(self, state):
        self.state, self.writable = state, True


def no_deferred_sums(part):
    """Products add into the stream at once (the parts under test then need no step function around them)."""
    for name in ("o_proj", "down_proj"):
        linear = getattr(part, name, None)
        if linear is not None:
            linear.accumulate_later = lambda ctx, x, acc: False


# ------------------------------------------------------------------ frequencies and pairing
def test_frequencies_slowed_down_by_wavelength_and_interleaved_pairs():
    from torchlet_b200.parts.rotary import pair_permutation, scaled_frequencies

    for base, dims, scaling in ((500.0, 8, (8.0, 1.0, 4.0, 64)), (50000.0, 32, (4.0, 1.0, 2.0, 32)), (1e4, 16, None),
                                (250.0, 12, (2.0, 2.0, 2.0, 16))):
        rot = {"base": base, "dims": dims}
        if scaling:
            rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
        want = plain.frequencies(rot)
        got, magnitude = scaled_frequencies(dims, base, rot.get("scaling"))
        assert magnitude == 1.0
        close(got, want, 1e-12, "frequencies")
        if scaling and scaling[1] != scaling[2]:  # all three ranges occur
            plainf = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
            kept, slowed = (want == plainf), torch.isclose(want, plainf / scaling[0], rtol=1e-12)
            assert kept.any() and slowed.any()
    # rows laid out by the permutation and turned split-half equal the interleaved rotation, pair by pair
    d, dims = 12, 8
    order = pair_permutation(d, dims, "interleaved")
    assert order == [0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11]
    x = rand(5, 1, d, seed=1).double()
    pos = torch.tensor([0, 1, 7, 300, 4001])
    freq = plain.frequencies({"base": 100.0, "dims": dims})
    want = plain.rotate_pairs(x, pos, freq)[:, 0][:, order]
    y = x[:, 0][:, order].clone()
    half = dims // 2
    angle = pos.double()[:, None] * freq[None, :]
    u, v = y[:, :half].clone(), y[:, half:dims].clone()
    y[:, :half], y[:, half:dims] = u * angle.cos() - v * angle.sin(), v * angle.cos() + u * angle.sin()
    close(y, want, 1e-12, "pairs")


# ------------------------------------------------------------------ chunked attention
def _paged(k, v, page_size, dtype, seed=0, extra_pages=5):
    """k, v [T, G, d] into a pool whose other pages are NaN, pages handed out in a scrambled order."""
    T, G, d = k.shape
    used = -(-T // page_size)
    total = used + extra_pages + 1
    order = torch.randperm(total - 1, generator=torch.Generator().manual_seed(seed))[:used] + 1
    pages = torch.full((total, 2, G, page_size, d), float("nan"), dtype=dtype)
    for t in range(T):
        page, at = int(order[t // page_size]), t % page_size
        pages[page, 0, :, at] = k[t].to(dtype)
        pages[page, 1, :, at] = v[t].to(dtype)
    return pages.to(DEV), order.to(torch.int32).view(1, -1).to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size,page_size", [(40, 16), (16, 16), (17, 8), (1, 8), (64, 32), (1000, 16), (13, 16)])
def test_chunked_mask_on_designed_keys(dtype, size, page_size):
    """Queries at many places of 700 keys.  Keys are weak except three made to stand out for the last query: the FIRST
    key of its chunk (just inside), the key BEFORE it (just outside, which must not be seen) and one far back.
    Values name their position, so a key that is off by one shows."""
    from torchlet_b200 import ops

    H, G, d, T, scale = 4, 2, 24, 700, 0.3
    td = TORCH[dtype]
    k = rand(T, G, d, seed=8, scale=0.05)
    v = rand(T, G, d, seed=9, scale=0.1)
    v[:, :, 0] = torch.arange(T).float().view(T, 1) / T
    q = rand(T, H, d, seed=10, scale=0.05)
    last = T - 1
    start = last - last % size
    for j, at in enumerate(m for m in (200, start, start - 1) if m >= 0):
        k[at, :, 3 + j] = 6.0
        q[last, :, 3 + j] = 5.0
    k, v, q = k.to(td).double(), v.to(td).double(), q.to(td).double()
    want = plain.softmax_attention(q, k, v, scale, lambda i, j: i // size == j // size)
    pages, table = _paged(k, v, page_size, td, seed=page_size)
    edges = {r for c in range(0, T, size) for r in (c - 1, c, c + 1) if 0 <= r < T}
    rows = sorted({0, 1, 2, 15, 16, 17, 255, 256, 698, 699} | set(list(edges)[:60]))
    qd = q[rows].reshape(len(rows), H * d).to(td).to(DEV)
    out = torch.full((len(rows), H * d), float("nan"), dtype=td, device=DEV)
    pos = torch.tensor(rows, dtype=torch.int32, device=DEV)
    req = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
    ops.attention_generic(qd, H * d, pages, table, req, pos, out, len(rows), H, G, d, page_size, -size, scale)
    close(out.view(len(rows), H, d), want[rows], 2e-5 if dtype == "float32" else 2e-2, "chunked attention")


@pytest.mark.parametrize("d,H,G", [(64, 4, 1), (128, 6, 2), (64, 2, 2)])
@pytest.mark.parametrize("size,page_size", [(150, 16), (64, 16), (48, 8), (1, 16), (1000, 16), (130, 16)])
def test_tensor_core_attention_with_chunks_equals_the_plain_kernel(d, H, G, size, page_size):
    """The mma.sync kernel (64-row tiles for a prompt portion, 16-row tiles with 1, 3 and 20 key splits for a single
    token) and the tcgen05 kernel (a prompt portion, whole and with key splits) against the one-warp-a-row kernel on
    the same pages, with designed keys on both sides of the last chunk's first position."""
    from torchlet_b200 import ops

    T, scale, g = 700, d ** -0.5, H // G
    td = torch.bfloat16
    k = rand(T, G, d, seed=21, scale=0.5)
    v = rand(T, G, d, seed=22, scale=0.5)
    q = rand(T, H, d, seed=23, scale=0.5)
    last = T - 1
    start = last - last % size
    if start > 0:
        k[start, :, 5] = 9.0
        k[start - 1, :, 6] = 9.0
        q[last, :, 5:7] = 6.0
    pages, table = _paged(k, v, page_size, td, seed=d + page_size)
    qd = q.reshape(T, H * d).to(td).to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    zeros = torch.zeros(T, dtype=torch.int32, device=DEV)
    want = torch.empty(T, H * d, dtype=td, device=DEV)
    window = -size
    ops.attention_generic(qd, H * d, pages, table, zeros, pos, want, T, H, G, d, page_size, window, scale)
    rows = torch.arange(0, T * g, 64, dtype=torch.int32, device=DEV)
    indptr = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    before = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = torch.full((T, H * d), float("nan"), dtype=td, device=DEV)
    ops.attention_mma(qd, pages, table, indptr, before, torch.zeros_like(rows), rows, rows.numel(), got, T, H, G, d, page_size,
                      window, scale, rows16=False)
    close(got, want.float().cpu(), 2e-2, "prompt portion")
    if ops.attention_tc_supported(d, g, page_size):
        per = ops.attention_tc_rows(g)
        rows = torch.arange(0, T * g, per, dtype=torch.int32, device=DEV)
        for splits, defer in ((1, False), (3, False), (2, True)):
            got = torch.full((T, H * d), float("nan"), dtype=td, device=DEV)
            merge = ops.attention_tc(qd, pages, table, indptr, before, torch.zeros_like(rows), rows, rows.numel(), got, H, G, d,
                                     page_size, window, scale, splits=splits, token_req=zeros, defer_merge=defer)
            if defer:
                merge()
            close(got, want.float().cpu(), 2e-2, f"prompt portion on tcgen05, {splits} key splits")
        ops.raise_on_wait_errors()
    # single tokens behind cached ones: the last, the first of a chunk, and the last of a chunk
    for at in sorted({last, start, max(start - 1, 0)}):
        indptr = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
        before = torch.tensor([at], dtype=torch.int32, device=DEV)
        for splits in (1, 3, 20):
            one = torch.full((1, H * d), float("nan"), dtype=td, device=DEV)
            ops.attention_mma(qd[at:at + 1], pages, table, indptr, before, None, None, 1, one, 1, H, G, d, page_size, window,
                              scale, rows16=True, splits=splits)
            close(one, want[at:at + 1].float().cpu(), 2e-2, f"single token at {at}, {splits} key splits")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,V,size,dims", [(4, 2, 24, 16, 13, 8), (2, 2, 8, 20, 5, 8), (3, 1, 40, 40, 64, 0),
                                               (4, 1, 64, 64, 48, 32), (2, 1, 64, 128, 100, 64)])
def test_chunked_attention_mixer_with_unequal_key_and_value_sizes(dtype, H, G, D, V, size, dims):
    """The mixer alone (its own projections, the interleaved rotation, heads padded to one size, the cache write and the
    paged kernels), as a whole prompt and as a portion behind cached tokens plus single tokens."""
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import MIXERS, build_part

    td, width, T, page = TORCH[dtype], 64, 150, 16
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.21, "mask": {"size": size}}
    positions = None
    if dims:
        m["rot"] = {"base": 300.0, "dims": dims, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
        positions = PartSpec("rotary_partial", {"head_dim": D, "dims": dims, "base": 300.0, "scaling": m["rot"]["scaling"],
                                                "pairing": "interleaved"})
    w = {"a.q": rand(H * D, width, seed=1, scale=0.3), "a.k": rand(G * D, width, seed=2, scale=0.3),
         "a.v": rand(G * V, width, seed=3, scale=0.3), "a.o": rand(width, H * V, seed=4, scale=0.3)}
    w = {k: t.to(torch.bfloat16).float() for k, t in w.items()}
    h = rand(T, width, seed=5).to(td).float()
    want = plain.chunked_attention(m, {k: t.double() for k, t in w.items()}, "a.", h.double())
    part = build_part(MIXERS, PartSpec("gated_attention", {
        "hidden_size": width, "num_heads": H, "num_kv_heads": G, "head_dim": D, "v_dim": V, "scale": 0.21, "chunk": size,
        "positions": positions, "eps": 1e-6}))
    part.load(w, "a.", DEV, td)
    no_deferred_sums(part)
    spec = part.kv_spec()
    assert spec.head_dim % 8 == 0 and spec.head_dim >= max(D, V) and spec.window == size
    pages = torch.full((40, 2, G, page, spec.head_dim), float("nan"), dtype=td, device=DEV)
    table = (torch.randperm(39, generator=torch.Generator().manual_seed(3))[:12] + 1).to(torch.int32).view(1, -1).to(DEV)

    def run(lengths, before):
        ctx = Ctx(td, lengths, before, [0])
        ctx.req_indptr_host = ctx.req_indptr.cpu().numpy()
        ctx.kv_before_host = ctx.kv_before.cpu().numpy()
        ctx.max_kv_len, ctx.max_q_len = before[0] + lengths[0], lengths[0]
        ctx.upload = lambda values: torch.as_tensor(values, dtype=torch.int32).to(DEV)
        cache = Cache(None)
        cache.pages, cache.block_table, cache.page_size = pages, table, page
        acc = torch.zeros(lengths[0], width, device=DEV)
        part.forward(ctx, h[before[0]:before[0] + lengths[0]].to(td).to(DEV), acc, cache)
        return acc

    tol = 3e-5 if dtype == "float32" else 3e-2
    close(run([T], [0]), want, tol, "whole prompt")
    pages.fill_(float("nan"))
    got = [run([70], [0]), run([60], [70])] + [run([1], [t]) for t in range(130, T)]
    close(torch.cat(got), want, tol, "portions and single tokens")


# ------------------------------------------------------------------ state-space mixer
def _mamba_weights(m, width, seed):
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, channels = H * V, H * V + 2 * G * N
    w = {"m.in": rand(2 * inner + 2 * G * N + H, width, seed=seed, scale=0.25),
         "m.conv": rand(channels, m["conv"], seed=seed + 1, scale=0.5), "m.conv.b": rand(channels, seed=seed + 2, scale=0.3),
         "m.dt_bias": rand(H, seed=seed + 3, scale=0.5), "m.A_log": rand(H, seed=seed + 4, scale=0.7),
         "m.D": 1.0 + rand(H, seed=seed + 5, scale=0.5), "m.norm": 1.0 + rand(inner, seed=seed + 6, scale=0.2),
         "m.o": rand(width, inner, seed=seed + 7, scale=0.25)}
    return {k: t.to(torch.bfloat16).float() for k, t in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,V,N,G,taps,parts", [(4, 12, 20, 2, 4, 2), (1, 8, 4, 1, 1, 1), (2, 24, 8, 1, 2, 1),
                                                (4, 32, 64, 2, 4, 4), (6, 16, 128, 3, 3, 1), (3, 40, 130, 1, 8, 3)])
def test_state_space_mixer_carries_state_and_convolution_inputs(dtype, H, V, N, G, taps, parts):
    """Two requests of unequal length in portions down to ONE and two tokens (shorter than the taps), beside a padding
    lane; the second request then runs again in the slot the first one left (cleared), and a NaN slot nobody owns stays
    NaN."""
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import MIXERS, build_part

    td, width, eps = TORCH[dtype], 48, 1e-5
    m = {"heads": H, "vdim": V, "state": N, "groups": G, "conv": taps, "norm_groups": parts}
    w = _mamba_weights(m, width, seed=H + N)
    part = build_part(MIXERS, PartSpec("mamba2", {"hidden_size": width, "num_heads": H, "v_dim": V, "state_size": N,
                                                  "groups": G, "conv_taps": taps, "norm_groups": parts, "eps": eps}))
    part.load(w, "m.", DEV, td)
    no_deferred_sums(part)
    seqs = [rand(n, width, seed=30 + i).to(td).float() for i, n in enumerate((57, 23))]
    wants = [plain.mamba2(m, {k: t.double() for k, t in w.items()}, "m.", s.double(), eps) for s in seqs]
    slots = 4
    state = {name: torch.zeros((slots, *spec.slot_shape(512)), device=DEV) for name, spec in part.state_spec().items()}
    for t in state.values():
        t[3] = float("nan")  # nobody's slot
    cuts = [[7, 1, 2, 30, 1, 1, 15], [2, 1, 9, 1, 3, 6, 1]]
    at, got = [0, 0], [[], []]
    for step in range(7):
        lengths = [cuts[0][step], cuts[1][step], 1]  # the third lane is padding (slot -1)
        ctx = Ctx(td, lengths, [at[0], at[1], 0], [0, 2, -1])
        x = torch.cat([seqs[0][at[0]:at[0] + lengths[0]], seqs[1][at[1]:at[1] + lengths[1]], torch.ones(1, width)])
        acc = torch.zeros(sum(lengths), width, device=DEV)
        part.forward(ctx, x.to(td).to(DEV), acc, Cache(state))
        got[0].append(acc[:lengths[0]].cpu())
        got[1].append(acc[lengths[0]:lengths[0] + lengths[1]].cpu())
        at = [at[0] + lengths[0], at[1] + lengths[1]]
    tol = 5e-5 if dtype == "float32" else 4e-2
    close(torch.cat(got[0]), wants[0], tol, "request 0")
    close(torch.cat(got[1]), wants[1], tol, "request 1")
    for t in state.values():
        assert torch.isnan(t[3]).all() and torch.isfinite(t[:3]).all()
        t[0].zero_()  # admission clears the slot
    ctx = Ctx(td, [23], [0], [0])
    acc = torch.zeros(23, width, device=DEV)
    part.forward(ctx, seqs[1].to(td).to(DEV), acc, Cache(state))
    close(acc, wants[1], tol, "in a slot used again")


def test_state_space_state_remembers_a_token_far_back():
    """A rate near zero keeps the state: the first token's x is read back by a C that matches its B, 600 tokens later,
    through portions and single tokens."""
    from torchlet_b200 import ops

    H, N, V, T = 1, 8, 8, 600
    scan_in = torch.zeros(T, 2 * N + V)
    scan_in[0, N] = 1.0  # B of token 0: channel 0
    scan_in[0, 2 * N:] = torch.arange(1, V + 1).float()  # dt x of token 0
    scan_in[T - 1, 0] = 1.0  # C of the last token reads channel 0
    decay = torch.full((T, H), 0.9999)
    state = torch.zeros(2, H, N, V, device=DEV)
    out = torch.empty(T, V, device=DEV)
    at = 0
    for n in [1, 200, 1, 1, 396, 1]:
        ind = torch.tensor([0, n], dtype=torch.int32, device=DEV)
        ops.gla_scan(scan_in[at:at + n].contiguous().to(DEV), decay[at:at + n].contiguous().to(DEV), ind,
                     torch.tensor([1], dtype=torch.int32, device=DEV), state, out[at:at + n], 1, H, N, V, 1.0,
                     token_decay=True, qk_heads=1)
        at += n
    want = torch.arange(1, V + 1).double() * 0.9999 ** (T - 1)
    close(out[T - 1], want, 1e-5, "remembered")
    assert float(out[1:T - 1].abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0


# ------------------------------------------------------------------ linear attention with silu and a whole norm
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,V,decay", [(3, 12, 20, (0.9, 0.97, 0.99)), (1, 16, 24, (1.0,)), (2, 64, 64, (0.5, 0.999)),
                                         (4, 128, 32, (0.6, 0.88, 0.97, 0.999))])
def test_lightning_attention_in_portions(dtype, H, D, V, decay):
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import MIXERS, build_part

    td, width, eps, T = TORCH[dtype], 40, 1e-5, 90
    m = {"heads": H, "dim": D, "vdim": V, "decay": list(decay)}
    w = {"r.q": rand(H * D, width, seed=1, scale=0.3), "r.k": rand(H * D, width, seed=2, scale=0.3),
         "r.v": rand(H * V, width, seed=3, scale=0.3), "r.g": rand(H * V, width, seed=4, scale=0.3),
         "r.o": rand(width, H * V, seed=5, scale=0.3), "r.norm": 1.0 + rand(H * V, seed=6, scale=0.2)}
    w = {k: t.to(torch.bfloat16).float() for k, t in w.items()}
    h = rand(T, width, seed=7).to(td).float()
    want = plain.lightning_attention(m, {k: t.double() for k, t in w.items()}, "r.", h.double(), eps)
    part = build_part(MIXERS, PartSpec("retention", {
        "hidden_size": width, "num_heads": H, "head_dim": D, "v_dim": V, "decay": tuple(decay), "eps": eps, "positions": None,
        "k_scale": 1.0, "activation": "silu", "norm": "whole", "gate": "sigmoid"}))
    part.load(w, "r.", DEV, td)
    no_deferred_sums(part)
    state = torch.zeros(3, H, D, V, device=DEV)
    got, at = [], 0
    for n in [1, 2, 40, 1, 1, 30, 15]:
        ctx = Ctx(td, [n], [at], [1])
        acc = torch.zeros(n, width, device=DEV)
        part.forward(ctx, h[at:at + n].to(td).to(DEV), acc, Cache(state))
        got.append(acc.cpu())
        at += n
    close(torch.cat(got), want, 5e-5 if dtype == "float32" else 4e-2, "lightning attention")
    assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


# ------------------------------------------------------------------ latent attention with direct queries and a gate
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,R,V,rank,dims", [(3, 20, 12, 28, 40, 8), (1, 8, 4, 8, 16, 4), (4, 32, 32, 32, 64, 32),
                                               (8, 32, 16, 32, 64, 16)])
def test_latent_attention_with_direct_queries_gate_and_interleaved_pairs(dtype, H, D, R, V, rank, dims):
    """One far key among 300 is made to stand out for the last query through the ROTATED part, whose pairs are
    interleaved: a wrong pairing or a wrong frequency loses it."""
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import MIXERS, build_part

    td, width, eps, T, page = TORCH[dtype], 64, 1e-5, 300, 16
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "kv_rank": rank, "scale": 0.3, "rot": {"base": 2000.0, "dims": dims}}
    w = {"l.q": rand(H * (D + R), width, seed=1, scale=0.2), "l.dkv": rand(rank + R, width, seed=2, scale=0.2),
         "l.dkv.norm": 1.0 + rand(rank, seed=3, scale=0.2), "l.uk": rand(H * D, rank, seed=4, scale=0.2),
         "l.uv": rand(H * V, rank, seed=5, scale=0.2), "l.g": rand(H * V, width, seed=6, scale=0.3),
         "l.o": rand(width, H * V, seed=7, scale=0.3)}
    h = rand(T, width, seed=8)
    # the last query and key 37 agree on a direction of the input that only the rotated rows read
    mark = torch.zeros(width)
    mark[5] = 6.0
    h[37] += mark
    h[T - 1] += mark
    for head in range(H):
        w["l.q"][head * (D + R) + D:head * (D + R) + D + 2, 5] = 1.5
    w["l.dkv"][rank:rank + 2, 5] = 1.5
    w = {k: t.to(torch.bfloat16).float() for k, t in w.items()}
    h = h.to(td).float()
    want = plain.latent_attention(m, {k: t.double() for k, t in w.items()}, "l.", h.double(), eps)
    part = build_part(MIXERS, PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": H, "head_dim": D, "rot_dim": R, "v_dim": V, "q_rank": None, "kv_rank": rank,
        "scale": 0.3, "rot_base": 2000.0, "rot_dims": dims, "eps": eps, "gate": "sigmoid", "pairing": "interleaved"}))
    part.load(w, "l.", DEV, td)
    no_deferred_sums(part)
    pages = torch.full((40, 1, 1, page, rank + R), float("nan"), dtype=td, device=DEV)
    table = (torch.randperm(39, generator=torch.Generator().manual_seed(5))[:20] + 1).to(torch.int32).view(1, -1).to(DEV)

    def run(n, before):
        ctx = Ctx(td, [n], [before], [0])
        ctx.req_indptr_host = ctx.req_indptr.cpu().numpy()
        ctx.max_kv_len = before + n
        ctx.upload = lambda values: torch.as_tensor(values, dtype=torch.int32).to(DEV)
        cache = Cache(None)
        cache.pages, cache.block_table, cache.page_size = pages.view(40, page, rank + R), table, page
        acc = torch.zeros(n, width, device=DEV)
        part.forward(ctx, h[before:before + n].to(td).to(DEV), acc, cache)
        return acc

    got = [run(250, 0), run(40, 250)] + [run(1, t) for t in range(290, T)]
    close(torch.cat(got), want, 5e-5 if dtype == "float32" else 4e-2, "latent attention")


# ------------------------------------------------------------------ feed-forwards
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,ff,tokens", [(96, 40, 33), (64, 72, 1), (128, 192, 300), (50, 21, 17)])
def test_dense_unit_with_gelu_and_biases(dtype, width, ff, tokens):
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import FEED_FORWARDS, build_part

    td = TORCH[dtype]
    w = {"f.gate": rand(ff, width, seed=1, scale=0.3), "f.up": rand(ff, width, seed=2, scale=0.3),
         "f.down": rand(width, ff, seed=3, scale=0.3), "f.gate.b": rand(ff, seed=4), "f.up.b": rand(ff, seed=5),
         "f.down.b": rand(width, seed=6)}
    w = {k: t.to(torch.bfloat16).float() for k, t in w.items()}
    x = rand(tokens, width, seed=7, scale=1.5).to(td).float()
    want = plain.dense_unit({k: t.double() for k, t in w.items()}, "f.", x.double())
    part = build_part(FEED_FORWARDS, PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": ff,
                                                            "activation": "gelu_tanh", "bias": True}))
    part.load(w, "f.", DEV, td)
    no_deferred_sums(part)
    acc = torch.zeros(tokens, width, device=DEV)
    part.forward(Ctx(td, [tokens], [0], [0]), x.to(td).to(DEV), acc)
    close(acc, want, 2e-5 if dtype == "float32" else 3e-2, "dense unit")


def _moe_weights(E, outputs, width, ff, seed, shared):
    w = {"m.router": rand(outputs, width, seed=seed, scale=0.15), "m.correction": rand(outputs, seed=seed + 1, scale=0.15)}
    for e in range(E):
        w[f"m.e{e}.gate"] = rand(ff, width, seed=seed + 10 + e, scale=0.3)
        w[f"m.e{e}.up"] = rand(ff, width, seed=seed + 40 + e, scale=0.3)
        w[f"m.e{e}.down"] = rand(width, ff, seed=seed + 70 + e, scale=0.3)
    if shared:
        w["m.shared.gate"] = rand(shared, width, seed=seed + 2, scale=0.3)
        w["m.shared.up"] = rand(shared, width, seed=seed + 3, scale=0.3)
        w["m.shared.down"] = rand(width, shared, seed=seed + 4, scale=0.3)
        w["m.shared.sg"] = rand(1, width, seed=seed + 5, scale=0.3)
    return {k: t.to(torch.bfloat16).float() for k, t in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,identity,top,width,ff,shared,tokens",
                         [(6, 2, 2, 96, 24, 40, 150), (1, 1, 1, 64, 24, 16, 40), (3, 0, 3, 64, 24, 0, 33),
                          (8, 2, 2, 128, 64, 64, 500), (12, 4, 2, 256, 96, 96, 1), (5, 3, 4, 50, 21, 0, 70),
                          (4, 0, 2, 128, 64, 0, 300), (2, 6, 3, 64, 32, 32, 90)])
def test_routed_experts_with_correction_identity_and_shared_expert(dtype, E, identity, top, width, ff, shared, tokens):
    """The whole part on inputs that both sides hold exactly, with close calls of the choice taken out.  The chosen
    experts are compared best first: by score + correction, while the weights are the scores themselves."""
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import FEED_FORWARDS, build_part

    td, outputs, scale = TORCH[dtype], E + identity, 1.7
    w = _moe_weights(E, outputs, width, ff, seed=E + identity, shared=shared)
    x = rand(tokens, width, seed=20, scale=1.2).to(td).float()
    pick = torch.softmax(x.double() @ w["m.router"].double().T, dim=1) + w["m.correction"].double()
    ranked = pick.sort(dim=1, descending=True).values
    if top < outputs:
        gaps = (ranked[:, :top] - ranked[:, 1:top + 1]).amin(dim=1)
        x = x[gaps > 1e-4] if tokens > 1 else x
        tokens = x.shape[0]
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top, "identity": identity, "scale": scale}}
    if shared:
        mlp["shared"] = {"ff": shared}
    wd = {k: t.double() for k, t in w.items()}
    want = plain.mixture(mlp, wd, "m.", x.double())
    chosen, weights = plain.route(mlp, wd, "m.", x.double())
    shared_part = None
    if shared:
        shared_part = PartSpec("gated_mlp", {"hidden_size": width, "intermediate_size": shared, "activation": "silu",
                                             "bias": False, "token_gate": "sg"})
    part = build_part(FEED_FORWARDS, PartSpec("routed_clamped_glu", {
        "hidden_size": width, "intermediate_size": ff, "limit": None, "num_experts": E, "top_k": top, "score": "softmax",
        "renormalize": True, "renorm_eps": 1e-20, "weight_on": "output", "correction": True, "weight_scale": scale,
        "identity": identity, "shared": shared_part, "shared_prefix": "shared."}))
    part.load(w, "m.", DEV, td)
    if part.shared is not None:
        no_deferred_sums(part.shared)
    ctx = Ctx(td, [tokens], [0], [0])
    acc = torch.zeros(tokens, width, device=DEV)
    part.forward(ctx, x.to(td).to(DEV), acc)
    close(acc, want, 3e-5 if dtype == "float32" else 3e-2, "routed experts")
    choice = ctx.buffers[("moe.choice", (top,), torch.int32)][:tokens].cpu()
    if tokens > 1 or top == outputs:
        assert torch.equal(choice.long(), chosen), "the chosen experts, best first"
        close(ctx.buffers[("moe.weight", (top,), torch.float32)][:tokens], weights, 1e-5, "weights")
    if identity:
        assert (chosen >= E).any(), "no identity expert was chosen: the test shows nothing"


def test_correction_changes_the_choice_and_not_the_weights():
    from torchlet_b200 import ops

    x = torch.zeros(2, 8)
    x[:, 0] = 1.0
    router = torch.zeros(4, 8)
    router[:, 0] = torch.tensor([2.0, 1.0, 0.0, -1.0])
    correction = torch.tensor([0.0, 0.0, 0.9, 0.0])
    choice = torch.empty(2, 2, dtype=torch.int32, device=DEV)
    weight = torch.empty(2, 2, device=DEV)
    ops.moe_route(x.to(DEV), router.to(DEV), choice, weight, softmax_scores=True, renormalize=True, renorm_eps=1e-20,
                  correction=correction.to(DEV), scale=2.5)
    s = torch.softmax(router[:, 0].double(), 0)
    assert choice.cpu().tolist() == [[2, 0], [2, 0]]  # expert 2 only by its correction
    close(weight[0], 2.5 * s[[2, 0]] / (s[2] + s[0]), 1e-6, "weights are the scores")
    ops.moe_route(x.to(DEV), router.to(DEV), choice, weight, softmax_scores=True, renormalize=True, renorm_eps=1e-20)
    assert choice.cpu().tolist() == [[0, 1], [0, 1]]
