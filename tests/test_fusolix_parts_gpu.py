"""Each mechanism of the Fusolix design alone: the kernels against the plain functions of tests/plain_fusolix.py, at
sizes of their own, with inputs designed so that a fault shows (one far block among hundreds, keys just inside and
just outside the window, blocks just seen and not yet seen, keys at a page's border, stale pages and slots full of NaN,
a state and a convolution history that must carry, experts and groups whose scores lie apart)."""
import math

import pytest
import torch

import plain_fusolix as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def close(got, want, tol, what=""):
    got, want = got.detach().cpu().double(), want.double()
    assert got.shape == want.shape, f"{what}: shapes {tuple(got.shape)} and {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    err = (got - want).abs().max()
    assert err <= tol * want.abs().max(), f"{what}: {err:.3e} > {tol:.1e} * {want.abs().max():.3f}"


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


# ------------------------------------------------- several streams: read + norm, write
@pytest.mark.parametrize("n,width", [(1, 64), (2, 100), (3, 96), (4, 1030), (8, 40)])
def test_streams_are_read_through_a_layer_norm_and_written_all_at_once(n, width):
    from torchlet_b200 import ops

    T = 9
    z = rand(T, n, width, seed=1, scale=3.0) + 0.7  # a mean that the norm must take off
    a, b, mix = rand(n, seed=2), rand(n, seed=3), rand(n, n, seed=4)
    w, bias = 1.0 + rand(width, seed=5, scale=0.3), rand(width, seed=6, scale=0.5)
    zs = z.double().permute(1, 0, 2)  # the plain functions hold [n, T, C]
    want = plain.layer_norm(plain.stream_read(zs, a.double()), w.double(), bias.double(), 1e-5)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        out = torch.empty(T, width, device=DEV, dtype=dtype)
        ops.hyper_read_norm(z.to(DEV), a.to(DEV), w.to(DEV), bias.to(DEV), 1e-5, out)
        close(out, want, tol, "read and norm")
    rows = ints([7, 0, 3])
    out = torch.empty(3, width, device=DEV)
    ops.hyper_read_norm(z.to(DEV), a.to(DEV), w.to(DEV), bias.to(DEV), 1e-5, out, rows=rows)
    close(out, want[[7, 0, 3]], 1e-5, "gathered rows")
    u = plain.stream_read(zs, a.double())
    out = torch.empty(T, width, device=DEV)
    ops.hyper_read_norm(z.to(DEV), a.to(DEV), w.to(DEV), None, 1e-5, out, centre=False)
    close(out, plain.unit_rms(u, 1e-5) * w.double(), 1e-5, "the same read with an RMS norm")
    y = rand(T, width, seed=7)
    got, side = z.to(DEV), y.to(DEV)
    ops.hyper_write(got, side, mix.to(DEV), b.to(DEV))
    close(got.permute(1, 0, 2), plain.stream_write(zs, y.double(), mix.double(), b.double()), 1e-5, "write")
    assert not side.any(), "the side stream is left zeroed"
    acc = rand(T, width, seed=8)
    fan = torch.empty(T, n, width, device=DEV)
    ops.hyper_fanout(acc.to(DEV), fan)
    assert all(torch.equal(fan[:, s].cpu(), acc) for s in range(n))
    total = torch.empty(T, width, device=DEV)
    ops.hyper_collapse(got, total)
    close(total, got.sum(dim=1).cpu(), 1e-6, "the streams' sum")


# ------------------------------------------------------------- input convolution
@pytest.mark.parametrize("taps,width", [(2, 64), (3, 100), (4, 96), (5, 1030), (8, 24)])
def test_input_convolution_carries_its_history_in_the_slot(taps, width):
    """A sequence in portions of 1, 2, many and 1 tokens (shorter and longer than the history), beside a second
    request that starts in the same launch, a padding lane, and the first slot used again from zero."""
    from torchlet_b200 import ops

    T, slots = 40, 3
    h = rand(T, width, seed=10)
    other = rand(11, width, seed=11)
    w = rand(width, taps, seed=12, scale=0.5)
    want = h.double() + plain.causal_conv(h.double(), w.double())
    want_other = other.double() + plain.causal_conv(other.double(), w.double())
    state = torch.full((slots, taps - 1, width), float("nan"), device=DEV)
    state[2].zero_()
    state[0].zero_()
    got = torch.empty(T, width)
    at = 0
    for step, size in enumerate((1, 2, 1, taps - 1, 17, 1, 1, 2)):
        size = min(size, T - at)
        rows = [h[at:at + size]]
        indptr, sl = [0, size], [2]
        if step == 2:  # the other request's whole prompt and a padding lane ride along
            rows += [torch.zeros(1, width), other]
            indptr += [size + 1, size + 1 + len(other)]
            sl += [-1, 0]
        x = torch.cat(rows).to(DEV)
        req = torch.repeat_interleave(torch.arange(len(sl)), torch.tensor(indptr[1:]) - torch.tensor(indptr[:-1]))
        out = torch.full(x.shape, float("nan"), device=DEV)
        ops.hyper_conv(x, w.to(DEV), state, req.int().to(DEV), ints(indptr), ints(sl), out)
        ops.hyper_conv_state(x, state, ints(indptr), ints(sl), len(sl))
        got[at:at + size] = out[:size].cpu()
        if step == 2:
            close(out[size + 1:], want_other, 1e-6, "the request that rode along")
        at += size
    rest = h[at:].to(DEV)
    out = torch.empty(T - at, width, device=DEV, dtype=torch.bfloat16)  # the engine's type for what the sub-layer reads
    ops.hyper_conv(rest, w.to(DEV), state, torch.zeros(T - at, dtype=torch.int32, device=DEV), ints([0, T - at]), ints([2]), out)
    close(got[:at], want[:at], 1e-6, "portions")
    close(out, want[at:], 1e-2, "the rest, rounded")
    assert torch.isnan(state[1]).all(), "a slot nobody owns is not touched"
    close(state[0], other[-(taps - 1):], 1e-7, "the last rows are kept")
    state[0].zero_()  # as at admission
    out = torch.empty(5, width, device=DEV)
    ops.hyper_conv(h[:5].to(DEV), w.to(DEV), state, torch.zeros(5, dtype=torch.int32, device=DEV), ints([0, 5]), ints([0]), out)
    close(out, want[:5], 1e-6, "a slot used again")


@pytest.mark.parametrize("n,taps,width", [(1, 2, 64), (2, 3, 100), (4, 4, 2048), (3, 1, 96), (8, 8, 40), (2, None, 72)])
def test_write_read_norm_and_convolution_in_one_pass(n, taps, width):
    """The read that also does the write before it, and in a step of single tokens the convolution and the slots'
    new rows too, against the separate kernels bit for bit: three requests decode for seven steps beside a padding
    lane, their slots used out of order, a slot nobody owns full of NaN."""
    from torchlet_b200 import ops

    R, slots = 4, 5
    dev = lambda t: t.to(DEV)
    a, b, mix = dev(rand(n, seed=2)), dev(rand(n, seed=3)), dev(rand(n, n, seed=4))
    w, bias = dev(1.0 + rand(width, seed=5, scale=0.3)), dev(rand(width, seed=6, scale=0.5))
    cw = dev(rand(width, taps, seed=12, scale=0.5)) if taps else None
    keep = (taps or 1) - 1
    sl, req, indptr = ints([3, -1, 0, 4]), ints(range(R)), ints(range(R + 1))
    states = []
    for _ in range(2):
        state = torch.full((slots, max(keep, 1), width), float("nan"), device=DEV)
        state[[0, 3, 4]] = 0.0
        states.append(state if keep else None)
    z_one = dev(rand(R, n, width, seed=1, scale=2.0) + 0.5)
    z_two = z_one.clone()
    for step in range(7):
        y = dev(rand(R, width, seed=20 + step))
        # separately: write, read and norm, convolution, the slots' rows
        side = y.clone()
        ops.hyper_write(z_one, side, mix, b)
        h = torch.empty(R, width, device=DEV)
        ops.hyper_read_norm(z_one, a, w, bias, 1e-5, h)
        want = h
        if taps:
            want = torch.empty(R, width, device=DEV)
            ops.hyper_conv(h, cw, states[0], req, indptr, sl, want)
            if keep:
                ops.hyper_conv_state(h, states[0], indptr, sl, R)
        # at once
        side = y.clone()
        got = torch.full((R, width), float("nan"), device=DEV)
        ops.hyper_read_norm(z_two, a, w, bias, 1e-5, got, write=(side, mix, b),
                            conv=(cw, states[1], req, sl) if taps else None)
        assert not side.any(), "the side stream is left zeroed"
        assert torch.equal(z_one, z_two), f"step {step}: the streams"
        assert torch.equal(got, want), f"step {step}: what the sub-layer reads"
        if keep:
            assert torch.equal(states[0][[0, 3, 4]], states[1][[0, 3, 4]]), f"step {step}: the slots' rows"
            assert torch.isnan(states[1][[1, 2]]).all(), "slots nobody owns are not touched"
    if taps and keep:  # and against the plain convolution: request 0's seven tokens through slot 3
        zs = rand(R, n, width, seed=1, scale=2.0) + 0.5
        hs = []
        zz = zs.double().permute(1, 0, 2)
        for step in range(7):
            zz = plain.stream_write(zz, rand(R, width, seed=20 + step).double(), mix.cpu().double(), b.cpu().double())
            hs.append(plain.layer_norm(plain.stream_read(zz, a.cpu().double()), w.cpu().double(), bias.cpu().double(), 1e-5)[0])
        hs = torch.stack(hs)
        x = hs + plain.causal_conv(hs, cw.cpu().double())
        close(got[0], x[-1], 1e-4, "the last token of request 0")


# ------------------------------------------- attention over a window and pooled blocks
class _Step:
    """What the bfloat16 dispatcher of the attention kernels reads of a step: ONE request that brings ``n`` tokens
    behind ``before`` cached ones, its pooled rows in slot 1."""

    def __init__(self, before, n, mixer):
        import numpy as np

        self.mixer, self.plans, self.dtype = mixer, {}, torch.bfloat16
        self.num_tokens, self.num_requests, self.decode_only, self.max_kv_len = n, 1, n == 1, before + n
        self.req_indptr_host, self.kv_before_host = np.array([0, n], dtype=np.int32), np.array([before], dtype=np.int32)
        self.req_indptr, self.kv_before, self.slots = ints([0, n]), ints([before]), ints([1])
        self.positions = torch.arange(before, before + n, dtype=torch.int32, device=DEV)
        self.token_req = torch.zeros(n, dtype=torch.int32, device=DEV)

    def upload(self, values):
        return torch.from_numpy(values).to(DEV)

    def buffer(self, name, shape, dtype):
        return torch.full(shape, float("nan"), dtype=dtype, device=DEV)


def _run_pooled(q, k, v, cuts, page_size, size, pool, scale, dtype, poison=True, seed=0, layout="joined"):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of ONE request through the store and attention kernels in portions
    ``cuts``; pages in shuffled order in a pool full of NaN, the pooled rows in slot 1 of three slots full of NaN;
    after every step the pages that lie wholly before the window and the open block are filled with NaN again.
    ``layout``: "joined" rows [key | value]; "split": a key plane and a value plane, the same kernel; "tensor": the
    split planes read by the tensor-core kernels, which join the pooled rows' softmax state."""
    from types import SimpleNamespace

    from torchlet_b200 import ops
    from torchlet_b200.cache.storage import LayerCache
    from torchlet_b200.parts import pooled_attention_bf16

    td = TORCH[dtype]
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(td).to(DEV)
    used = -(-T // page_size)
    num_pages = used + 5
    g = torch.Generator().manual_seed(70 + seed)
    order = torch.randperm(num_pages, generator=g)[:used]
    table = order.int().view(1, used).to(DEV)
    if layout == "joined":
        pages = torch.full((num_pages, 1, G, page_size, d + dv), float("nan"), dtype=td, device=DEV)
    else:
        pages = torch.full((num_pages, 2, G, page_size, d), float("nan"), dtype=td, device=DEV)
    mixer = SimpleNamespace(head_dim=d, v_dim=dv, num_heads=H, num_kv_heads=G, window=size, pool=pool, scale=scale)
    max_blocks = -(-T // pool)
    pooled = torch.full((3, max_blocks, G, d + dv), float("nan"), device=DEV)
    out = torch.full((T, H * dv), float("nan"), dtype=td, device=DEV)
    at = 0
    for n in cuts:
        positions = torch.arange(at, at + n, dtype=torch.int32, device=DEV)
        req = torch.zeros(n, dtype=torch.int32, device=DEV)
        part = proj[at:at + n]
        ops.pooled_store(part, H * d, H * d + G * d, pages, table, req, positions, ints([0, n]), ints([1]), pooled, G, d, dv,
                         page_size, pool)
        if layout == "tensor":
            # poisoned pages hold NaN; the tensor-core kernels load whole tiles and mask the scores, but 0 x NaN
            # would spoil P V: as in the engine, stale pages hold finite numbers
            pages.nan_to_num_(nan=1e4)
            step = _Step(at, n, mixer)
            cache = LayerCache(pages, table, page_size, pooled, writable=True)
            assert pooled_attention_bf16.forward(mixer, step, part, cache, out[at:at + n])
        else:
            ops.pooled_attention(part, pages, table, req, positions, ints([1]), pooled, out[at:at + n], H, G, d, dv,
                                 page_size, size, pool, scale)
        at += n
        if poison:
            for p in range(max(0, at - max(size, pool)) // page_size):
                pages[int(order[p])] = float("nan") if layout != "tensor" else 1e4
    assert at == T
    assert torch.isnan(pooled[0]).all() and torch.isnan(pooled[2]).all(), "other requests' slots are not touched"
    return out.float().cpu().view(T, H, dv)


def _plain_pooled(q, k, v, scale, size, pool):
    H, G = q.shape[1], k.shape[1]
    heads = [plain.pooled_window_attention(q[:, h].double(), k[:, h // (H // G)].double(), v[:, h // (H // G)].double(),
                                           scale, size, pool) for h in range(H)]
    return torch.stack(heads, dim=1)


def _aim(q, k, scale, i, j, score=14.0):
    """Make every head's query at position i point at key j, so that j's score stands out wherever j is seen."""
    H, G = q.shape[1], k.shape[1]
    for h in range(H):
        key = k[j, h // (H // G)]
        q[i, h] = key * (score / (scale * float(key @ key)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,size,pool,page_size", [
    (4, 2, 24, 16, 13, 5, 16), (1, 1, 40, 8, 1, 1, 8), (2, 1, 12, 40, 7, 16, 8), (6, 3, 8, 8, 20, 4, 16),
    (4, 1, 64, 64, 150, 16, 16), (6, 2, 128, 64, 70, 24, 32), (2, 2, 64, 128, 33, 8, 16), (3, 1, 256, 72, 16, 16, 16),
    (8, 2, 128, 128, 40, 8, 64), (3, 3, 64, 64, 129, 3, 24), (2, 1, 24, 24, 10, 7, 8)])
def test_window_and_pooled_blocks_on_designed_keys(dtype, H, G, d, dv, size, pool, page_size):
    """Queries that point at the key just inside the window, at the key just outside it (seen only if it ends a block,
    and then as its block's mean), at a token of the newest block that is seen and of the next one, which is not yet;
    among the last tokens, which are run in a prompt, decoded one by one, and in portions down to two tokens; and at
    the first tokens of the sequence."""
    T = 230
    td = TORCH[dtype]
    scale = 1.3 / math.sqrt(d)
    q, k, v = rand(T, H, d, seed=1), rand(T, G, d, seed=2), rand(T, G, dv, seed=3)
    k, v = k.to(td).float(), v.to(td).float()
    probes = []
    for n, i in enumerate(range(T - 36, T, 3)):
        newest = (i - size + 1) // pool - 1  # the newest block the query sees (if any)
        targets = [i - size + 1, i - size, newest * pool + pool // 2, (newest + 1) * pool, i - size - 1]
        j = targets[n % len(targets)]
        if 0 <= j <= i:
            _aim(q, k, scale, i, j)
            probes.append(i)
    for i, j in ((size - 1, 0), (size, 0), (size + pool - 1, 0), (size + pool - 2, pool - 1), (0, 0), (1, 0), (2, 1)):
        if 0 <= j <= i < T - 40:
            _aim(q, k, scale, i, j)
    q = q.to(td).float()
    want = _plain_pooled(q, k, v, scale, size, pool)
    tol = 2e-5 if dtype == "float32" else 2e-2
    whole = _run_pooled(q, k, v, [T], page_size, size, pool, scale, dtype, poison=False)
    close(whole, want, tol, "a whole prompt")
    decoded = _run_pooled(q, k, v, [T - 40] + [1] * 40, page_size, size, pool, scale, dtype, seed=1)
    close(decoded, want, tol, "decoded")
    cuts, pattern = [], [7, 2, 5, 3, 16, 2, 9, 1, 4, 33, 2, 6, 17, 8, 15, 1, 2, 2, 13, 37]
    while sum(cuts) < T:
        cuts.append(min(pattern[len(cuts) % len(pattern)], T - sum(cuts)))
    portions = _run_pooled(q, k, v, cuts, page_size, size, pool, scale, dtype, seed=2)
    close(portions, want, tol, "portions")
    if dtype == "float32":  # the order of every sum depends on the position alone
        assert torch.equal(whole, decoded) and torch.equal(whole, portions)
    assert probes
    if d == dv:
        split = _run_pooled(q, k, v, cuts, page_size, size, pool, scale, dtype, seed=3, layout="split")
        assert torch.equal(split, portions), "a key plane and a value plane hold the same numbers as joined rows"
        if dtype == "bfloat16" and d in (64, 128):
            for name, these in (("a whole prompt", [T]), ("decoded", [T - 40] + [1] * 40), ("portions", cuts)):
                got = _run_pooled(q, k, v, these, page_size, size, pool, scale, dtype, seed=4, layout="tensor")
                close(got, want, tol, f"tensor cores: {name}")


@pytest.mark.parametrize("dtype,d,layout", [("float32", 16, "joined"), ("bfloat16", 16, "joined"), ("float32", 64, "split"),
                                             ("bfloat16", 64, "tensor"), ("bfloat16", 128, "tensor")])
def test_one_block_far_back_among_hundreds(dtype, d, layout):
    """700 tokens in blocks of 4 behind a window of 20: the last queries point at a key of block 3; its value, through
    the block's mean, is what comes out."""
    T, H, G, dv, size, pool = 700, 2, 1, d, 20, 4
    td = TORCH[dtype]
    scale = 0.25
    q, k, v = rand(T, H, d, seed=4), rand(T, G, d, seed=5, scale=0.3), rand(T, G, dv, seed=6, scale=0.3)
    k[12:16] = 0.0
    k[12:16, 0, 5] = 3.0  # the four keys of block 3 agree, so the mean is as long as each
    v[12:16, 0] = torch.arange(dv).float() - 7.0
    k, v = k.to(td).float(), v.to(td).float()
    for i in range(T - 5, T):
        _aim(q, k, scale, i, 13, score=20.0)
    q = q.to(td).float()
    want = _plain_pooled(q, k, v, scale, size, pool)
    tol = 2e-5 if dtype == "float32" else 2e-2
    for cuts in ([T], [T - 8] + [1] * 8, [350, 2, 340, 8]):
        got = _run_pooled(q, k, v, cuts, 16, size, pool, scale, dtype, layout=layout)
        close(got, want, tol, f"cuts {cuts[:3]}")
        close(got[-1, 0], v[13, 0], 5e-2, "the far block's value")


# -------------------------------------------------------------------- retention
@pytest.mark.parametrize("heads,dim,dims,base,first", [(6, 24, 8, 500.0, 0), (2, 16, 16, 100.0, 37), (3, 40, 2, 1e6, 1500),
                                                       (1, 64, 32, 10000.0, 2000)])
def test_rotation_of_float32_heads_far_into_a_sequence(heads, dim, dims, base, first):
    from torchlet_b200 import ops
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import POSITIONS, build_part

    T = 50
    part = build_part(POSITIONS, PartSpec("rotary_partial", {"head_dim": dim, "dims": dims, "base": base, "scaling": None}))
    part.load({}, "", DEV, torch.float32)
    x = rand(T, heads * dim + 10, seed=20)  # ten more entries behind the heads, which stay
    rows = x.to(DEV)
    ops.rotate_heads_f32(rows, torch.arange(first, first + T, dtype=torch.int32, device=DEV), part.inv_freq, heads, dim, dims)
    want = plain.rotate_heads(x[:, :heads * dim].double().view(T, heads, dim), {"dims": dims, "base": base}, first)
    # float32 angles: a position of 2,000 is held to 1.2e-4 radians
    close(rows[:, :heads * dim].view(T, heads, dim), want, 1e-5 if first < 100 else 1e-3, "rotation")
    assert torch.equal(rows[:, heads * dim:].cpu(), x[:, heads * dim:])
    assert torch.equal(rows[:, dims:dim].cpu(), x[:, dims:dim]), "entries behind the rotated ones pass unchanged"


@pytest.mark.parametrize("H,D,V,decay", [(3, 12, 20, (0.9, 0.97, 0.99)), (1, 40, 8, (1.0,)), (2, 64, 64, (0.99, 0.5)),
                                         (1, 128, 32, (0.98,)), (2, 10, 6, (0.25, 0.999)), (1, 256, 72, (0.95,))])
def test_retention_carries_the_state(H, D, V, decay):
    """Scan and finish against the plain recurrence: a sequence in three portions (the state is carried in the slot), a
    second request in another slot in the same launch, a padding lane, and the first slot used again from zero."""
    from torchlet_b200 import ops

    T, slots = 57, 3
    proj = rand(T, 2 * H * D + 2 * H * V, seed=24, scale=0.7)
    q = proj[:, :H * D].double().view(T, H, D)
    k = proj[:, H * D:2 * H * D].double().view(T, H, D) / math.sqrt(D)
    v = proj[:, 2 * H * D:2 * H * D + H * V].double().view(T, H, V)
    g = proj[:, 2 * H * D + H * V:].double()

    def plain_run(first, last):
        return torch.cat([plain.retention(q[first:last, h], k[first:last, h], v[first:last, h], decay[h])[0] for h in range(H)], dim=1)

    dproj, a = proj.to(DEV), torch.tensor(decay, device=DEV)
    state = torch.full((slots, H, D, V), float("nan"), device=DEV)
    state[0].zero_()
    state[2].zero_()
    rows1 = list(range(0, 20)) + [20] + list(range(40, 57))  # request A (slot 2), a padding lane, request B (slot 0)
    o1 = torch.full((len(rows1), H * V), float("nan"), device=DEV)
    ops.gla_scan(dproj[rows1].contiguous(), a, ints([0, 20, 21, 38]), ints([2, -1, 0]), state, o1, 3, H, D, V, D ** -0.5,
                 fixed_decay=True)
    close(o1[:20], plain_run(0, 20), 2e-5, "A, first portion")
    assert torch.equal(o1[20], torch.zeros(H * V, device=DEV)), "a padding lane writes zeros"
    close(o1[21:], plain_run(40, 57), 2e-5, "B")
    assert torch.isnan(state[1]).all(), "a slot nobody owns is not touched"
    out = torch.empty(T, H * V, device=DEV)
    for first, last in ((20, 22), (22, 40)):
        ops.gla_scan(dproj[first:last], a, ints([0, last - first]), ints([2]), state, out[first:last], 1, H, D, V, D ** -0.5,
                     fixed_decay=True)
    close(out[20:40], plain_run(0, 40)[20:], 2e-5, "A, carried")
    state[0].zero_()
    o = torch.empty(9, H * V, device=DEV)
    ops.gla_scan(dproj[:9], a, ints([0, 9]), ints([0]), state, o, 1, H, D, V, D ** -0.5, fixed_decay=True)
    close(o, plain_run(0, 9), 2e-5, "a slot used again")
    want = plain.unit_rms(plain_run(0, 9).view(9, H, V), 1e-5).reshape(9, H * V) * (g[:9] * torch.sigmoid(g[:9]))
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        fin = torch.empty(9, H * V, device=DEV, dtype=dtype)
        ops.gla_finish(o, dproj[:9], 2 * H * D + H * V, None, fin, H, V, 1e-5)
        close(fin, want, tol, "unit norm without a weight, gate")


def test_retention_remembers_a_token_far_back():
    """Token 3's key is orthogonal to all others; 600 single-token steps later a query along it still reads token 3's
    value, decayed 597 times, and nothing else."""
    from torchlet_b200 import ops

    T, H, D, V = 604, 2, 16, 8
    decay = (0.995, 1.0)
    proj = rand(T, 2 * H * D + 2 * H * V, seed=30, scale=0.5)
    keys = proj[:, H * D:2 * H * D].view(T, H, D)
    keys[:, :, 0] = 0.0
    keys[3, :, 0] = 2.0
    proj[T - 1, :H * D].view(H, D).zero_()
    proj[T - 1, :H * D].view(H, D)[:, 0] = 1.0
    state = torch.zeros(1, H, D, V, device=DEV)
    dproj, a = proj.to(DEV), torch.tensor(decay, device=DEV)
    out = torch.empty(T, H * V, device=DEV)
    ops.gla_scan(dproj[:4], a, ints([0, 4]), ints([0]), state, out[:4], 1, H, D, V, D ** -0.5, fixed_decay=True)
    for t in range(4, T):
        ops.gla_scan(dproj[t:t + 1], a, ints([0, 1]), ints([0]), state, out[t:t + 1], 1, H, D, V, D ** -0.5, fixed_decay=True)
    v3 = proj[3, 2 * H * D:2 * H * D + H * V].double().view(H, V)
    want = torch.stack([v3[h] * (2.0 / math.sqrt(D)) * decay[h] ** (T - 1 - 3) for h in range(H)])
    close(out[T - 1].view(H, V), want, 1e-4, "the value remembered")


# ----------------------------------------------------------- routed feed-forward
def test_only_experts_of_the_best_groups_are_chosen():
    """Given scores: the best expert of a group that is not kept loses to lesser ones of kept groups; equal group scores
    and equal scores: the lower index wins; the weights are the softmax scores over ALL experts, divided by the chosen
    ones' sum."""
    from torchlet_b200 import ops

    logits = torch.tensor([
        [0.0, 5.0, 4.0, 0.1, 4.5, 0.2, 0.3, 3.0],   # groups of two: maxima 5, 4, 4.5, 3
        [1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0],   # all equal
        [0.0, 0.0, 3.0, 2.9, 0.0, 0.0, 2.95, 2.8],  # groups 1 and 3 lead
        [2.0, -1.0, 1.9, 1.8, 1.7, -3.0, 0.0, 1.95],
    ])
    E = logits.shape[1]
    x = torch.eye(4, 8)
    router = torch.zeros(E, 8)
    router[:, :4] = logits.T
    scores = torch.softmax(logits.double(), dim=1)
    for groups, keep, top in ((4, 2, 2), (4, 2, 3), (4, 3, 4), (2, 1, 3), (8, 3, 3), (1, 1, 4), (4, 4, 5), (4, 1, 1)):
        choice = torch.empty(4, top, dtype=torch.int32, device=DEV)
        weight = torch.empty(4, top, device=DEV)
        ops.moe_route(x.to(DEV), router.to(DEV), choice, weight, softmax_scores=True, renormalize=True, groups=groups,
                      keep=keep, renorm_eps=1e-20)
        for t in range(4):
            want = plain.choose_experts(scores[t], top, groups, keep)
            assert choice[t].cpu().tolist() == want, f"groups {groups}, keep {keep}, top {top}, token {t}"
            close(weight[t], scores[t, want] / scores[t, want].sum(), 1e-6, "weights")
    choice = torch.empty(4, 2, dtype=torch.int32, device=DEV)
    weight = torch.empty(4, 2, device=DEV)
    ops.moe_route(x.to(DEV), router.to(DEV), choice, weight, softmax_scores=True, renormalize=True, groups=4, keep=2,
                  renorm_eps=1e-20)
    assert choice.cpu().tolist() == [[1, 4], [0, 1], [2, 6], [0, 7]]


def _moe_weights(E, width, ff, seed):
    w = {"router": rand(E, width, seed=seed, scale=0.15).to(torch.bfloat16).float()}
    for e in range(E):
        w[f"e{e}.gate"] = rand(ff, width, seed=seed + 10 + e, scale=0.3).to(torch.bfloat16).float()
        w[f"e{e}.up"] = rand(ff, width, seed=seed + 40 + e, scale=0.3).to(torch.bfloat16).float()
        w[f"e{e}.down"] = rand(width, ff, seed=seed + 70 + e, scale=0.3).to(torch.bfloat16).float()
    return w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,groups,keep,width,ff,tokens", [
    (6, 2, 3, 2, 96, 40, 150), (1, 1, 1, 1, 64, 24, 7), (3, 3, 3, 3, 64, 24, 33), (8, 2, 4, 2, 128, 64, 300),
    (16, 4, 4, 2, 128, 64, 1), (4, 1, 2, 1, 50, 21, 70), (12, 3, 6, 2, 256, 320, 600), (32, 2, 8, 1, 64, 48, 20)])
def test_routed_plain_gated_experts_with_groups(dtype, E, top, groups, keep, width, ff, tokens):
    """The whole part on inputs that BOTH sides hold exactly (rounded to the engine's type first), so the choice of
    groups and experts is the same unless two scores tie: experts silu(gate) * up without a clamp, softmax scores,
    renormalized weights on the experts' outputs."""
    from torchlet_b200.config import PartSpec
    from torchlet_b200.parts import FEED_FORWARDS, build_part

    td = TORCH[dtype]
    w = _moe_weights(E, width, ff, seed=E)
    x = rand(tokens + 20, width, seed=21, scale=1.2).to(td).float()
    scores = torch.softmax(x.double() @ w["router"].double().T, dim=1)
    ranked = scores.sort(dim=1, descending=True).values
    apart = torch.ones(x.shape[0], dtype=torch.bool)
    if E > 1:
        apart &= (ranked[:, :-1] - ranked[:, 1:]).amin(dim=1) > 1e-4 * ranked[:, 0]  # no close calls
    x = x[apart][:tokens]
    tokens = x.shape[0]
    assert tokens >= 1
    mlp = {"router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}, "expert": {"ff": ff}}
    chosen = []
    want = plain.routed_feed_forward(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", mlp, chosen)
    part = build_part(FEED_FORWARDS, PartSpec("routed_clamped_glu", {
        "hidden_size": width, "intermediate_size": ff, "limit": None, "num_experts": E, "top_k": top, "score": "softmax",
        "renormalize": True, "renorm_eps": 1e-20, "weight_on": "output", "groups": groups, "keep": keep}))
    part.load({"m." + k: v for k, v in w.items()}, "m.", DEV, td)

    class Ctx:
        dtype = td
        token_capacity = 64  # smaller than the step: the scratch must grow with it

        def __init__(self):
            self.buffers = {}

        def buffer(self, name, shape, dt):
            key = (name, tuple(shape[1:]), dt)
            if key not in self.buffers or self.buffers[key].shape[0] < shape[0]:
                self.buffers[key] = torch.full(shape, float("nan") if dt != torch.int32 else -7, dtype=dt, device=DEV)
            return self.buffers[key][:shape[0]]

    ctx = Ctx()
    acc = torch.zeros(tokens, width, device=DEV)
    part.forward(ctx, x.to(td).to(DEV), acc)
    close(acc, want, 2e-5 if dtype == "float32" else 3e-2, "routed feed-forward")
    choice = ctx.buffers[("moe.choice", (top,), torch.int32)][:tokens].cpu()
    assert choice.tolist() == chosen, "the chosen experts, best first"
