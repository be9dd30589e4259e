"""The Kilatar design, plainly: float64, whole sequences, no cache, one function a mechanism.  It shares no code
with the engine; the GPU tests compare the engine with it.

``cfg`` is the configuration as ``config.json`` holds it, ``w`` a dict of float64 tensors by checkpoint name.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    """x divided by its root mean square over the last dimension (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ------------------------------------------------------------------------------------------------ rotation
def frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` the long wavelengths are slowed down."""
    dims = int(rot["dims"])
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    s = rot.get("scaling")
    if s:
        factor, low, high, original = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < original / high:
                out.append(fi)
            elif wavelength > original / low:
                out.append(fi / factor)
            else:
                blend = (original / wavelength - low) / (high - low)
                out.append((1.0 - blend) * fi / factor + blend * fi)
        f = out
    return torch.tensor(f, dtype=F)


def rotate_pairs(x, positions, freq):
    """x [T, heads, d]: entries (2i, 2i+1), i < len(freq), turn by positions * freq_i; the rest stay."""
    out = x.clone()
    n = freq.numel()
    angle = positions.to(F)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(angle), torch.sin(angle)
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------------------- attention
def softmax_attention(q, k, v, scale, visible):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; ``visible(i, j)`` (index tensors -> bool tensor) says which keys
    j <= i query i sees; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & visible(i, j)
    out = torch.zeros(T, H, v.shape[2], dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        p = torch.softmax(s.masked_fill(~seen, -math.inf), dim=-1)
        out[:, h] = p @ v[:, g]
    return out


def latent_attention(m, w, p, h, eps):
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    freq = frequencies(m["rot"])
    q = (h @ w[p + "q"].T).view(T, H, D + R)
    down = h @ w[p + "dkv"].T
    c = rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(down[:, None, rank:], pos, freq)  # [T, 1, R], shared by the heads
    q_rot = rotate_pairs(q[:, :, D:], pos, freq)
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    value = (c @ w[p + "uv"].T).view(T, H, V)
    keys = torch.cat([k_plain, k_rot.expand(T, H, R)], dim=-1)
    queries = torch.cat([q[:, :, :D], q_rot], dim=-1)
    o = softmax_attention(queries, keys, value, float(m["scale"]), lambda i, j: j >= 0).reshape(T, H * V)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def chunked_attention(m, w, p, h):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    if m.get("rot"):
        freq = frequencies(m["rot"])
        q, k = rotate_pairs(q, pos, freq), rotate_pairs(k, pos, freq)
    size = int(m["mask"]["size"])
    o = softmax_attention(q, k, v, float(m["scale"]), lambda i, j: i // size == j // size).reshape(T, H * V)
    return o @ w[p + "o"].T


# -------------------------------------------------------------------------------------------- recurrences
def lightning_attention(m, w, p, h, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, D)
    k = silu(h @ w[p + "k"].T).view(T, H, D)
    v = silu(h @ w[p + "v"].T).view(T, H, V)
    o = torch.zeros(T, H, V, dtype=F)
    for n in range(H):
        S = torch.zeros(D, V, dtype=F)
        for t in range(T):
            S = float(m["decay"][n]) * S + torch.outer(k[t, n], v[t, n])
            o[t, n] = S.T @ q[t, n]
    o = rms(o.reshape(T, H * V), eps) * w[p + "norm"]
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def causal_conv(x, weight, bias):
    """x [T, C], weight [C, taps] (the last column is the current token's), zeros before the start."""
    T, C = x.shape
    taps = weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), x])
    out = bias.expand(T, C).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * weight[:, j]
    return out


def mamba2(m, w, p, h, eps):
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, V)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = torch.zeros(T, H, V, dtype=F)
    for n in range(H):
        g = n // (H // G)
        rate = torch.exp(w[p + "A_log"][n])
        S = torch.zeros(N, V, dtype=F)
        for t in range(T):
            S = torch.exp(-rate * dt[t, n]) * S + dt[t, n] * torch.outer(B[t, g], x[t, n])
            y[t, n] = S.T @ C[t, g] + w[p + "D"][n] * x[t, n]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(m, w, p, h, eps):
    left = chunked_attention(m["left"], w, p + "left.", h)
    right = lightning_attention(m["right"], w, p + "right.", h, eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


# ------------------------------------------------------------------------------------------- feed-forward
def dense_unit(w, p, h):
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (gelu_tanh(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


def expert(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(mlp, w, p, h):
    """(chosen experts [T, top], weights [T, top]) best first; identity experts have the last indices."""
    r = mlp["router"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    pick = s + w[p + "correction"]
    T, top = h.shape[0], int(r["top"])
    chosen = torch.zeros(T, top, dtype=torch.long)
    for t in range(T):
        row = pick[t].clone()
        for j in range(top):
            chosen[t, j] = int(torch.argmax(row))
            row[chosen[t, j]] = -math.inf
    weight = torch.gather(s, 1, chosen)
    weight = weight / (weight.sum(dim=-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    return chosen, weight


def mixture(mlp, w, p, h):
    real = int(mlp["router"]["experts"])
    chosen, weight = route(mlp, w, p, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(chosen.shape[1]):
            e = int(chosen[t, j])
            y = h[t] if e >= real else expert(w, f"{p}e{e}.", h[t:t + 1])[0]
            out[t] += weight[t, j] * y
    if mlp.get("shared"):
        out = out + expert(w, p + "shared.", h) * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return out


def feed_forward(mlp, w, p, h):
    return dense_unit(w, p, h) if mlp["kind"] == "dense" else mixture(mlp, w, p, h)


# -------------------------------------------------------------------------------------------------- model
def layer_runs(cfg):
    """The layers in the order they run: (layer, adds the embedding output first)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or int(loop.get("times", 1)) <= 1:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(start)]
    for k in range(times):
        runs += [(i, k > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def layer(cfg, w, i, x):
    spec, eps = cfg["layers"][i], float(cfg["norm"]["eps"])
    p = f"l{i}."
    h = rms(x, eps) * w[p + "norm1"]
    kind = spec["type"]
    if kind == "latent_attention":
        y = latent_attention(spec["mixer"], w, p + "mix.", h, eps)
    elif kind == "mamba2":
        y = mamba2(spec["mixer"], w, p + "mix.", h, eps)
    elif kind == "parallel":
        y = parallel_mixer(spec["mixer"], w, p + "mix.", h, eps)
    else:
        raise ValueError(kind)
    if spec.get("mlp") is not None:
        y = y + feed_forward(spec["mlp"], w, p + "mlp.", h)
    return x + y


def forward(cfg, w, ids, streams=False):
    """Logits [T, vocab] of one sequence; ``streams``: also the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = rms(w["embed"][torch.as_tensor(ids)], eps) * w["embed.norm"]
    first, seen = x, []
    for i, again in layer_runs(cfg):
        if again:
            x = x + first
        x = layer(cfg, w, i, x)
        seen.append(x)
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    return (logits, torch.stack(seen)) if streams else logits
