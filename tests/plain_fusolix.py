"""A plain, slow implementation of the Fusolix design in float64 on the CPU: whole sequences, no cache,
one function per mechanism, written from the design's equations and sharing no code with the package.

The model keeps ``streams`` copies z_1 .. z_n of the residual stream (all start as E[token] * scale).
A sub-layer f (the mixer, then the feed-forward) with its vectors a (in), b (out) and matrix M (mix):

    u = sum_s a_s z_s;   h = LN(u);   h' = h + conv(h);   y = f(h');   z_t <- sum_s M[s, t] z_s + b_t y

LN is a layer norm with weight and bias, conv a causal per-channel convolution over time.  The mixer
is a softmax attention over a sliding window plus the means of whole blocks of older tokens, beside a
retention (a linear recurrence with a fixed decay per head); the feed-forward a clamped gated unit or a
mixture of experts with group-limited routing.  Output: logits = W_head LN_final(sum_s z_s).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt(centred.pow(2).mean(dim=-1, keepdim=True) + eps) * w + b


def unit_rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt(y.pow(2).mean(dim=-1, keepdim=True) + eps)


def causal_conv(h: torch.Tensor, w: torch.Tensor, history: torch.Tensor | None = None) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] h_(t - taps + 1 + j); ``history`` holds the taps - 1
    rows before the first (zeros at a sequence's start)."""
    T, C = h.shape
    taps = w.shape[1]
    before = torch.zeros(taps - 1, C, dtype=h.dtype) if history is None else history
    padded = torch.cat([before, h], dim=0)
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            out[t] += w[:, j] * padded[t + j]
    return out


def stream_read(z: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """z [n, T, C] -> sum_s a_s z_s."""
    return torch.einsum("s,stc->tc", a, z)


def stream_write(z: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """z_t <- sum_s mix[s, t] z_s + b_t y, all streams at once from the old ones."""
    return torch.einsum("st,sjc->tjc", mix, z) + b.view(-1, 1, 1) * y.unsqueeze(0)


def visible_blocks(i: int, size: int, pool: int) -> int:
    """How many whole blocks of ``pool`` tokens lie before the window of the query at position i: block b
    (positions b pool .. b pool + pool - 1) counts if its last position is at most i - size."""
    n = 0
    while n * pool + pool - 1 <= i - size:
        n += 1
    return n


def pooled_window_attention(q, k, v, scale: float, size: int, pool: int) -> torch.Tensor:
    """One head, query by query: q, k [T, d], v [T, dv].  Query i sees the tokens j with 0 <= i - j < size
    and the mean key / mean value of every block that lies wholly before its window; one softmax."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for i in range(T):
        first = max(0, i - size + 1)
        keys, values = [k[first:i + 1]], [v[first:i + 1]]
        for b in range(visible_blocks(i, size, pool)):
            keys.append(k[b * pool:(b + 1) * pool].mean(dim=0, keepdim=True))
            values.append(v[b * pool:(b + 1) * pool].mean(dim=0, keepdim=True))
        keys, values = torch.cat(keys), torch.cat(values)
        out[i] = torch.softmax((keys @ q[i]) * scale, dim=0) @ values
    return out


def left_mixer(h: torch.Tensor, w: dict, p: str, m: dict) -> torch.Tensor:
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    heads = [pooled_window_attention(q[:, i], k[:, i // (H // G)], v[:, i // (H // G)], m["scale"],
                                     m["mask"]["size"], m["mask"]["pool"]) for i in range(H)]
    return torch.cat(heads, dim=1) @ w[p + "o"].T + w[p + "o.b"]


def rotate_heads(x: torch.Tensor, rot: dict, first_position: int = 0) -> torch.Tensor:
    """x [T, heads, d]: the first rot.dims entries of every head, entry i paired with i + dims / 2, turned
    by the angle position * base^(-2 i / dims)."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    out = x.clone()
    for t in range(x.shape[0]):
        angle = (first_position + t) * f
        c, s = torch.cos(angle), torch.sin(angle)
        u, v = x[t, :, :half], x[t, :, half:dims]
        out[t, :, :half] = u * c - v * s
        out[t, :, half:dims] = v * c + u * s
    return out


def retention(q, k, v, decay: float, state=None):
    """One head: q, k [T, D], v [T, V].  S_t = decay S_(t-1) + k_t v_t^T; o_t = S_t^T q_t.
    Returns (o [T, V], the last state)."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=F64) if state is None else state.clone()
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = decay * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out, S


def right_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rotate_heads((h @ w[p + "q"].T).view(T, H, D), m["rot"])
    k = rotate_heads((h @ w[p + "k"].T).view(T, H, D), m["rot"]) / math.sqrt(D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    heads = [unit_rms(retention(q[:, i], k[:, i], v[:, i], m["decay"][i])[0], eps) for i in range(H)]
    gate = h @ w[p + "g"].T
    return (torch.cat(heads, dim=1) * gate * torch.sigmoid(gate)) @ w[p + "o"].T


def parallel_mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    return (m["left_scale"] * left_mixer(h, w, p + "left.", m["left"])
            + m["right_scale"] * right_mixer(h, w, p + "right.", m["right"], eps))


def dense_feed_forward(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    limit = mlp["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def choose_experts(scores: torch.Tensor, top: int, groups: int, keep: int) -> list:
    """scores [E] of one token: the ``top`` largest among the experts of the ``keep`` best groups (a group:
    E / groups neighbours, scored by its largest member); the lower index wins a tie."""
    E = scores.shape[0]
    per = E // groups
    best = sorted(range(groups), key=lambda g: (-float(scores[g * per:(g + 1) * per].max()), g))[:keep]
    allowed = [e for e in range(E) if e // per in best]
    return sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]


def routed_feed_forward(h: torch.Tensor, w: dict, p: str, mlp: dict, chosen: list | None = None) -> torch.Tensor:
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    scores = torch.softmax(h @ w[p + "router"].T, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        picked = choose_experts(scores[t], router["top"], groups["count"], groups["keep"])
        if chosen is not None:
            chosen.append(picked)
        total = sum(scores[t, e] for e in picked) + 1e-20
        for e in picked:
            g, u = w[f"{p}e{e}.gate"] @ h[t], w[f"{p}e{e}.up"] @ h[t]
            out[t] += scores[t, e] / total * (w[f"{p}e{e}.down"] @ (g * torch.sigmoid(g) * u))
    return out


def forward(cfg: dict, weights: dict, ids, streams: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; ``streams`` receives the sum of the streams after every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps, n = cfg["norm"]["eps"], cfg.get("streams", 1)
    x = w["embed"][torch.tensor(list(ids), dtype=torch.long)] * cfg["embedding"]["scale"]
    z = x.unsqueeze(0).repeat(n, 1, 1)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        for which, sub in (("1", "mixer"), ("2", "mlp")):
            if sub == "mlp" and layer.get("mlp") is None:
                continue
            h = layer_norm(stream_read(z, w[f"{p}hc{which}.in"]), w[f"{p}norm{which}"], w[f"{p}norm{which}.b"], eps)
            if cfg.get("canon"):
                h = h + causal_conv(h, w[f"{p}canon{which}"])
            if sub == "mixer":
                y = parallel_mixer(h, w, p + "mix.", layer["mixer"], eps)
            elif layer["mlp"]["kind"] == "dense":
                y = dense_feed_forward(h, w, p + "mlp.", layer["mlp"])
            else:
                y = routed_feed_forward(h, w, p + "mlp.", layer["mlp"])
            z = stream_write(z, y, w[f"{p}hc{which}.mix"], w[f"{p}hc{which}.out"])
        if streams is not None:
            streams.append(z.sum(dim=0))
    return layer_norm(z.sum(dim=0), w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
