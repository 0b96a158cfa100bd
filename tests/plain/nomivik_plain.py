"""The Nomivik decoder written plainly: one function a mechanism, float64, whole sequences, no cache, no batching. It
shares nothing with the package; the tests compare the engine with it.

A model: a token embedding plus a hashed embedding of the (previous, current) token pair; layers in the order the
configuration gives, a range of which runs several times with the same weights (the embedding's output is added again before
every pass but the first); a final norm; logits against the embedding table. A layer: x <- x + mixer(norm1(x)),
x <- x + ff(norm2(x)) where it has a feed-forward, then x <- x + unit(proj(gelu(gate x) * e)) * w with e a slice of a
second embedding of the token. Mixers: a gated linear recurrence behind a short convolution (``rglru``), or two mixers side by
side whose normed outputs are averaged (``parallel``): a windowed attention with grouped heads, biases, a rotation of split
halves, unit-root-mean-square queries and keys, a tanh cap on the scores and one added to the softmax's denominator; and a
matrix memory with exponential gates kept stable by a running maximum.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
RGLRU_RATE = 8.0          # log a = -RGLRU_RATE * r * softplus(lam)
MATRIX_MEMORY_FLOOR = 1e-6  # added to the matrix memory's denominator
# ``forward(..., rounding=f)`` passes every norm's and projection's output through f: with a rounding to 16 bits it shows at
# which positions such rounding alone moves the logits far (a dot product next to zero that decides a direction), so that a
# test of a 16-bit engine can tell an ill-conditioned position from a fault.
_ROUND = None


def _r(z):
    return z if _ROUND is None else _ROUND(z)


# ------------------------------------------------------------------------------------------------ small functions
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z):
    return -softplus(-z)


def rotate_halves(x, positions, dims, base):
    """x [T, heads, dim]: element i < dims/2 is paired with element i + dims/2 and the pair turned by the angle
    position * base^(-2i/dims); elements from ``dims`` on pass."""
    out = x.clone()
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ embedding
def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """The hashed table's row of every token: (previous * mul_prev + token * mul_cur) mod buckets; the sequence's first
    token takes the row after the buckets."""
    return [buckets if t == 0 else (tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(len(tokens))]


def embedding(w, cfg, tokens):
    b = (cfg.get("embedding") or {}).get("bigram")
    if b is None:
        return w["embed"][torch.as_tensor(tokens)]
    rows = pair_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])
    return w["embed"][torch.as_tensor(tokens)] + w["bigram"][torch.as_tensor(rows)]


# ------------------------------------------------------------------------------------------------ mixers
def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps] whose last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], 0)
    out = torch.zeros(T, C, dtype=F64) + bias
    for j in range(taps):
        out = out + padded[j : j + T] * taps_w[:, j]
    return out


def rglru(h, w, p, m):
    """The gated linear recurrence from an empty state. p: the tensors' prefix ('l0.mix.')."""
    T = h.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(_r(h @ w[p + "y"].T + w[p + "y.b"]))
    u = _r(causal_conv(_r(h @ w[p + "x"].T + w[p + "x.b"]), w[p + "conv"], w[p + "conv.b"]))
    ub = u.reshape(T, B, W // B)
    r = sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ra"], ub) + w[p + "ra.b"]).reshape(T, W)
    i = sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ri"], ub) + w[p + "ri.b"]).reshape(T, W)
    log_a = -RGLRU_RATE * r * softplus(w[p + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(W, dtype=F64)
    out = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ w[p + "o"].T


def window_attention(h, w, p, m, eps, positions=None):
    """Grouped-query attention over the last ``mask.size`` positions (the query's own included) with a sink."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(T)) if positions is None else positions
    q = _r(h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    k = _r(h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = _r(h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = unit_rms(rotate_halves(q, positions, m["rot"]["dims"], m["rot"]["base"]), eps)
    k = unit_rms(rotate_halves(k, positions, m["rot"]["dims"], m["rot"]["base"]), eps)
    pos = torch.as_tensor(positions)
    gap = pos[:, None] - pos[None, :]
    seen = (gap >= 0) & (gap < m["mask"]["size"])
    cap = m["softcap"]
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = cap * torch.tanh(s / cap)
        e = torch.where(seen, torch.exp(s), torch.zeros_like(s))
        out[:, head] = (e / (1.0 + e.sum(-1, keepdim=True))) @ v[:, g]       # the sink: a key of score 0 without a value
    return out.reshape(T, H * dv) @ w[p + "o"].T


def matrix_memory(h, w, p, m, eps):
    """The matrix memory with exponential gates, token by token from an empty memory."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = _r(h @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = _r(h @ w[p + "k"].T).reshape(T, H, d)
    v = _r(h @ w[p + "v"].T).reshape(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                       # [T, H], the logarithm of the input gate
    gf = log_sigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))         # the logarithm of the forget gate
    S = torch.zeros(H, d, dv, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + MATRIX_MEMORY_FLOOR
        out[t] = num / den[:, None]
    o = unit_rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    return (o * sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel(h, w, p, m, eps, positions=None):
    left = window_attention(h, w, p + "left.", m["left"], eps, positions)
    right = matrix_memory(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ------------------------------------------------------------------------------------------------ feed-forward, token input
def dense(h, w, p):
    return _r(silu(_r(h @ w[p + "gate"].T)) * _r(h @ w[p + "up"].T)) @ w[p + "down"].T


def token_input(x, w, p, tokens, layer, dim, eps):
    """What a layer adds at its end from the token itself: a slice of a second embedding, gated by the stream."""
    e = w["side.embed"][torch.as_tensor(tokens)][:, layer * dim : (layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return unit_rms(y, eps) * w[p + "norm"]


# ------------------------------------------------------------------------------------------------ the model
def layer_order(cfg):
    """[(layer, whether the embedding's output is added before it)] in the order of running."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for turn in range(times):
        order += [(i, turn > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(cfg, weights, tokens, collect=None, rounding=None):
    """Logits [T, vocab] of a whole sequence. ``collect``: a list that receives the residual after every layer run."""
    global _ROUND
    _ROUND = rounding
    try:
        return _forward(cfg, weights, tokens, collect)
    finally:
        _ROUND = None


def _forward(cfg, weights, tokens, collect):
    w = {k: v.to(F64) if v.is_floating_point() else v for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    side = cfg.get("token_side")
    x0 = embedding(w, cfg, tokens)
    x = x0.clone()
    for i, again in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if again:
            x = x + x0
        hn = _r(rms_norm(x, w[p + "norm1"], eps))
        if layer["type"] == "rglru":
            x = x + rglru(hn, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "parallel":
            x = x + parallel(hn, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense(_r(rms_norm(x, w[p + "norm2"], eps)), w, p + "mlp.")
        if side:
            x = x + token_input(x, w, p + "side.", tokens, i, side["dim"], eps)
        if collect is not None:
            collect.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T
