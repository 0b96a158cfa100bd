"""The Lovurax decoder written out plainly in float64: one function a mechanism, loops over tokens and keys where the
formula has them. It shares no code with the package and is what the engine's results are compared with.

Layers are pre-norm: x <- x + gate1 * mixer(n1), x <- x + gate2 * ff(n2) with n = rms_norm(x) and gate = sigmoid(W n + b).
Mixers: ``retention`` (a decaying sum of k v^T a head, rotated q and k), ``attention`` (grouped heads, normed q and k, a query
temperature that grows with the position, a bias that grows with the distance, a sigmoid of every score as its key's weight, an
output gate) and ``latent_attention`` (keys and values made from one cached latent vector a token, softmax, a gate a head).
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2; z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2."""
    ap, an = softplus(p), 0.5 + softplus(q)
    zn = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(zn) - zn) + 0.5 * zn)


def rotate_halves(x, positions, dims, base):
    """x [T, heads, dim]: element i of the first ``dims`` is paired with element i + dims/2 and the pair turned by
    position * base^(-2i/dims)."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = positions.double()[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def retention(h, w, p, m, eps, rounding=None):
    """h [T, width] of one sequence from position 0. S_t = decay S_(t-1) + k_t v_t^T; o_t = S_t^T q_t."""
    rd = rounding or (lambda t: t)
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rd(h @ w[p + "q"].T).reshape(T, H, d)
    k = rd(h @ w[p + "k"].T).reshape(T, H, d)
    v = rd(h @ w[p + "v"].T).reshape(T, H, dv)
    g = rd(h @ w[p + "g"].T)
    q = rotate_halves(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_halves(k, pos, m["rot"]["dims"], m["rot"]["base"]) * d ** -0.5
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=torch.float64)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = rms_norm(out, None, eps).reshape(T, H * dv)
    out = rd(out * (g * sigmoid(g)))
    return rd(out @ w[p + "o"].T)


def head_slopes(heads):
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def attention(h, w, p, m, eps, rounding=None):
    rd = rounding or (lambda t: t)
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rd(h @ w[p + "q"].T).reshape(T, H, d)
    k = rd(h @ w[p + "k"].T).reshape(T, G, d)
    v = rd(h @ w[p + "v"].T).reshape(T, G, dv)
    g = rd(h @ w[p + "g"].T)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rd(rms_norm(k, w[p + "k.norm"], eps))
    if m.get("q_temp") is not None:
        coef, every = m["q_temp"]["coef"], m["q_temp"]["every"]
        temp = torch.tensor([1.0 + coef * math.log((i + 1) // every + 1) for i in range(T)], dtype=torch.float64)
        q = q * temp[:, None, None]
    q = rd(q)
    slopes = head_slopes(H)
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for hd in range(H):
        kv = hd // (H // G)
        for i in range(T):
            distance = i - torch.arange(i + 1, dtype=torch.float64)
            s = (k[: i + 1, kv] @ q[i, hd]) * m["scale"] - slopes[hd] * distance
            out[i, hd] = (sigmoid(s + w[p + "pb"][hd])[:, None] * v[: i + 1, kv]).sum(0)
    out = rd(out.reshape(T, H * dv) * sigmoid(g))
    return rd(out @ w[p + "o"].T)


def latent_attention(h, w, p, m, eps, rounding=None):
    rd = rounding or (lambda t: t)
    T = h.shape[0]
    H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q = rd(h @ w[p + "q"].T).reshape(T, H, d)
    c = rd(rms_norm(rd(h @ w[p + "dkv"].T), w[p + "dkv.norm"], eps))
    k = (c @ w[p + "uk"].T).reshape(T, H, d)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    g = sigmoid(h @ w[p + "g"].T)                    # [T, H]
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for hd in range(H):
        for i in range(T):
            s = (k[: i + 1, hd] @ q[i, hd]) * m["scale"]
            pw = torch.softmax(s, dim=0)
            out[i, hd] = (pw[:, None] * v[: i + 1, hd]).sum(0) * g[i, hd]
    return rd(rd(out.reshape(T, H * dv)) @ w[p + "o"].T)


def dense_ff(h, w, p, rounding=None):
    rd = rounding or (lambda t: t)
    act = w[p + "act"]
    return rd(rd(xielu(rd(h @ w[p + "up"].T), act[0], act[1])) @ w[p + "down"].T)


MIXERS = {"retention": retention, "attention": attention, "latent_attention": latent_attention}


def forward(cfg, w, ids, rounding=None, layer_outputs=None):
    """Logits [T, vocab] of one sequence from its first token; ``layer_outputs``: a list that gets the stream after every layer."""
    rd = rounding or (lambda t: t)
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        n1 = rd(rms_norm(x, w[p + "norm1"], eps))
        y = MIXERS[layer["type"]](n1, w, p + "mix.", layer["mixer"], eps, rounding)
        x = x + y * sigmoid(n1 @ w[p + "rg1"].T + w[p + "rg1.b"])
        if layer.get("mlp") is not None:
            n2 = rd(rms_norm(x, w[p + "norm2"], eps))
            x = x + dense_ff(n2, w, p + "mlp.", rounding) * sigmoid(n2 @ w[p + "rg2"].T + w[p + "rg2.b"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    final = rd(rms_norm(x, w["final.norm"], eps))
    return final @ w["embed"].T * cfg["logit_scale"]
