"""Small Lovurax models for the tests: configurations that differ in every size and option, and weights drawn so that faults
show.

Weights: matrices N(0, std) scaled by their fan-in; norm weights around one; output projections small beside the residual; head
biases of the attention below zero, so that a key's weight is small unless its score is large. ``sharpen`` makes one query token
of the first layer score one key token far above all others, so that whether that key is seen (and at which distance) decides the
output.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from roost_b200.weights.safetensors_io import write_safetensors


def retention(heads=2, dim=8, vdim=6, decay=(0.9, 0.995), rot=4, base=300.0):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"dims": rot, "base": base}}}


def attention(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.4, coef=0.25, every=5):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=6, vdim=5, rank=10, scale=0.5):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def config(layers, width=40, vocab=97, eps=1e-5, logit_scale=1.5):
    return {"architecture": "Lovurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}


# Configurations. None uses the sizes of anyone's released model; they differ from one another in every size.
MIXED = config([(retention(), dense()), (attention(), None), (latent(), dense(ff=18)),
                (attention(heads=3, kv_heads=1, dim=6, vdim=9, scale=0.7, coef=0.6, every=3), dense(ff=30)),
                (retention(heads=3, dim=5, vdim=7, decay=(0.8, 0.99, 0.999), rot=2, base=50.0), None)])
# values that many models make equal or 1 differ here, and the other way round: as many key/value heads as query heads, keys and
# values of one size and of different sizes, a rotation as wide as the head, one head, a decay of one, no query temperature, a
# period of one, a latent wider than the heads, a logit scale of one, layers without a feed-forward, a latent layer first
ODD = config([(latent(heads=1, dim=4, vdim=9, rank=24, scale=1.1), None),
              (attention(heads=3, kv_heads=3, dim=10, vdim=10, scale=0.3, coef=None), dense(ff=31)),
              (retention(heads=1, dim=10, vdim=10, decay=(0.875,), rot=10, base=10000.0), dense(ff=10)),
              (attention(heads=6, kv_heads=2, dim=4, vdim=7, scale=1.1, coef=1.0, every=1), None),
              (retention(heads=4, dim=3, vdim=2, decay=(0.75, 0.9375, 0.984375, 1.0), rot=2, base=2.0), None)], width=36, vocab=61, eps=1e-6,
             logit_scale=1.0)
# sizes of whole vectors (multiples of 8 and 64), heads of more than 128 keys (the recurrence's state in shared memory), values
# beyond 32 columns, a latent the tensor-core form serves, a period the prompts cross once
WIDE = config([(attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.11, coef=0.35, every=64), dense(ff=128)),
               (retention(heads=2, dim=160, vdim=40, decay=(0.9375, 0.998046875), rot=64, base=10000.0), None),
               (latent(heads=4, dim=32, vdim=48, rank=64, scale=0.18), dense(ff=64)),
               (retention(heads=2, dim=64, vdim=64, decay=(0.9, 0.99), rot=64, base=500000.0), dense(ff=64)),
               (attention(heads=4, kv_heads=1, dim=32, vdim=48, scale=0.2, coef=0.1, every=200), None)], width=128, vocab=200, logit_scale=0.7)
CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE}


def tensor_shapes(cfg) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        q = p + "mix."
        shapes.update({p + "norm1": (W,), p + "rg1": (W, W), p + "rg1.b": (W,)})
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "retention":
            shapes.update({q + "q": (H * d, W), q + "k": (H * d, W), q + "v": (H * dv, W), q + "g": (H * dv, W), q + "o": (W, H * dv)})
        elif layer["type"] == "attention":
            G = m["kv_heads"]
            shapes.update({q + "q": (H * d, W), q + "k": (G * d, W), q + "v": (G * dv, W), q + "q.norm": (d,), q + "k.norm": (d,), q + "pb": (H,),
                           q + "g": (H * dv, W), q + "o": (W, H * dv)})
        else:
            r = m["kv_rank"]
            shapes.update({q + "q": (H * d, W), q + "dkv": (r, W), q + "dkv.norm": (r,), q + "uk": (H * d, r), q + "uv": (H * dv, r), q + "g": (H, W),
                           q + "o": (W, H * dv)})
        f = layer["mlp"]
        if f is not None:
            shapes.update({p + "norm2": (W,), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"]), p + "mlp.act": (2,), p + "rg2": (W, W),
                           p + "rg2.b": (W,)})
    return shapes


def draw_tensors(cfg, seed: int, std: float = 0.12) -> dict:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g)
        fan = (32.0 / max(shape[-1], 1)) ** 0.5
        if "norm" in name:
            t = 1.0 + 0.1 * r
        elif name.endswith(".pb"):
            t = -4.0 + 0.7 * r                      # a key counts little unless its score is large: nothing divides the weights by their sum
        elif name.endswith(".act"):
            t = -0.5 + 0.8 * r
        elif name.endswith("mlp.up"):
            t = std * r * fan                       # the activation grows with the square of its argument
        elif name.endswith(".b"):
            t = 0.5 * r
        elif name == "embed":
            t = r
        elif name.endswith(".o") or name.endswith(".down"):
            t = std * r * fan
        else:
            t = 2.0 * std * r * fan
        out[name] = t.to(torch.bfloat16)
    return out


def sharpen(cfg, tensors: dict, key_token: int, query_token: int, strength: float = 12.0, value: float = 6.0) -> None:
    """Changes the mixer of layer 0 so that ``query_token``'s queries point along ``key_token``'s keys, whatever stands around
    either, and the key token's value is large. The key token alone fills element 0 of the stream and the query token alone
    element 1 (no other embedding row writes there); the key, query and value projections read those elements with large
    weights. In a retention layer the direction lies in the elements the rotation leaves alone, so the score does not turn with
    the distance; in the attention the head biases are pushed down so far that every other key weighs next to nothing."""
    layer = cfg["layers"][0]
    m, kind = layer["mixer"], layer["type"]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    emb = tensors["embed"].float()
    emb[:, :2] = 0.0
    emb[key_token, 0] = 4.0
    emb[query_token, 1] = 4.0
    tensors["embed"] = emb.to(torch.bfloat16)
    q = "l0.mix."
    g = torch.Generator().manual_seed(1000 + key_token)

    def boost(name, column, rows_a_head, direction, heads, amount):
        w = tensors[name].float().reshape(heads, rows_a_head, -1)
        w[:, :, column] += amount * direction[None, :]
        tensors[name] = w.reshape(heads * rows_a_head, -1).to(torch.bfloat16)

    if kind != "attention":      # outputs that a norm or a softmax keeps small: the projection makes them count in the stream
        tensors[q + "o"] = (4.0 * tensors[q + "o"].float()).to(torch.bfloat16)
    if kind == "latent_attention":
        r = m["kv_rank"]
        w = tensors[q + "dkv"].float()
        w[0] = 0.0                                     # no other token's latent has a first element
        w[0, 0] = 30.0                                 # the key token's latent is (nearly) its first element alone
        tensors[q + "dkv"] = w.to(torch.bfloat16)
        direction = torch.randn(d, generator=g)
        direction /= direction.norm()
        uk = 0.1 * tensors[q + "uk"].float().reshape(H, d, r)       # other keys score low against the large query
        uk[:, :, 0] += 2.0 * direction[None, :]
        tensors[q + "uk"] = uk.reshape(H * d, r).to(torch.bfloat16)
        boost(q + "q", 1, d, direction, H, strength / (2.0 * r ** 0.5 * m["scale"]))
        vdir = torch.randn(dv, generator=g)
        uv = tensors[q + "uv"].float().reshape(H, dv, r)
        uv[:, :, 0] += value * vdir[None, :] / vdir.norm()
        tensors[q + "uv"] = uv.reshape(H * dv, r).to(torch.bfloat16)
        return
    first_free = m["rot"]["dims"] if kind == "retention" else 0
    assert first_free < d, "the rotation leaves no element alone"
    direction = torch.zeros(d)
    direction[first_free:] = torch.randn(d - first_free, generator=g)
    direction /= direction.norm()
    kv_heads = H if kind == "retention" else m["kv_heads"]
    # a retention state is a sum over hundreds of tokens: the key token's own term is made to stand out among them
    boost(q + "k", 0, d, direction, kv_heads, 60.0 if kind == "retention" else 8.0)
    boost(q + "q", 1, d, direction, H, 8.0)
    vdir = torch.randn(dv, generator=g)
    boost(q + "v", 0, dv, vdir / vdir.norm(), kv_heads, 4.0 * value if kind == "retention" else value)
    if kind == "attention":
        # unit-norm queries and keys along one direction meet with a score of about dim * scale * temperature
        tensors[q + "pb"] = torch.full((H,), -0.55 * d * m["scale"]).to(torch.bfloat16)


def write_model(model_dir, cfg, tensors) -> Path:
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(model_dir / "model.safetensors", tensors, metadata={"format": "pt"})
    return model_dir


def plain_weights(tensors: dict) -> dict:
    """The stored bfloat16 values in float64."""
    return {k: v.double() for k, v in tensors.items()}
