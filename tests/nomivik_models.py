"""Small Nomivik models for the tests: configurations that differ in every size and option, and weights drawn so that faults
show.

Weights: matrices N(0, std) scaled by their fan-in; norm weights around one; output projections small beside the residual,
so that a layer's rounding error is not doubled by the next one; the recurrence's lam so that a state lives for tens to
hundreds of tokens (a lost or misplaced state changes every later logit); gate biases of the matrix memory spread so that its
running maximum moves both ways. ``sharpen`` makes one query token of the first layer score one key token far above all
others, so that whether that key is seen decides the output.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from roost_b200.weights.safetensors_io import write_safetensors
from tests.plain import nomivik_plain as P


def recurrence(width=12, blocks=3, conv=3):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def attention(heads=4, kv_heads=2, dim=8, vdim=6, rot=4, base=300.0, scale=0.5, window=9, softcap=7.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap, "mask": {"size": window},
            "rot": {"base": base, "dims": rot}}


def memory(heads=2, dim=6, vdim=10, gate_cap=9.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}


def parallel(left=None, right=None):
    return {"type": "parallel", "mixer": {"left": left or attention(), "right": right or memory()}}


def dense(ff=24):
    return {"kind": "dense", "ff": ff}


def config(layers, width=40, vocab=97, eps=1e-5, pairs=(53, 31, 5), side=6, loop=None):
    c = {"architecture": "Nomivik", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}
    if pairs is not None:
        c["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), pairs))}
    if side is not None:
        c["token_side"] = {"dim": side}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# Configurations. None uses the sizes of anyone's released model; they differ from one another in every size.
MIXED = config([(recurrence(), None), (parallel(), dense()), (parallel(attention(heads=3, kv_heads=1, dim=6, vdim=9, rot=6, scale=0.7, window=17, softcap=3.0),
                                                                       memory(heads=3, dim=5, vdim=4, gate_cap=4.0)), None),
                (recurrence(width=20, blocks=2, conv=4), dense(ff=18))], loop=(1, 3, 2))
# values that many models make equal or 1 differ here, and the other way round: as many key/value heads as query heads, keys
# and values of one size, a rotation as wide as the head, a window of one key, two taps, one block, one bucket, a multiplier
# of zero, a token input of one number, a parallel layer first, a feed-forward after a recurrence, no loop
ODD = config([(parallel(attention(heads=3, kv_heads=3, dim=10, vdim=10, rot=10, base=50.0, scale=0.3, window=1, softcap=50.0), memory(heads=1, dim=9, vdim=9, gate_cap=30.0)),
               dense(ff=31)),
              (recurrence(width=9, blocks=1, conv=2), dense(ff=10)),
              (parallel(attention(heads=6, kv_heads=2, dim=4, vdim=7, rot=2, base=50.0, scale=1.1, window=64, softcap=1.5), memory(heads=5, dim=3, vdim=2, gate_cap=1.0)), None),
              (recurrence(width=16, blocks=16, conv=5), None)], width=36, vocab=61, eps=1e-6, pairs=(1, 0, 3), side=1)
# sizes of whole vectors (multiples of 8 and 64), heads the tensor-core attention kernels serve, a loop of one layer run thrice
# that ends the model, windows that end inside and at the edge of a tile of keys
WIDE = config([(parallel(attention(heads=4, kv_heads=2, dim=64, vdim=64, rot=32, base=10000.0, scale=0.125, window=40, softcap=15.0), memory(heads=2, dim=32, vdim=64)), dense(ff=128)),
               (recurrence(width=128, blocks=4, conv=4), None),
               (parallel(attention(heads=4, kv_heads=1, dim=32, vdim=48, rot=32, base=10000.0, scale=0.2, window=32, softcap=30.0), memory(heads=4, dim=64, vdim=32, gate_cap=15.0)),
                dense(ff=64))],
              width=128, vocab=200, pairs=(211, 1000003, 999983), side=16, loop=(2, 3, 3))
# a loop that starts the model and covers all of it; large key heads of the matrix memory; a window longer than any prompt here
LOOPED = config([(parallel(attention(heads=2, kv_heads=1, dim=8, vdim=4, rot=8, window=1000), memory(heads=2, dim=40, vdim=8, gate_cap=6.0)), None),
                 (recurrence(width=10, blocks=5, conv=4), dense(ff=20))], width=24, vocab=50, pairs=(7, 3, 11), side=5, loop=(0, 2, 2))
CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "looped": LOOPED}


def tensor_shapes(cfg) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    L, sd = len(cfg["layers"]), cfg.get("token_side", {}).get("dim")
    shapes = {"embed": (V, W), "final.norm": (W,)}
    if "embedding" in cfg:
        shapes["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    if sd is not None:
        shapes["side.embed"] = (V, L * sd)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "rglru":
            C, B, K = m["width"], m["blocks"], m["conv"]
            shapes.update({p + "mix.y": (C, W), p + "mix.y.b": (C,), p + "mix.x": (C, W), p + "mix.x.b": (C,), p + "mix.conv": (C, K), p + "mix.conv.b": (C,),
                           p + "mix.ra": (B, C // B, C // B), p + "mix.ra.b": (B, C // B), p + "mix.ri": (B, C // B, C // B), p + "mix.ri.b": (B, C // B),
                           p + "mix.lam": (C,), p + "mix.o": (W, C)})
        else:
            a, r = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            shapes.update({q + "q": (H * d, W), q + "q.b": (H * d,), q + "k": (G * d, W), q + "k.b": (G * d,), q + "v": (G * dv, W), q + "v.b": (G * dv,),
                           q + "o": (W, H * dv), q + "out": (W,)})
            H, d, dv = r["heads"], r["dim"], r["vdim"]
            q = p + "mix.right."
            shapes.update({q + "q": (H * d, W), q + "k": (H * d, W), q + "v": (H * dv, W), q + "g": (H * dv, W), q + "o": (W, H * dv), q + "norm": (H * dv,),
                           q + "i": (H, W), q + "i.b": (H,), q + "f": (H, W), q + "f.b": (H,), q + "out": (W,)})
        f = layer["mlp"]
        if f is not None:
            shapes.update({p + "norm2": (W,), p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        if sd is not None:
            shapes.update({p + "side.gate": (sd, W), p + "side.proj": (W, sd), p + "side.norm": (W,)})
    return shapes


def draw_tensors(cfg, seed: int, std: float = 0.25) -> dict:
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        r = torch.randn(shape, generator=g)
        fan = (32.0 / max(shape[-1], 1)) ** 0.5
        if name.endswith("side.norm"):
            t = 0.3 + 0.1 * r                       # the token input is small beside the stream
        elif name.endswith("left.out") or name.endswith("right.out"):
            t = 0.5 + 0.15 * r
        elif "norm" in name:
            t = 1.0 + 0.1 * r
        elif name.endswith(".lam"):
            t = -6.0 + 4.0 * torch.rand(shape, generator=g)
        elif name.endswith("mix.conv"):
            t = 0.5 * r
        elif name.endswith("i.b") or name.endswith("f.b"):
            t = 1.5 * r
        elif name.endswith(".i") or name.endswith(".f"):
            t = 4.0 * std * r * fan                 # gates that move: the running maximum rises and decays
        elif name.endswith(".b"):
            t = 0.2 * r
        elif name in ("embed", "bigram", "side.embed"):
            t = r if name == "embed" else 0.5 * r
        elif name.endswith(".ra") or name.endswith(".ri"):
            t = 2.0 * std * r * fan
        elif name.endswith(".o") or name.endswith(".down"):
            t = std * r * fan
        else:
            t = 2.0 * std * r * fan
        out[name] = t.to(torch.bfloat16)
    return out


def sharpen(cfg, tensors: dict, key_token: int, query_token: int, value: float = 20.0, weight: float = 6.0) -> None:
    """Changes the attention of layer 0 (a parallel layer run first, whose rotation is narrower than its heads) so that
    ``query_token``'s queries point along ``key_token``'s keys in the elements the rotation leaves alone, whatever token stood
    before either: queries and keys of unit root mean square then meet with nearly the largest score there is, wherever the two
    tokens stand, and the key token's value is large. The key and the query come from the biases and the token's own embedding
    row; the hashed pair row is small beside them."""
    layer = cfg["layers"][0]
    assert layer["type"] == "parallel" and P.layer_order(cfg)[0][0] == 0
    m = layer["mixer"]["left"]
    H, G, d, rot = m["heads"], m["kv_heads"], m["dim"], m["rot"]["dims"]
    assert rot < d
    tensors["bigram"] = (0.05 * tensors["bigram"].float()).to(torch.bfloat16)
    # The value goes through one element of the stream that only the key token has (no other embedding row and no pair row
    # writes there): carried by a direction of the stream that other tokens share in part, the tokens that resemble the key
    # token would both score high and bring a like value, and the output would turn little when the key is lost.
    column = 0
    for name in ("embed", "bigram"):
        tensors[name][:, column] = 0.0
    tensors["embed"][key_token, column] = 4.0
    w = {k: v.double() for k, v in tensors.items()}
    x = P.rms_norm(w["embed"][[key_token, query_token]], w["l0.norm1"], cfg["norm"]["eps"])
    L = "l0.mix.left."
    keys = (x[0] @ w[L + "k"].T + w[L + "k.b"]).reshape(G, d)
    q = w[L + "q"].reshape(H, d, -1).clone()
    xq = x[1]
    for h in range(H):
        k = keys[h // (H // G)].clone()
        k[:rot] = 0.0
        q[h] = q[h] * 0.05 + torch.outer(k / k.norm(), xq) * (8.0 / float(xq @ xq))
    tensors[L + "q"] = q.reshape(w[L + "q"].shape).to(torch.bfloat16)
    tensors[L + "q.b"] = (0.05 * w[L + "q.b"]).to(torch.bfloat16)
    g = torch.Generator().manual_seed(key_token)
    direction = torch.randn(w[L + "v"].shape[0], generator=g, dtype=torch.float64)
    v = w[L + "v"].clone()
    v[:, column] = value * direction / direction.norm() / float(x[0][column])
    tensors[L + "v"] = v.to(torch.bfloat16)
    # the branches' outputs are normed before they are averaged, so a large value turns the attention's output without
    # lengthening it: the branch's weight is what makes it count in the stream
    tensors[L + "out"] = (weight * w[L + "out"]).to(torch.bfloat16)


def write_model(model_dir, cfg, tensors) -> Path:
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(model_dir / "model.safetensors", tensors, metadata={"format": "pt"})
    return model_dir


def plain_weights(tensors: dict) -> dict:
    """The stored bfloat16 values in float64."""
    return {k: v.double() for k, v in tensors.items()}
