"""Retention: a matrix state a head that fades by a constant factor a token, as a mixer with a fixed-size state per request.

Per step: one projection gives a token's [q | k | v | g] (g: the output gate's argument, ``heads`` x ``v_dim`` wide); one kernel
turns the first ``rotary_dim`` elements of every query and key head in pairs (i, i + rotary_dim / 2) by position x frequency
(angles formed in double), multiplies the keys by head_dim^(-1/2) and leaves both as 32-bit numbers: what enters the recurrence is
not rounded to the activation dtype; one kernel walks every (row, head) through its tokens with the head's matrix in registers,
S <- decay_h S + k v^T, o = S^T q; one kernel divides each head's o by its root mean square (no weight), multiplies by
g sigmoid(g) and rounds once; then the output projection. Steps of many tokens cut their rows into chunks that run side by side.

A request's slot holds S [heads, head_dim, v_dim] as one float32 vector; the executor zeroes it when the request's first token
arrives. The kernels read the step's device tables only, so steps are captured.
"""
from __future__ import annotations

import torch

from ..config.spec import RetentionSpec
from .base import POSITIONS, CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear


class Retention(Mixer):
    state_capturable = True

    def __init__(self, spec: RetentionSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.num_heads, s.head_dim, s.v_dim) <= 0 or not s.eps > 0:
            raise ValueError("retention: every size and eps must be positive")
        if len(s.decay) != s.num_heads or not all(0.0 <= float(d) <= 1.0 for d in s.decay):
            raise ValueError(f"retention: {s.num_heads} heads need as many decays between 0 and 1; got {list(s.decay)}")
        if s.head_dim > 1024:
            raise ValueError(f"retention: heads of {s.head_dim} keys; the kernel keeps up to 1,024 keys a head")
        self.spec, self.rt = s, runtime
        self.qk_width, self.v_width = s.num_heads * s.head_dim, s.num_heads * s.v_dim
        self.proj_in = Linear(runtime, 2 * self.qk_width + 2 * self.v_width, s.hidden)
        self.out = Linear(runtime, s.hidden, self.v_width)
        self.position = POSITIONS.build(s.position, runtime) if s.position is not None else None
        if self.position is not None and self.position.rotation()[1]:
            if getattr(self.position, "pairing", None) != "halves":
                raise ValueError(f"retention: the kernel rotates split halves; position encoding '{s.position.kind}' pairs otherwise")
            if self.position.rotation()[1] > s.head_dim:
                raise ValueError("retention: the rotation is wider than a head")
        self.decay = torch.tensor([float(d) for d in s.decay], dtype=torch.float32, device=runtime.device)

    @classmethod
    def parameters(cls, spec: RetentionSpec):
        s = spec
        QK, V = s.num_heads * s.head_dim, s.num_heads * s.v_dim
        return {"in": ParamDecl(shape=(2 * QK + 2 * V, s.hidden), row_splits=(QK, QK, V, V)), "out": ParamDecl(shape=(s.hidden, V))}

    def load(self, params):
        self.proj_in.load(params["in"])
        self.out.load(params["out"])

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(kind="state", state_shape=(s.num_heads * s.head_dim * s.v_dim,), state_dtype=torch.float32)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if not write_cache:
            raise ValueError("retention: a run cannot read another run's state")
        slots = batch.groups[cache.group].state_slots
        inv_freq, rotary_dim = self.position.rotation() if self.position is not None else (None, 0)
        qkvg = self.proj_in(x)                                              # [T, q | k | v | g]
        qk = k.retention_prepare(qkvg, inv_freq, rotary_dim, batch.positions, s.num_heads, s.head_dim, float(s.head_dim) ** -0.5)
        o = k.retention_scan(qk, qkvg, 2 * self.qk_width, cache.state, self.decay, batch.q_indptr, slots, s.num_heads, s.head_dim, s.v_dim)
        y = k.head_norm_gate(o, qkvg, 2 * self.qk_width + self.v_width, None, s.num_heads, s.eps, self.rt.dtype, gate="silu")
        return self.out(y)


register_mixer("retention", Retention)
