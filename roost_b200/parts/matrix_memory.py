"""A matrix memory a head with exponential gates (the mLSTM cell), as a mixer with a fixed-size state per request.

Per step: one projection gives a token's [q | k | v | g] (g: the output gate's argument, ``heads`` x ``v_dim`` wide), a second
the two gates' arguments a head as 32-bit sums; one kernel walks every (row, head) through its tokens with the head's matrix
in registers: i = c tanh((. + b) / c), f = logsigmoid(c tanh((. + b) / c)), m' = max(f + m, i), S <- exp(f + m - m') S +
exp(i - m') k v^T, n likewise with k alone, o = S^T q / (max(|n . q|, exp(-m')) + floor) with q scaled by 1 / sqrt(head_dim); one
kernel divides each head's o by its root mean square, multiplies by the weight and by sigmoid(g) and rounds once; then the
output projection. Gates, maxima, S, n and o are 32-bit.

A request's slot holds, head after head, [S: head_dim x v_dim | n: head_dim | m] as one float32 vector; the executor zeroes it
when the request's first token arrives (m starts at 0). The kernels read the step's device tables only, so steps are captured.
"""
from __future__ import annotations

import torch

from ..config.spec import MatrixMemorySpec
from .base import CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear


class MatrixMemory(Mixer):
    state_capturable = True

    def __init__(self, spec: MatrixMemorySpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.num_heads, s.head_dim, s.v_dim) <= 0 or not s.gate_cap > 0 or not s.eps > 0 or s.floor < 0:
            raise ValueError("matrix_memory: every size, the gates' cap and eps must be positive")
        if s.head_dim > 1024 or s.v_dim > 65535 * 32:
            raise ValueError(f"matrix_memory: heads of {s.head_dim} keys and {s.v_dim} values; the kernel keeps up to 1,024 keys a head")
        self.spec, self.rt = s, runtime
        self.qk_width, self.v_width = s.num_heads * s.head_dim, s.num_heads * s.v_dim
        self.head_state = s.head_dim * s.v_dim + s.head_dim + 1
        self.proj_in = Linear(runtime, 2 * self.qk_width + 2 * self.v_width, s.hidden)
        self.proj_gates = Linear(runtime, 2 * s.num_heads, s.hidden)
        self.out = Linear(runtime, s.hidden, self.v_width)
        self.weight = None

    @classmethod
    def parameters(cls, spec: MatrixMemorySpec):
        s = spec
        QK, V = s.num_heads * s.head_dim, s.num_heads * s.v_dim
        return {"in": ParamDecl(shape=(2 * QK + 2 * V, s.hidden), row_splits=(QK, QK, V, V)),
                "gates": ParamDecl(shape=(2 * s.num_heads, s.hidden), row_splits=(s.num_heads, s.num_heads)),
                "gates_bias": ParamDecl(shape=(2 * s.num_heads,), row_splits=(s.num_heads, s.num_heads), role="vector", init=("normal", 0.0, 1.0)),
                "norm": ParamDecl(shape=(V,), role="vector"), "out": ParamDecl(shape=(s.hidden, V))}

    def load(self, params):
        self.proj_in.load(params["in"])
        self.proj_gates.load(params["gates"], params["gates_bias"])
        self.out.load(params["out"])
        self.weight = params["norm"].float().contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(self.spec.num_heads * self.head_state,), state_dtype=torch.float32)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if not write_cache:
            raise ValueError("matrix_memory: a run cannot read another run's state")
        slots = batch.groups[cache.group].state_slots
        qkvg = self.proj_in(x)                                              # [T, q | k | v | g]
        gates = self.proj_gates(x, out_dtype=torch.float32)                 # [T, i of every head | f of every head], biases added
        o = k.matrix_memory_scan(qkvg, gates, cache.state, batch.q_indptr, slots, s.num_heads, s.head_dim, s.v_dim, s.gate_cap, s.floor)
        y = k.head_norm_gate(o, qkvg, 2 * self.qk_width + self.v_width, self.weight, s.num_heads, s.eps, self.rt.dtype)
        return self.out(y)


register_mixer("matrix_memory", MatrixMemory)
