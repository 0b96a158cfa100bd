"""A gated linear recurrence a channel behind a short convolution (the real-gated linear recurrent unit), as a mixer with a
fixed-size state per request.

Per step: one projection gives a token's [y | x] (with biases); one kernel runs the causal convolution over x (bias, no
activation), reading the taps before a row's first token from the request's state, and one moves the row's last ``conv_taps``
- 1 inputs into the state (the convolution kernels of the Mamba mixers, which take any channel range); a batched product over
the ``blocks`` parts of u gives the two gates' arguments as 32-bit sums; one kernel walks every (row, channel) through its
tokens: r = sigmoid(. + b), i = sigmoid(. + b), a = exp(-rate r softplus(lam)), S <- a S + sqrt(1 - a^2) i u, and writes
S gelu_tanh(y) rounded once; then the output projection. rate softplus(lam) is formed once at load. Gates, decays and the state
are 32-bit.

A request's slot holds [S: width | the convolution's last inputs] as one float32 vector; the executor zeroes it when the
request's first token arrives. The kernels read the step's device tables only, so steps are captured.
"""
from __future__ import annotations

import torch

from ..config.spec import GatedRecurrenceSpec
from .base import CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear, batched_linear_f32


class GatedRecurrence(Mixer):
    state_capturable = True

    def __init__(self, spec: GatedRecurrenceSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.width, s.blocks, s.conv_taps) <= 0 or not s.rate > 0:
            raise ValueError("gated_recurrence: every size and the rate must be positive")
        if s.width % s.blocks:
            raise ValueError(f"gated_recurrence: {s.width} channels do not divide into {s.blocks} equal blocks")
        if s.conv_taps > 16:
            raise ValueError(f"gated_recurrence: {s.conv_taps} taps are beyond 16, the most the convolution kernel serves")
        self.spec, self.rt = s, runtime
        self.block_width = s.width // s.blocks
        self.conv_offset = s.width                                  # where the convolution's inputs start in a slot
        self.state_size = s.width + (s.conv_taps - 1) * s.width
        self.proj_in = Linear(runtime, 2 * s.width, s.hidden)
        self.out = Linear(runtime, s.hidden, s.width)
        self.gates = self.gate_bias = self.conv = self.conv_bias = self.decay = None

    @classmethod
    def parameters(cls, spec: GatedRecurrenceSpec):
        s, bw = spec, spec.width // max(spec.blocks, 1)
        v = lambda *shape, init=None: ParamDecl(shape=shape, role="vector", init=init)
        # the random-weights mode draws a lam with which a state lives for tens to hundreds of tokens
        return {"in": ParamDecl(shape=(2 * s.width, s.hidden), row_splits=(s.width, s.width)),
                "in_bias": ParamDecl(shape=(2 * s.width,), row_splits=(s.width, s.width), role="vector", init=("normal", 0.0, 0.1)),
                "conv": v(s.width, s.conv_taps, init=("normal", 0.0, 0.4)), "conv_bias": v(s.width, init=("normal", 0.0, 0.1)),
                "recur_gate": ParamDecl(shape=(s.blocks, bw, bw)), "recur_gate_bias": v(s.blocks, bw, init=("normal", 0.0, 0.3)),
                "input_gate": ParamDecl(shape=(s.blocks, bw, bw)), "input_gate_bias": v(s.blocks, bw, init=("normal", 0.0, 0.3)),
                "lam": v(s.width, init=("uniform", -6.0, -2.0)), "out": ParamDecl(shape=(s.hidden, s.width))}

    def load(self, params):
        s = self.spec
        f = lambda name: params[name].float().contiguous()
        self.proj_in.load(params["in"], params["in_bias"])
        self.out.load(params["out"])
        self.conv, self.conv_bias = f("conv"), f("conv_bias")
        # per block the rows [recurrence gate | input gate]: one batched product gives both
        self.gates = torch.cat([params["recur_gate"], params["input_gate"]], dim=1).to(self.rt.dtype).contiguous()     # [blocks, 2 bw, bw]
        self.gate_bias = torch.cat([f("recur_gate_bias"), f("input_gate_bias")], dim=1).contiguous()                   # [blocks, 2 bw]
        self.decay = (float(s.rate) * torch.nn.functional.softplus(f("lam"))).contiguous()                             # -log a = decay * r

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(self.state_size,), state_dtype=torch.float32)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if not write_cache:
            raise ValueError("gated_recurrence: a run cannot read another run's state")
        slots = batch.groups[cache.group].state_slots
        yx = self.proj_in(x)                                                                  # [T, y | x]
        u = k.mamba2_conv(yx, s.width, s.width, self.conv, self.conv_bias, cache.state, self.conv_offset, batch.token_row, batch.q_indptr,
                          slots, activation="none")
        k.mamba2_conv_state(yx, s.width, s.width, s.conv_taps, cache.state, self.conv_offset, batch.q_indptr, slots)
        T = u.shape[0]
        gates = batched_linear_f32(self.rt, u.view(T, s.blocks, self.block_width).transpose(0, 1), self.gates)     # [blocks, T, 2 bw] float32
        g = k.gated_recurrence_scan(u, gates, yx, self.gate_bias, self.decay, cache.state, batch.q_indptr, slots, s.width, s.blocks)
        return self.out(g)


register_mixer("gated_recurrence", GatedRecurrence)
