"""Hyper-connections: the residual as several 32-bit streams that every sublayer reads as a weighted sum and writes back to
through a mixing matrix.

With streams x_1 .. x_S (all equal to the embedding at the start), a sublayer f with norm n does
    u = sum_s in[s] x_s;  y = f(n(u));  x_t <- sum_s mix[s, t] x_s + out[t] y   (every stream from the old ones)
and the model's output is the sum of the streams. One kernel does a write-back and the next read together: it applies the
pending (mix, out, y) of the sublayer before, forms u for the sublayer ahead and norms it, so the streams make one trip
through memory a sublayer. Everything is 32-bit; only the normed read is rounded to the activation dtype. Without learned
weights (in, mix and out all ones, one stream) this is the plain residual sum.
"""
from __future__ import annotations

import torch

from ..config.spec import ConnectionSpec, GatedResidualSpec
from .base import Connection, ParamDecl, Runtime, register_connection
from .linear import Linear

MAX_STREAMS = 8     # the kernel keeps a channel's streams in registers


class HyperConnection(Connection):
    def __init__(self, spec: ConnectionSpec, runtime: Runtime):
        if not 1 <= spec.streams <= MAX_STREAMS:
            raise ValueError(f"hyper_connection: {spec.streams} streams; the kernel serves 1 to {MAX_STREAMS}")
        if not spec.learned and spec.streams != 1:
            raise ValueError("hyper_connection: several streams need learned weights")
        self.spec = spec
        self.rt = runtime
        self.read = self.mix = self.write = None      # float32 [S], [S, S] indexed [from, to], [S]
        if not spec.learned:
            self.load({})

    @classmethod
    def parameters(cls, spec: ConnectionSpec):
        if not spec.learned:
            return {}
        S = spec.streams
        v = lambda *shape, init: ParamDecl(shape=shape, role="vector", init=init)
        return {"in": v(S, init=("normal", 1.0 / S, 0.1 / S)), "out": v(S, init=("normal", 1.0, 0.1)), "mix": v(S, S, init=("eye_normal", 1.0, 0.05))}

    def load(self, params):
        S = self.spec.streams
        if not self.spec.learned:
            ones = lambda *shape: torch.ones(shape, dtype=torch.float32, device=self.rt.device)
            self.read, self.mix, self.write = ones(S), ones(S, S), ones(S)
            return
        f = lambda name: params[name].float().contiguous()
        self.read, self.mix, self.write = f("in"), f("mix"), f("out")


register_connection("hyper_connection", HyperConnection)


class SigmoidGate(Connection):
    """x <- x + y sigmoid(W h + b): a sublayer's output y scaled element by element by a gate made from the sublayer's own input h.
    ``arguments(h)`` gives W h as 32-bit sums; the bias, the sigmoid and the product with y belong to the kernel that adds y to the
    32-bit residual (the next norm's), so the gated output is never rounded on its own."""

    def __init__(self, spec: GatedResidualSpec, runtime: Runtime):
        if spec.hidden <= 0:
            raise ValueError("sigmoid_gate: hidden must be positive")
        self.spec, self.rt = spec, runtime
        self.linear = Linear(runtime, spec.hidden, spec.hidden)
        self.bias = None

    @classmethod
    def parameters(cls, spec: GatedResidualSpec):
        return {"gate": ParamDecl(shape=(spec.hidden, spec.hidden)), "gate_bias": ParamDecl(shape=(spec.hidden,), role="vector", init=("normal", 0.0, 0.5))}

    def load(self, params):
        self.linear.load(params["gate"])
        self.bias = params["gate_bias"].float().contiguous()

    def arguments(self, h: torch.Tensor) -> torch.Tensor:
        return self.linear(h, out_dtype=torch.float32)


register_connection("sigmoid_gate", SigmoidGate)
