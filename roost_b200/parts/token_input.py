"""What a layer adds to the residual stream from the token itself: a slice of a second embedding table, gated by the stream.

e = table[id] (``dim`` numbers: the layer's own columns of a table that all layers share in the checkpoint); g = gelu_tanh(W_gate x)
* e on the 32-bit values of the product; y = W_proj g; the addend is y / sqrt(mean(y^2) + eps) * w, formed in 32-bit and
rounded once to the activation dtype. x is the stream's value in the activation dtype.
"""
from __future__ import annotations

import torch

from ..config.spec import TokenInputSpec
from .base import ParamDecl, Runtime, TokenInput, register_token_input
from .linear import Linear


class GatedTokenInput(TokenInput):
    def __init__(self, spec: TokenInputSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.vocab, s.dim) <= 0 or s.eps <= 0:
            raise ValueError("gated_token_input: hidden, vocab, dim and eps must be positive")
        if s.column < 0 or s.column + s.dim > s.columns:
            raise ValueError(f"gated_token_input: columns {s.column} to {s.column + s.dim} lie outside a table of {s.columns}")
        self.spec, self.rt = s, runtime
        self.gate = Linear(runtime, s.dim, s.hidden)
        self.proj = Linear(runtime, s.hidden, s.dim)
        self.table = self.weight = None

    @classmethod
    def parameters(cls, spec: TokenInputSpec):
        s = spec
        return {"table": ParamDecl(shape=(s.vocab, s.dim), columns=(s.column, s.column + s.dim, s.columns)),
                "gate": ParamDecl(shape=(s.dim, s.hidden)), "proj": ParamDecl(shape=(s.hidden, s.dim)),
                "norm": ParamDecl(shape=(s.hidden,), role="vector")}

    def load(self, params):
        self.gate.load(params["gate"])
        self.proj.load(params["proj"])
        self.table = params["table"].to(self.rt.dtype).contiguous()
        self.weight = params["norm"].contiguous()

    def __call__(self, x, ids):
        k = self.rt.kernels
        g = k.gelu_mul_rows(self.gate(x), self.table, ids)          # gelu_tanh(gate) * table[id]
        return k.rms_norm(self.proj(g), self.weight, self.spec.eps)


register_token_input("gated_token_input", GatedTokenInput)
