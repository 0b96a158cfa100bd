"""RMS norm: y = x / sqrt(mean(x^2) + eps) * w with the weight as stored
(src/Starlings.Roost.Ops/CpuOps.cs:87-101), alone or fused with the residual sum that precedes it
(src/Starlings.Roost.Ops/CpuOps.Fused.cs:26-34). And the layer norm with weight and bias over a 32-bit stream."""
from __future__ import annotations

import torch

from ..config.spec import NormSpec
from .base import Norm, ParamDecl, Runtime, register_norm


class RmsNorm(Norm):
    def __init__(self, spec: NormSpec, runtime: Runtime):
        if spec.size <= 0 or spec.eps <= 0:
            raise ValueError(f"rms_norm: size {spec.size} and eps {spec.eps} must be positive")
        self.spec = spec
        self.rt = runtime
        self.weight: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec: NormSpec):
        return {"weight": ParamDecl(shape=(spec.size,), role="vector")}

    def load(self, params):
        self.weight = params["weight"].contiguous()
        if self.spec.weight_offset:     # a weight stored around zero: offset + w, formed once in 32-bit
            self.weight = (self.weight.float() + float(self.spec.weight_offset)).contiguous()

    def __call__(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return self.rt.kernels.rms_norm(x, self.weight, self.spec.eps, rows)

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor, rows: torch.Tensor | None = None):
        """Returns (norm(residual + x), residual + x); without ``rows`` the sum replaces ``residual`` in place."""
        out = self.rt.kernels.add_rms_norm(x, residual, self.weight, self.spec.eps, rows)
        return out, residual


class LayerNorm(Norm):
    """(x - mean) / sqrt(var + eps) * w + b over a 32-bit stream; the output has the activation dtype. ``add_norm`` adds a
    branch output (activation dtype) to the stream in 32-bit first: the stream is never rounded."""

    def __init__(self, spec: NormSpec, runtime: Runtime):
        if spec.size <= 0 or spec.eps <= 0:
            raise ValueError(f"layer_norm: size {spec.size} and eps {spec.eps} must be positive")
        self.spec = spec
        self.rt = runtime
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec: NormSpec):
        return {"weight": ParamDecl(shape=(spec.size,), role="vector"), "bias": ParamDecl(shape=(spec.size,), role="vector", init=("normal", 0.0, 0.05))}

    def load(self, params):
        self.weight = params["weight"].float().contiguous()
        self.bias = params["bias"].float().contiguous()

    def __call__(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return self.rt.kernels.layer_norm(x, self.weight, self.bias, self.spec.eps, self.rt.dtype, None, rows)

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor, rows: torch.Tensor | None = None):
        """Returns (norm(residual + x), residual + x); without ``rows`` the sum replaces ``residual`` in place."""
        out = self.rt.kernels.layer_norm(residual, self.weight, self.bias, self.spec.eps, self.rt.dtype, x, rows)
        return out, residual


class WideRmsNorm(Norm):
    """x / sqrt(mean(x^2) + eps) * w over a 32-bit stream; the output has the activation dtype. ``add_norm`` adds a branch
    output (activation dtype) to the stream in 32-bit first, and with ``extra`` a second 32-bit addend (the embedding's output
    added again): the stream is never rounded. ``add_only`` makes the sums and hands the stream's value on in the activation
    dtype without a norm (for a part that reads the stream itself)."""

    def __init__(self, spec: NormSpec, runtime: Runtime):
        if spec.size <= 0 or spec.eps <= 0:
            raise ValueError(f"rms_norm_wide: size {spec.size} and eps {spec.eps} must be positive")
        self.spec = spec
        self.rt = runtime
        self.weight: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec: NormSpec):
        return {"weight": ParamDecl(shape=(spec.size,), role="vector")}

    def load(self, params):
        self.weight = (params["weight"].float() + float(self.spec.weight_offset)).contiguous()

    def __call__(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return self.rt.kernels.wide_rms_norm(x, self.weight, self.spec.eps, self.rt.dtype, None, None, rows)

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor, rows: torch.Tensor | None = None, extra: torch.Tensor | None = None,
                 gate: tuple | None = None):
        """Returns (norm(residual + x [+ extra]), the sum); without ``rows`` the sum replaces ``residual`` in place. ``gate``
        (arguments: float32 like x, bias: float32 [hidden]): x is multiplied by sigmoid(arguments + bias) before it is added."""
        if gate is not None:
            if extra is not None:
                raise ValueError("rms_norm_wide: a gated sum takes no second addend")
            return self.rt.kernels.wide_rms_norm_gated(residual, self.weight, self.spec.eps, self.rt.dtype, x, gate[0], gate[1], rows), residual
        return self.rt.kernels.wide_rms_norm(residual, self.weight, self.spec.eps, self.rt.dtype, x, extra, rows), residual

    def add_only(self, x: torch.Tensor, residual: torch.Tensor):
        """Returns (residual + x in the activation dtype, the sum, which replaces ``residual`` in place)."""
        return self.rt.kernels.wide_rms_norm(residual, None, self.spec.eps, self.rt.dtype, x, None, None), residual


register_norm("rms_norm_wide", WideRmsNorm)
register_norm("rms_norm", RmsNorm)
register_norm("layer_norm", LayerNorm)
