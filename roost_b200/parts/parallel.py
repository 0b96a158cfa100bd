"""Several mixers side by side over one input: the result is the mean of their outputs, each divided by its root mean square
over the model width and multiplied by a weight of its own (one kernel, 32-bit, rounded once).

The branches are mixers of any registered kind, built from their own specs; each keeps the cache or state its kind asks for
(``cache_need`` returns one entry a branch and the call gets the views in the same order), and each makes the per-step work
lists its kernels want. Parameters are declared under the branch's index: "0.qkv", "1.in", ..., and "weight.<i>".
"""
from __future__ import annotations

import torch

from ..config.spec import ParallelMixerSpec
from .base import MIXERS, Mixer, ParamDecl, Runtime, register_mixer

MAX_BRANCHES = 4     # what the combining kernel takes


class ParallelMixer(Mixer):
    def __init__(self, spec: ParallelMixerSpec, runtime: Runtime):
        if not 1 <= len(spec.branches) <= MAX_BRANCHES:
            raise ValueError(f"parallel: {len(spec.branches)} branches; the combining kernel takes 1 to {MAX_BRANCHES}")
        if spec.hidden <= 0 or not spec.eps > 0:
            raise ValueError("parallel: hidden and eps must be positive")
        self.spec, self.rt = spec, runtime
        self.branches = [MIXERS.build(b, runtime) for b in spec.branches]
        self.weights: list = []
        self.state_capturable = all(getattr(b, "state_capturable", False) or (b.cache_need() is None or b.cache_need().kind != "state")
                                    for b in self.branches)
        self.capturable = all(getattr(b, "capturable", True) for b in self.branches)

    @classmethod
    def parameters(cls, spec: ParallelMixerSpec):
        out = {}
        for i, b in enumerate(spec.branches):
            for name, decl in MIXERS.get(b.kind).parameters(b).items():
                out[f"{i}.{name}"] = decl
            out[f"weight.{i}"] = ParamDecl(shape=(spec.hidden,), role="vector")
        return out

    def load(self, params):
        self.weights = []
        for i, b in enumerate(self.branches):
            b.load({name[len(f"{i}."):]: t for name, t in params.items() if name.startswith(f"{i}.")})
            self.weights.append(params[f"weight.{i}"].float().contiguous())

    def cache_need(self) -> tuple:
        return tuple(b.cache_need() for b in self.branches)

    def step_class(self, row_counts):
        return tuple(x for b in self.branches for x in (b.step_class(row_counts) if hasattr(b, "step_class") else ()))

    def __call__(self, x, batch, cache, write_cache: bool = True):
        outs = [b(x, batch, c, write_cache) for b, c in zip(self.branches, cache)]
        return self.rt.kernels.normed_mean(outs, self.weights, self.spec.eps)


register_mixer("parallel", ParallelMixer)
