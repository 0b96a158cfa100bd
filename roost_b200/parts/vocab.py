"""The two ends of a model: the token embedding and the head that turns final hidden states into logits.

``table``: h0[t, :] = table[ids[t], :], a bit-exact row copy with no scaling (src/Starlings.Roost.Ops/CpuOps.cs:441-458).
``linear``: logits[s, v] = sum_d final[s, d] W[v, d] in 32-bit whatever the activation dtype is, no soft cap
(src/Starlings.Roost.Ops/CpuOps.cs:465-495); with tied embeddings W is the embedding's table. An architecture that scales
its embeddings or caps its logits registers other kinds; the model only knows the two interfaces.
"""
from __future__ import annotations

import torch

from ..config.spec import EmbeddingSpec, HeadSpec
from .base import CacheNeed, Embedding, Head, ParamDecl, Runtime, register_embedding, register_head
from .linear import Linear


class TableEmbedding(Embedding):
    def __init__(self, spec: EmbeddingSpec, runtime: Runtime):
        if spec.vocab <= 0 or spec.hidden <= 0:
            raise ValueError("table embedding: vocab and hidden must be positive")
        self.spec, self.rt = spec, runtime
        self.table: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec: EmbeddingSpec):
        return {"table": ParamDecl(shape=(spec.vocab, spec.hidden))}

    def load(self, params):
        self.table = params["table"].to(self.rt.dtype).contiguous()

    def tied_weight(self):
        return self.table

    def __call__(self, ids, batch=None):
        return self.rt.kernels.embedding(self.table, ids)


class LinearHead(Head):
    def __init__(self, spec: HeadSpec, runtime: Runtime):
        self.spec, self.rt = spec, runtime
        self.linear = Linear(runtime, spec.vocab, spec.hidden)

    @classmethod
    def parameters(cls, spec: HeadSpec):
        return {"weight": ParamDecl(shape=(spec.vocab, spec.hidden))}

    def load(self, params):
        w = params["weight"]
        if w.dtype == self.rt.dtype and w.is_contiguous() and tuple(w.shape) == (self.spec.vocab, self.spec.hidden):
            self.linear.weight = w          # as it is: a tied head shares the embedding's memory
        else:
            self.linear.load(w)

    @property
    def weight(self):
        return self.linear.weight

    def __call__(self, final, batch=None):
        return self.linear(final, out_dtype=torch.float32)


class ScaledTableEmbedding(TableEmbedding):
    """h0[t, :] = table[ids[t], :] * scale as a float32 stream (the product is formed in 32-bit and not rounded)."""

    def __call__(self, ids, batch=None):
        return self.rt.kernels.embedding_scaled(self.table, ids, float(self.spec.scale))


class CappedLinearHead(LinearHead):
    """cap * tanh(logits / cap) on the 32-bit logits."""

    def __init__(self, spec, runtime: Runtime):
        super().__init__(spec, runtime)
        if not spec.cap > 0:
            raise ValueError(f"capped_linear: cap {spec.cap} must be positive")

    def __call__(self, final, batch=None):
        return self.rt.kernels.softcap_(self.linear(final, out_dtype=torch.float32), float(self.spec.cap))


class ScaledLinearHead(LinearHead):
    """logits * scale on the 32-bit logits."""

    def __call__(self, final, batch=None):
        logits = self.linear(final, out_dtype=torch.float32)
        return logits if self.spec.scale == 1.0 else self.rt.kernels.scale_(logits, float(self.spec.scale))


class PairHashedEmbedding(TableEmbedding):
    """h0[t, :] = table[id_t, :] + pairs[row_t, :] as a float32 stream, row_t = (id_(t-1) * mul_prev + id_t * mul_cur) mod
    buckets, and the row after the buckets for a request's first token. The token before a step's first token of a request
    is kept on the device, one int32 a request (a state group of the cache manager): the kernel reads it through the step's
    slot table and a second kernel stores the row's last token, so steps replay from graphs and a step started ahead of the
    host finds its predecessor's token where it left it."""
    state_capturable = True

    def __init__(self, spec, runtime: Runtime):
        super().__init__(spec, runtime)
        if spec.buckets <= 0 or spec.mul_prev < 0 or spec.mul_cur < 0:
            raise ValueError("pair_hashed_table: buckets must be positive and the multipliers not negative")
        self.pairs: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec):
        return {"table": ParamDecl(shape=(spec.vocab, spec.hidden)), "pairs": ParamDecl(shape=(spec.buckets + 1, spec.hidden))}

    def load(self, params):
        super().load(params)
        self.pairs = params["pairs"].to(self.rt.dtype).contiguous()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kind="state", state_shape=(1,), state_dtype=torch.int32)

    def __call__(self, ids, batch, cache=None):
        s, k = self.spec, self.rt.kernels
        slots = batch.groups[cache.group].state_slots
        out = k.pair_embedding(self.table, self.pairs, ids, batch.positions, batch.token_row, batch.q_indptr, slots, cache.state,
                               s.buckets, s.mul_prev, s.mul_cur)
        k.last_token_store(ids, batch.q_indptr, slots, cache.state)
        return out


register_embedding("pair_hashed_table", PairHashedEmbedding)
register_embedding("table", TableEmbedding)
register_embedding("scaled_table", ScaledTableEmbedding)
register_head("capped_linear", CappedLinearHead)
register_head("scaled_linear", ScaledLinearHead)
register_head("linear", LinearHead)
