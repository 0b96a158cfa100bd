"""Grouped-query causal attention with a sink in the softmax, unit-norm queries and keys, and values of their own size.

Per step: one fused q/k/v projection (rows [q heads | k heads | v heads], with a bias where the spec says so); one kernel that
rotates the query and key heads (interleaved pairs or split halves, as the position encoding says; angles formed in double
precision), divides each by its root mean square over the head (no weight), writes the query back in place and the key and
value into the step's page slots; attention of the step's queries over the pages with p_j = exp(s_j) / (1 + sum exp(s_j)) (with
``sink``; the plain softmax without), scores and weights in 32-bit, over every earlier key or the last ``window`` (the cache
group then gives back the pages the window has passed), a score s becoming c tanh(s / c) with ``softcap`` c; the output projection
over the concatenated heads.

The cache is a paged group. When keys and values have the same size it has two planes (keys, values), the layout of the
framework's tensor-core attention kernels, which then serve the bfloat16 steps with the sink added at their end; otherwise it
has one plane whose entries are [key | value] of one key/value head, and the 32-bit kernel, which takes any sizes, reads that.
On the tensor cores the 32-bit softmax weights enter P V as two bfloat16 operands, their rounding and what it left over (16 bits
of the weights), which the mma.sync kernels serve; the denominator is summed from the 32-bit weights.
"""
from __future__ import annotations

import numpy as np
import torch

from ..config.spec import SinkAttentionSpec
from .attention_work import AttentionPlan, attention_caps, attention_work
from .base import POSITIONS, CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear

SHORT_ROW_TOKENS = 16   # rows of at most this many tokens may go to the split decode kernel


class SinkAttention(Mixer):
    def __init__(self, spec: SinkAttentionSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim) <= 0:
            raise ValueError("sink_attention: hidden, head counts, head_dim and v_dim must be positive")
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"sink_attention: {s.num_heads} query heads are not a multiple of {s.num_kv_heads} key/value heads")
        if s.head_dim > 512 or s.v_dim > 512:
            raise ValueError(f"sink_attention: heads of {s.head_dim} and values of {s.v_dim} numbers; the kernels serve up to 512")
        if s.scale <= 0:
            raise ValueError(f"sink_attention: scale {s.scale} must be positive")
        if s.unit_norm_eps is not None and s.unit_norm_eps <= 0:
            raise ValueError(f"sink_attention: the unit norm's eps {s.unit_norm_eps} must be positive")
        self.spec = s
        self.rt = runtime
        self.q_width, self.k_width, self.v_width = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.v_dim
        self.qkv = Linear(runtime, self.q_width + self.k_width + self.v_width, s.hidden)
        self.out = Linear(runtime, s.hidden, s.num_heads * s.v_dim)
        self.position = POSITIONS.build(s.position, runtime) if s.position is not None else None
        if self.position is not None and self.position.rotation()[1]:
            if getattr(self.position, "pairing", None) not in ("interleaved", "halves"):
                raise ValueError(f"sink_attention: the kernel rotates interleaved pairs or split halves; position encoding '{s.position.kind}' pairs otherwise")
            if self.position.rotation()[1] > s.head_dim:
                raise ValueError("sink_attention: the rotation is wider than a head")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"sink_attention: a window of {s.window} keys must be positive")
        if s.softcap < 0:
            raise ValueError(f"sink_attention: the scores' cap {s.softcap} cannot be negative")
        self.halves = self.position is not None and getattr(self.position, "pairing", None) == "halves"
        self.two_planes = s.head_dim == s.v_dim

    @classmethod
    def parameters(cls, spec: SinkAttentionSpec):
        Q, K, V = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim, spec.num_kv_heads * spec.v_dim
        decls = {"qkv": ParamDecl(shape=(Q + K + V, spec.hidden), row_splits=(Q, K, V)), "out": ParamDecl(shape=(spec.hidden, spec.num_heads * spec.v_dim))}
        if spec.bias:
            decls["qkv_bias"] = ParamDecl(shape=(Q + K + V,), row_splits=(Q, K, V), role="vector", init=("normal", 0.0, 0.1))
        return decls

    def load(self, params):
        self.qkv.load(params["qkv"], params["qkv_bias"] if self.spec.bias else None)
        self.out.load(params["out"])

    def cache_need(self) -> CacheNeed:
        s = self.spec
        if self.two_planes:
            return CacheNeed(kind="paged", kv_heads=s.num_kv_heads, head_dim=s.head_dim, planes=2, window=s.window)
        return CacheNeed(kind="paged", kv_heads=s.num_kv_heads, head_dim=s.head_dim + s.v_dim, planes=1, window=s.window)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if not write_cache:
            raise ValueError("sink_attention: a run cannot read another run's cache")
        tables = batch.groups[cache.group]
        inv_freq, rotary_dim = self.position.rotation() if self.position is not None else (None, 0)
        qkv = self.qkv(x)
        # Of the tensor-core kernels only the prompt kernels know a cap on the scores: a capped model runs them in steps all of whose
        # rows are prompt portions (no row of SHORT_ROW_TOKENS tokens or fewer: the step's class, so a captured step keeps its way),
        # and the 32-bit kernel in steps that decode.
        capped_ok = not s.softcap or (getattr(k, "attention_mma_softcap", False) and batch.row_counts
                                      and not any(n <= SHORT_ROW_TOKENS for n in batch.row_counts))
        tensor_cores = (self.two_planes and qkv.dtype == torch.bfloat16 and capped_ok and getattr(k, "attention_mma_sink", False)
                        and getattr(k, "attention_mma_supported", lambda d: False)(s.head_dim))
        q = torch.empty((qkv.shape[0], s.num_heads, s.head_dim), dtype=qkv.dtype, device=qkv.device) if tensor_cores else None
        k.sink_attention_prepare(qkv, cache.k_pool, cache.v_pool, inv_freq, rotary_dim, batch.positions, tables.slot_mapping, s.num_heads,
                                 s.num_kv_heads, s.head_dim, s.v_dim, s.unit_norm_eps, cache.page_size, **({"q_out": q} if tensor_cores else {}),
                                 **({"halves": True} if self.halves else {}))
        if tensor_cores:
            o = self._attend_tensor_cores(q, batch, cache, tables)
        else:
            o = k.sink_attention(qkv, cache.k_pool, cache.v_pool, batch.positions, batch.token_row, tables.kv_indptr, tables.kv_indices,
                                 s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim, s.scale, s.sink, kv_cap=batch.kv_cap,
                                 **({"window": s.window} if s.window is not None else {}), **({"softcap": s.softcap} if s.softcap else {}))
        return self.out(o)

    # ---- bfloat16 with keys and values of one size: the framework's tensor-core kernels, with the sink
    def _attend_tensor_cores(self, q, batch, cache, tables):
        s, k = self.spec, self.rt.kernels
        group = s.num_heads // s.num_kv_heads
        tile_rows = k.attention_prefill_tile_rows(s.num_heads, cache.k_pool, cache.v_pool, batch.num_tokens * group, tensor_memory=False)
        split_for = getattr(k, "decode_split_for", None)
        chunk, cluster = split_for(batch.num_rows, batch.kv_cap, cache.k_pool, cache.v_pool) if split_for and batch.kv_cap else (k.decode_chunk, 0)
        plan = batch.step_work(self, ("sink_attention", group, s.window, chunk, tile_rows, cluster))
        return k.attention_mma(q, cache.k_pool, cache.v_pool, batch.q_indptr, batch.kv_lens, tables.kv_indptr, tables.kv_indices, plan,
                               s.scale, s.window, sink=s.sink, wide_weights=True, **({"softcap": s.softcap} if s.softcap else {}))

    def step_class(self, row_counts):
        return ("short_rows", any(n <= SHORT_ROW_TOKENS for n in row_counts))

    def step_work_arrays(self, key, row_starts, row_counts):
        _, group, window, chunk, tile_rows, cluster = key
        prefill, decode, merge, _ = attention_work(row_starts, row_counts, group, window, chunk, tile_rows, cluster)
        return [np.asarray(prefill, np.int32), np.asarray(decode, np.int32), np.asarray(merge, np.int32)]

    def step_work_caps(self, key, num_tokens, num_rows, kv_cap, step_class):
        _, group, _, chunk, tile_rows, cluster = key
        short = dict([step_class[i : i + 2] for i in range(0, len(step_class), 2)]).get("short_rows", True)
        pc, dc, mc = attention_caps(num_tokens, num_rows, kv_cap, group, chunk, tile_rows, short, cluster)
        return [(pc * 2, -1), (dc * 4, -1), (mc * 4, -1)]

    def step_work_bind(self, key, tensors, host_arrays=None, captured=None):
        _, group, _, _, tile_rows, cluster = key
        prefill, decode, merge = tensors
        if captured is not None:
            num_tokens, num_rows, kv_cap, step_class = captured
            (pc, _), (dc, _), (mc, _) = self.step_work_caps(key, num_tokens, num_rows, kv_cap, step_class)
            return AttentionPlan(prefill_items=pc // 2, prefill_tile_rows=tile_rows, decode_items=dc // 4, merge_items=mc // 4,
                                 slots=0 if cluster else dc // 4, cluster_chunks=cluster,
                                 merge_rows=min(16, group) if num_tokens == num_rows else 16, prefill_work=prefill, decode_work=decode,
                                 merge_work=merge)
        hp, hd, hm = host_arrays
        slots = 0 if cluster else int((hd[3::4] >= 0).sum())
        return AttentionPlan(prefill_items=hp.size // 2, prefill_tile_rows=tile_rows, decode_items=hd.size // 4, merge_items=hm.size // 4,
                             slots=slots, cluster_chunks=cluster, merge_rows=int((hm[2::4] >> 24).max()) if hm.size else 1, prefill_work=prefill,
                             decode_work=decode, merge_work=merge)


register_mixer("sink_attention", SinkAttention)
