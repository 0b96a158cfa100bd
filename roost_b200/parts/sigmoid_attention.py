"""Grouped-query causal attention whose weights are sigmoids of the scores, not a softmax over them.

Per step: one fused projection (rows [q heads | k heads | v heads | gate]); one kernel that divides every query and key head by
its root mean square and multiplies by the queries' or the keys' weight, multiplies the queries by the temperature of their
position, 1 + c ln(floor((p + 1) / every) + 1), writes them to a tensor of their own and the keys and values into the step's
page slots; attention of the step's queries over the pages, key j of query i weighing sigmoid((q_i . k_j) scale - slope_h (i - j)
+ b_h), the weighted sum of the values multiplied by sigmoid(gate) in the same kernel; the output projection. Scores, weights and
sums are 32-bit. A step of few rows deals a token's keys to several blocks whose partial sums a second kernel adds in order; a
bfloat16 step that brings prompt portions runs the same sums on the tensor cores (mma.sync), the 32-bit weights entering P V as two
bfloat16 operands.

The cache is a paged group: two planes (keys, values) when keys and values have one size, else one plane whose entries are
[key | value] of one key/value head.
"""
from __future__ import annotations

import torch

from ..config.spec import SigmoidAttentionSpec
from .base import CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear


class SigmoidAttention(Mixer):
    def __init__(self, spec: SigmoidAttentionSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim) <= 0:
            raise ValueError("sigmoid_attention: hidden, head counts, head_dim and v_dim must be positive")
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"sigmoid_attention: {s.num_heads} query heads are not a multiple of {s.num_kv_heads} key/value heads")
        if s.head_dim > 512 or s.v_dim > 512:
            raise ValueError(f"sigmoid_attention: heads of {s.head_dim} and values of {s.v_dim} numbers; the kernels serve up to 512")
        if not s.scale > 0 or not s.qk_norm_eps > 0:
            raise ValueError("sigmoid_attention: scale and the norm's eps must be positive")
        if s.temp_coef < 0 or (s.temp_coef and s.temp_every <= 0):
            raise ValueError("sigmoid_attention: the temperature's coefficient cannot be negative and its period must be positive")
        if s.slopes and len(s.slopes) != s.num_heads:
            raise ValueError(f"sigmoid_attention: {len(s.slopes)} slopes for {s.num_heads} heads")
        self.spec, self.rt = s, runtime
        self.q_width, self.k_width, self.v_width = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.v_dim
        self.gate_width = s.num_heads * s.v_dim if s.output_gate else 0
        self.qkv = Linear(runtime, self.q_width + self.k_width + self.v_width + self.gate_width, s.hidden)
        self.out = Linear(runtime, s.hidden, s.num_heads * s.v_dim)
        self.two_planes = s.head_dim == s.v_dim
        self.slopes = torch.tensor([float(v) for v in (s.slopes or (0.0,) * s.num_heads)], dtype=torch.float32, device=runtime.device)
        self.head_bias = torch.zeros(s.num_heads, dtype=torch.float32, device=runtime.device)
        self.q_weight = self.k_weight = None

    @classmethod
    def parameters(cls, spec: SigmoidAttentionSpec):
        s = spec
        Q, K, V = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.v_dim
        G = s.num_heads * s.v_dim if s.output_gate else 0
        decls = {"qkv": ParamDecl(shape=(Q + K + V + G, s.hidden), row_splits=(Q, K, V, G) if G else (Q, K, V)),
                 "out": ParamDecl(shape=(s.hidden, s.num_heads * s.v_dim)),
                 "q_norm": ParamDecl(shape=(s.head_dim,), role="vector"), "k_norm": ParamDecl(shape=(s.head_dim,), role="vector")}
        if s.head_bias:
            decls["head_bias"] = ParamDecl(shape=(s.num_heads,), role="vector", init=("normal", -2.0, 1.0))
        return decls

    def load(self, params):
        self.qkv.load(params["qkv"])
        self.out.load(params["out"])
        self.q_weight = params["q_norm"].float().contiguous()
        self.k_weight = params["k_norm"].float().contiguous()
        if self.spec.head_bias:
            self.head_bias = params["head_bias"].float().contiguous()

    def cache_need(self) -> CacheNeed:
        s = self.spec
        if self.two_planes:
            return CacheNeed(kind="paged", kv_heads=s.num_kv_heads, head_dim=s.head_dim, planes=2)
        return CacheNeed(kind="paged", kv_heads=s.num_kv_heads, head_dim=s.head_dim + s.v_dim, planes=1)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if not write_cache:
            raise ValueError("sigmoid_attention: a run cannot read another run's cache")
        tables = batch.groups[cache.group]
        qkv = self.qkv(x)
        q = k.sigmoid_attention_prepare(qkv, cache.k_pool, cache.v_pool, self.q_weight, self.k_weight, batch.positions, tables.slot_mapping,
                                        s.num_heads, s.num_kv_heads, s.head_dim, s.v_dim, s.qk_norm_eps, s.temp_coef, s.temp_every, cache.page_size)
        gate_col = self.q_width + self.k_width + self.v_width if s.output_gate else None
        # steps that bring prompt portions run on the tensor cores in bfloat16 where the sizes allow (a function of the step's size
        # and kind only, so a captured step keeps its way); steps that decode, float32 and other sizes run the 32-bit kernel
        portions = not batch.all_single and batch.num_tokens >= getattr(k, "SIGMOID_MMA_MIN_TOKENS", 1 << 30)
        o = k.sigmoid_attention(q, cache.k_pool, cache.v_pool, qkv, gate_col, self.slopes, self.head_bias, batch.positions, batch.token_row,
                                tables.kv_indptr, tables.kv_indices, s.num_kv_heads, s.v_dim, s.scale, kv_cap=batch.kv_cap,
                                **({"q_indptr": batch.q_indptr} if portions else {}))
        return self.out(o)


register_mixer("sigmoid_attention", SigmoidAttention)
