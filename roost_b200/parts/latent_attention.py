"""Latent attention over the paged cache, as a mixer.

A token's cache entry is one vector: its latent c (``kv_rank`` numbers: the down projection divided by its root mean
square, times a weight) followed by one rotated key part of ``rope_dim`` numbers that all heads share. Head h's key is
[W_uk,h c | shared part], its value W_uv,h c, its query [q_plain | q_rot]. Since q_plain . (W_uk,h c) = (W_uk,h^T q_plain) . c
and sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j, the step runs in the latent space: every head's query is carried into
it by one batched product, the attention kernel reads each cached vector once for all heads (as key, and its first
``kv_rank`` numbers as value), and a second batched product carries the heads' sums out again. Scores, softmax and
sums are 32-bit.

Per step: the q projection (and, for a run that makes its own latent, the down projection); one kernel that divides
the latent by its root mean square, rotates the shared key part and every head's rotated query part and writes the
cache entry; the batched product into the latent space; attention; the batched product out of it; the output
projection. A run that reads another run's cache makes no latent and writes nothing; its window may differ from the
owner's (the cache is kept for the widest). With ``rope_dim`` 0 keys and queries have no rotated part: nothing is rotated and the
cache entry is the latent alone. With ``head_gate`` one more small projection gives a number a token and head, and a kernel
multiplies every head's output by its sigmoid before the output projection. bfloat16 steps of prompt portions of such a run (no
rotated part, no window) carry the rows' cached latents out to keys and values a head (a gather and two products) and attend there
on the tensor cores: a prompt needs a quarter of the products that way when the latent is four times as wide as a head.
"""
from __future__ import annotations

import torch

from ..config.spec import LatentAttentionSpec
from .base import POSITIONS, CacheNeed, Mixer, ParamDecl, Runtime, register_mixer
from .linear import Linear, batched_linear


class LatentAttention(Mixer):
    def __init__(self, spec: LatentAttentionSpec, runtime: Runtime):
        s = spec
        if min(s.hidden, s.num_heads, s.nope_dim, s.v_dim, s.kv_rank) <= 0 or s.rope_dim < 0:
            raise ValueError("latent_attention: hidden, heads, nope_dim, v_dim and kv_rank must be positive and rope_dim not negative")
        if s.kv_rank + s.rope_dim > 1024:
            raise ValueError(f"latent_attention: a cache entry of {s.kv_rank + s.rope_dim} numbers is beyond 1024, the largest the kernel serves")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"latent_attention: window {s.window} must be positive")
        if s.cache_window is not None and (s.window is None or s.window > s.cache_window):
            raise ValueError(f"latent_attention: the window {s.window} reaches beyond what the cache keeps ({s.cache_window})")
        if s.scale <= 0:
            raise ValueError(f"latent_attention: scale {s.scale} must be positive")
        if s.rope_dim and (s.position is None or s.position.rotary_dim > s.rope_dim):
            raise ValueError("latent_attention: a rotation of at most rope_dim elements is needed")
        if not s.rope_dim and s.position is not None and s.position.kind != "none":
            raise ValueError("latent_attention: keys without a rotated part take no position encoding")
        self.spec = s
        self.rt = runtime
        self.q_head = s.nope_dim + s.rope_dim
        self.entry = s.kv_rank + s.rope_dim
        self.q = Linear(runtime, s.num_heads * self.q_head, s.hidden)
        self.down = Linear(runtime, self.entry, s.hidden) if s.own_latent else None
        self.out = Linear(runtime, s.hidden, s.num_heads * s.v_dim)
        self.position = POSITIONS.build(s.position, runtime) if s.rope_dim else None
        self.head_gate = Linear(runtime, s.num_heads, s.hidden) if s.head_gate else None
        # Prompt portions of a run without a rotated part and without a window may leave the latent space: the rows' cached latents
        # are carried out to keys and values a head by two products, and the attention runs over those, a quarter of the products
        # the latent space costs when the latent is four times as wide as a head. Decode steps stay in the latent space, where the
        # cache is read once for all heads.
        self.carried = (s.rope_dim == 0 and s.window is None and s.own_latent and not runtime.full_precision and runtime.kernels is not None
                        and getattr(runtime.kernels, "carried_attention_supported", lambda d, v: False)(s.nope_dim, s.v_dim))
        self.key_full = Linear(runtime, s.num_heads * s.nope_dim, s.kv_rank) if self.carried else None
        self.value_full = Linear(runtime, s.num_heads * s.v_dim, s.kv_rank) if self.carried else None
        self.carried_min_tokens = 128        # tokens of a step from which its prompt portions are worth the two products
        self.carried_max_entries = 16384     # rows x the bound on their lengths up to which the carried keys and values are made
        self.key_up: torch.Tensor | None = None      # [heads, kv_rank, nope_dim]: W_uk,h^T as a weight stored [out, in]
        self.value_up: torch.Tensor | None = None    # [heads, v_dim, kv_rank]
        self.latent_weight: torch.Tensor | None = None

    @classmethod
    def parameters(cls, spec: LatentAttentionSpec):
        s = spec
        p = {"q": ParamDecl(shape=(s.num_heads * (s.nope_dim + s.rope_dim), s.hidden)),
             "uk": ParamDecl(shape=(s.num_heads * s.nope_dim, s.kv_rank)), "uv": ParamDecl(shape=(s.num_heads * s.v_dim, s.kv_rank)),
             "out": ParamDecl(shape=(s.hidden, s.num_heads * s.v_dim))}
        if s.head_gate:
            p["head_gate"] = ParamDecl(shape=(s.num_heads, s.hidden))
        if s.own_latent:
            p["dkv"] = ParamDecl(shape=(s.kv_rank + s.rope_dim, s.hidden))
            p["latent_norm"] = ParamDecl(shape=(s.kv_rank,), role="vector")
        return p

    def load(self, params):
        s = self.spec
        self.q.load(params["q"])
        self.out.load(params["out"])
        self.key_up = params["uk"].to(self.rt.dtype).reshape(s.num_heads, s.nope_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.value_up = params["uv"].to(self.rt.dtype).reshape(s.num_heads, s.v_dim, s.kv_rank).contiguous()
        if s.head_gate:
            self.head_gate.load(params["head_gate"])
        if self.carried:
            self.key_full.load(params["uk"])
            self.value_full.load(params["uv"])
        if s.own_latent:
            self.down.load(params["dkv"])
            self.latent_weight = params["latent_norm"].float().contiguous()

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(kind="paged", kv_heads=1, head_dim=self.entry, window=s.cache_window, planes=1)

    def __call__(self, x, batch, cache, write_cache: bool = True):
        s, k = self.spec, self.rt.kernels
        if write_cache != s.own_latent:
            raise ValueError("latent_attention: a run writes the cache exactly when it makes its own latent")
        tables = batch.groups[cache.group]
        T, H = x.shape[0], s.num_heads
        inv_freq, rotary_dim = self.position.rotation() if self.position is not None else (None, 0)
        q = self.q(x)                                                       # [T, H * (nope + rope)]
        down = self.down(x) if s.own_latent else None                       # [T, kv_rank + rope]
        k.latent_prepare(q, down, cache.k_pool, self.latent_weight, inv_freq, rotary_dim, batch.positions,
                         tables.slot_mapping if s.own_latent else None, H, s.nope_dim, s.rope_dim, s.kv_rank, s.latent_eps, cache.page_size)
        if (self.carried and not batch.all_single and T >= self.carried_min_tokens and batch.kv_cap
                and batch.num_rows * batch.kv_cap <= self.carried_max_entries):
            # a function of the step's sizes and kind only, so a captured step keeps its way
            latents = k.latent_gather(cache.k_pool, batch.kv_lens, tables.kv_indptr, tables.kv_indices, batch.num_rows, batch.kv_cap)
            o = k.carried_attention(q, self.key_full(latents), self.value_full(latents), batch.positions, batch.q_indptr, H, s.nope_dim, s.v_dim,
                                    batch.kv_cap, s.scale)
            if s.head_gate:
                k.head_gate_mul_(o, self.head_gate(x), 0, H)
            return self.out(o)
        q_heads = q.view(T, H, self.q_head).transpose(0, 1)                 # [H, T, nope + rope], a view
        q_latent = torch.empty((H, T, s.kv_rank), dtype=q.dtype, device=q.device)
        batched_linear(self.rt, q_heads[:, :, : s.nope_dim], self.key_up, q_latent)
        o_latent = k.latent_attention(q_latent, q, cache.k_pool, batch.positions, batch.token_row, tables.kv_indptr, tables.kv_indices,
                                      H, s.nope_dim, s.rope_dim, s.kv_rank, s.scale, s.window, batch.kv_cap, batch.all_single, batch.q_indptr)
        o = torch.empty((T, H * s.v_dim), dtype=q.dtype, device=q.device)
        batched_linear(self.rt, o_latent, self.value_up, o.view(T, H, s.v_dim).transpose(0, 1))
        if s.head_gate:
            k.head_gate_mul_(o, self.head_gate(x), 0, H)                     # head h's output times sigmoid((W_g x)_h)
        return self.out(o)


register_mixer("latent_attention", LatentAttention)
