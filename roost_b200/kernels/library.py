"""The Python side of the kernel library's C ABI: loads the shared object, checks its version and wraps every
entry point so that tensors go in and a non-OK status becomes an exception with the library's message.

There is no other implementation behind these functions: when the library cannot be built or loaded, or when
no CUDA device is present, ``load()`` raises and nothing in the engine runs.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p

import torch

from . import build

ABI_VERSION = 15
F32, BF16 = 0, 1
GATE_FUNCTIONS = {"silu": 0, "gelu_tanh": 1, "clamped_swish": 2}   # the codes of csrc/roost_kernels.h


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is neither float32 nor bfloat16")


def _ptr(t):
    """The address as a plain integer (ctypes converts it by the entry point's declared argument types)."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle. The wrappers run hundreds of times a step, so this goes through torch's raw getter
    (a fraction of a microsecond) where the build has it, instead of building a Stream object (several microseconds)."""
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    return _raw_stream(torch.cuda.current_device())


def _need(t: torch.Tensor, name: str, dtype=None):
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}; expected {dtype}")


_SIGNATURES = {
    "roost_status_snapshot": [c_void_p, c_int, c_void_p],
    "roost_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_rms_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "roost_add_rms_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "roost_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_gemm_tcgen05_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_void_p],
    "roost_qk_norm_rope_cache": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int64, c_int, c_int, c_int,
                                 c_void_p],
    "roost_rope_table": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "roost_paged_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "roost_attention_mma_supported": [c_int],
    "roost_attention_prefill_tile_rows": [c_int, c_int, c_int, c_int, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong],
    "roost_attention_set_prefill_tc": [c_int],
    "roost_attention_prefill_tile_rows_mma": [c_int, c_int, ctypes.c_longlong],
    "roost_attention_prefill": [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_longlong, c_float, c_int, c_void_p],
    "roost_attention_prefill_capped": [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_int, c_int, c_int, c_int, c_int, c_int, ctypes.c_longlong, c_float, c_int, c_float, c_void_p],
    "roost_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, ctypes.c_longlong, c_float, c_int,
                               c_void_p],
    "roost_attention_decode_cluster": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                       c_int, c_int, c_int, c_int, ctypes.c_longlong, c_float, c_int, c_void_p],
    "roost_attention_decode_cluster_supported": [c_int, c_int, ctypes.c_longlong, c_int, c_void_p, c_void_p],
    "roost_sample_penalise": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p],
    "roost_sample_count_tokens": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "roost_sample_prompt_bits": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "roost_sample_logprobs": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
    "roost_gemm_simt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_void_p],
    "roost_gemm_tcgen05_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    "roost_gemm_tcgen05_status": [],
    "roost_attention_status": [],
    "roost_attention_set_decode_tma": [c_int],
    "roost_gemm_stream_workspace_floats": [],
    "roost_gemm_stream_workspace_flags": [],
    "roost_gemm_stream_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_preferred": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_swiglu_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_split_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    "roost_gemm_split": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p],
    "roost_gemm_stream": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                          c_void_p],
    "roost_gemm_stream_swiglu_supported": [c_int, c_int, c_int, c_int64, c_int64],
    "roost_gemm_stream_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                 c_void_p],
    "roost_embedding_scaled": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "roost_layer_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "roost_softcap": [c_void_p, c_int64, c_float, c_void_p],
    "roost_gemm_simt_batched": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                c_int, c_int, c_void_p],
    "roost_latent_prepare": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_float, c_int, c_void_p],
    "roost_latent_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
    "roost_latent_attention_tc_supported": [c_int, c_int, c_int],
    "roost_latent_attention_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_float, c_int, c_void_p],
    "roost_mamba2_conv": [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int,
                          c_int, c_int, c_int, c_int, c_void_p],
    "roost_mamba2_conv_state": [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_mamba2_scan": [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "roost_mamba2_scan_chunks": [c_int, c_int],
    "roost_gated_group_norm": [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "roost_moe_tile_rows": [],
    "roost_moe_router_logits": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_moe_wide_tile_rows": [],
    "roost_moe_route": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
    "roost_gemm_tcgen05_grouped": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "roost_moe_gather_scale": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_moe_expert_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                              c_int, c_int, c_void_p],
    "roost_moe_combine_weighted": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                   c_int, c_int, c_void_p],
    "roost_stream_step": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                          c_int, c_void_p],
    "roost_gated_act_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "roost_sink_attention_prepare": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_float, c_int, c_int, c_int, c_void_p],
    "roost_sink_attention": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "roost_wide_rms_norm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "roost_normed_mean": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "roost_pair_embedding": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, c_void_p],
    "roost_last_token_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "roost_add_bias": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "roost_gelu_mul_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_gated_recurrence_scan_chunks": [c_int, c_int],
    "roost_gated_recurrence_scan": [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "roost_matrix_memory_scan_chunks": [c_int, c_int],
    "roost_matrix_memory_scan": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_float, c_void_p, c_int, c_void_p],
    "roost_head_norm_gate": [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "roost_retention_prepare": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "roost_retention_scan_chunks": [c_int, c_int],
    "roost_retention_scan": [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                             c_void_p, c_int, c_void_p],
    "roost_sigmoid_attention_prepare": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_int, c_float, c_float, c_int, c_int, c_int, c_void_p],
    "roost_sigmoid_attention": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p],
    "roost_sigmoid_attention_mma_supported": [c_int, c_int, c_int],
    "roost_sigmoid_attention_mma": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_void_p],
    "roost_latent_gather": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_carried_attention_supported": [c_int, c_int],
    "roost_carried_attention": [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                c_void_p],
    "roost_xielu": [c_void_p, c_void_p, c_int64, c_float, c_float, c_int, c_void_p],
    "roost_head_gate_mul": [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "roost_wide_rms_norm_gated": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "roost_scale": [c_void_p, c_int64, c_float, c_void_p],
    "roost_mamba1_scan": [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "roost_mamba1_scan_chunks": [c_int, c_int],
    "roost_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "roost_argmax": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p],
    "roost_argmax_split": [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "roost_sample": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                     c_void_p, c_void_p],
}


@dataclass
class MoeRoute:
    """What ``moe_route`` leaves on the device: the (token, choice) pairs sorted by expert. ``token``/``weight``/``expert``:
    a sorted row's token, weight and expert; ``inverse[token * top + k]``: where the token's k-th choice went; ``offsets``:
    the experts' row ranges; ``tiles``: (expert, first row, one past the last) of every tile of sorted rows, -1 beyond.
    ``form``: which expert product the step runs (0: tiles of rows, 1: a warp an output, for few rows)."""
    top: int
    rows: int
    token: torch.Tensor
    weight: torch.Tensor
    expert: torch.Tensor
    inverse: torch.Tensor
    offsets: torch.Tensor
    tiles: torch.Tensor
    max_tiles: int
    form: int
    real: int = 1 << 30                        # experts from here on are identity experts: rows without weights
    wide_tiles: torch.Tensor | None = None     # the same rows in tiles of 128, for the tcgen05 product of steps of many rows
    max_wide_tiles: int = 0


MOE_TCGEN05_MIN_ROWS = 1024  # sorted rows from which a bfloat16 step runs the experts' products on tcgen05
MOE_ROW_FORM_MAX_ROWS = 64   # sorted rows up to which a bfloat16 step streams each row's expert instead of tiling the rows


class KernelLibrary:
    def __init__(self, path):
        self.path = str(path)
        self._lib = ctypes.CDLL(self.path)
        self._lib.roost_abi_version.restype = c_int
        self._lib.roost_last_error.restype = c_char_p
        got = self._lib.roost_abi_version()
        if got != ABI_VERSION:
            raise KernelError(f"{self.path} has ABI version {got}; this package needs {ABI_VERSION}")
        for name, args in _SIGNATURES.items():
            fn = getattr(self._lib, name)
            fn.argtypes = args
            fn.restype = c_int
        self.decode_chunk = 512  # keys per work item of the split decode attention (see decode_chunk_for)
        self.decode_cluster = True  # split rows merged by thread-block clusters where they fit (see decode_cluster_for)
        self._decode_ctas = 0
        self.launches = 0  # kernels launched through this handle (a host-side count of entry-point calls that launch)
        self.library_launches = 0  # products handed to cuBLAS through torch beside them (counted where they are called)

    def _call(self, name: str, *args, launches: int = 1):
        status = getattr(self._lib, name)(*args)
        if status != 0:
            msg = self._lib.roost_last_error().decode(errors="replace")
            raise KernelError(f"{name}: {msg} (status {status})")
        self.launches += launches

    def decode_chunk_for(self, rows: int, kv_cap: int, kv_heads: int) -> int:
        """Keys per work item of the split decode attention for a step of ``rows`` rows whose requests hold at most
        ``kv_cap`` keys (the bound of the captured step, so that every replay of it agrees). The persistent decode
        kernel runs two CTAs an SM; when ``decode_chunk`` keys an item give more items than CTAs but at most twice as
        many, the second round would be half empty, and items of twice the keys run as one full round instead (batch 8
        at 4096 keys: 4.42 against 4.51 ms a step). A row's bits then depend on the step's size class, within rounding."""
        if not self._decode_ctas:
            self._decode_ctas = 2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        items = rows * kv_heads * (-(-max(kv_cap, 1) // self.decode_chunk))
        return 2 * self.decode_chunk if self._decode_ctas < items <= 2 * self._decode_ctas else self.decode_chunk

    def decode_cluster_for(self, rows: int, kv_cap: int, chunk: int, k_pool: torch.Tensor, v_pool: torch.Tensor) -> int:
        """CTAs of a cluster that takes one (row, key/value head) of the split decode attention and merges the row's
        chunks itself, for a step of ``rows`` rows whose requests hold at most ``kv_cap`` keys in chunks of ``chunk``: the
        power of two that covers the chunks, when that is 2 to 8 and all the clusters run at once (two CTAs an SM);
        else 0: partial results go through memory and the merge kernel. Same bits either way."""
        if not self.decode_cluster:
            return 0
        if not self._decode_ctas:
            self._decode_ctas = 2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        pages, nkv, page, d = k_pool.shape
        chunks = -(-max(kv_cap, 1) // chunk)
        size = 1
        while size < chunks:
            size *= 2
        if size < 2 or size > 8 or rows * nkv * size > self._decode_ctas:
            return 0
        return size if self._lib.roost_attention_decode_cluster_supported(d, page, pages, nkv, _ptr(k_pool), _ptr(v_pool)) else 0

    def decode_split_for(self, rows: int, kv_cap: int, k_pool: torch.Tensor, v_pool: torch.Tensor) -> tuple[int, int]:
        """(keys per work item, CTAs a cluster or 0) of the split decode attention for a step of ``rows`` rows whose
        requests hold at most ``kv_cap`` keys (the bounds of the captured step, so that every replay of it agrees). Where
        clusters serve, the smallest chunk of 128, 256, 512 or 1024 keys whose clusters all run at once: more CTAs pull
        on the memory and the merge costs no kernel (one row of 1,024 keys: 7.7 us in chunks of 128, 12.6 us in chunks of
        512). Else the chunk of ``decode_chunk_for`` through the merge kernel. A row's bits depend on the chunk, so on
        the step's size class, within rounding."""
        if self.decode_cluster and kv_cap > 0:
            for chunk in (128, 256, 512, 1024):
                cluster = self.decode_cluster_for(rows, kv_cap, chunk, k_pool, v_pool)
                if cluster:
                    return chunk, cluster
        return self.decode_chunk_for(rows, kv_cap, k_pool.shape[1]), 0

    # ------------------------------------------------------------------ ops
    def embedding(self, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        _need(table, "table"); _need(ids, "ids", torch.int32)
        T, (V, H) = ids.numel(), table.shape
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
        self._call("roost_embedding", _ptr(table), _ptr(ids), _ptr(out), T, H, V, dtype_code(table.dtype), _stream())
        return out

    def rms_norm(self, x: torch.Tensor, w: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> torch.Tensor:
        _need(x, "x"); _need(w, "w")
        H = x.shape[-1]
        if w.numel() != H:
            raise KernelError(f"rms_norm: weight has {w.numel()} elements for rows of {H}")
        n = x.numel() // H if rows is None else rows.numel()
        out = torch.empty((n, H) if rows is not None else x.shape, dtype=x.dtype, device=x.device)
        self._call("roost_rms_norm", _ptr(x), _ptr(w), _ptr(out), _ptr(rows), n, H, eps, dtype_code(x.dtype),
                   dtype_code(w.dtype), _stream())
        return out

    def add_rms_norm(self, x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                     rows: torch.Tensor | None = None) -> torch.Tensor:
        """residual += x (in place, unless ``rows`` gathers) and the norm of the sum."""
        _need(x, "x"); _need(residual, "residual", x.dtype); _need(w, "w")
        H = x.shape[-1]
        if residual.shape != x.shape or w.numel() != H:
            raise KernelError("add_rms_norm: x, residual and weight do not agree in shape")
        n = x.numel() // H if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=x.dtype, device=x.device)
        self._call("roost_add_rms_norm", _ptr(x), _ptr(residual), _ptr(w), _ptr(out), _ptr(rows), n, H, eps,
                   dtype_code(x.dtype), dtype_code(w.dtype), _stream())
        return out

    def silu_mul(self, x: torch.Tensor, block: int = 0) -> torch.Tensor:
        """silu(gate) * up over rows [gate | up] (block 0) or rows of blocks of ``block`` gate then ``block`` up values."""
        _need(x, "x")
        T, two_i = x.shape
        out = torch.empty((T, two_i // 2), dtype=x.dtype, device=x.device)
        self._call("roost_silu_mul", _ptr(x), _ptr(out), T, two_i // 2, block, dtype_code(x.dtype), _stream())
        return out

    def gemm_tcgen05_swiglu(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """silu(a Wg^T) * (a Wu^T) in one kernel; w holds gate and up rows interleaved in blocks of 128."""
        _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = a.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_tcgen05_swiglu: a has {K} columns, w has {K2}")
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device)
        self._call("roost_gemm_tcgen05_swiglu", _ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0), _stream())
        return out

    def rope_table(self, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
        """(cos, sin) of positions[t] * inv_freq[i] as float32 [T, half, 2]: a step computes it once for all its layers."""
        _need(positions, "positions", torch.int32); _need(inv_freq, "inv_freq", torch.float64)
        T, half = positions.numel(), inv_freq.numel()
        out = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
        self._call("roost_rope_table", _ptr(positions), _ptr(inv_freq), T, half, _ptr(out), _stream())
        return out

    def qk_norm_rope_cache(self, qkv, q_heads, kv_heads, head_dim, *, q_w, k_w, eps, inv_freq, rotary_dim, positions,
                           k_pool=None, v_pool=None, slot_mapping=None, page_size=0, write_kv=True, cos_sin=None) -> torch.Tensor:
        """qkv: [T, (q_heads + 2 kv_heads) * head_dim] (or [T, q_heads * head_dim] with write_kv False). Returns
        q: [T, q_heads, head_dim], normed and rotated; k and v go into the pools. ``cos_sin``: the step's table from
        ``rope_table`` for these positions and this ``inv_freq`` (else the kernel computes the same values itself)."""
        _need(qkv, "qkv")
        T = qkv.shape[0]
        width = (q_heads + (2 * kv_heads if write_kv else 0)) * head_dim
        if qkv.shape[1] != width:
            raise KernelError(f"qk_norm_rope_cache: qkv rows have {qkv.shape[1]} elements; expected {width}")
        q = torch.empty((T, q_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
        wd = dtype_code(q_w.dtype) if q_w is not None else F32
        pages = 0
        if write_kv:
            _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype); _need(slot_mapping, "slot_mapping", torch.int32)
            pages = k_pool.shape[0]
            if tuple(k_pool.shape[1:]) != (kv_heads, page_size, head_dim) or k_pool.shape != v_pool.shape:
                raise KernelError(f"qk_norm_rope_cache: pool shape {tuple(k_pool.shape)} is not [pages, {kv_heads}, {page_size}, {head_dim}]")
        if rotary_dim:
            _need(inv_freq, "inv_freq", torch.float64); _need(positions, "positions", torch.int32)
            if inv_freq.numel() != rotary_dim // 2:
                raise KernelError("qk_norm_rope_cache: inv_freq must have rotary_dim / 2 entries")
            if cos_sin is not None:
                _need(cos_sin, "cos_sin", torch.float32)
                if tuple(cos_sin.shape) != (T, rotary_dim // 2, 2):
                    raise KernelError(f"qk_norm_rope_cache: the table is {tuple(cos_sin.shape)}; expected {(T, rotary_dim // 2, 2)}")
        else:
            cos_sin = None
        self._call("roost_qk_norm_rope_cache", _ptr(qkv), qkv.stride(0), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(q_w),
                   _ptr(k_w), _ptr(inv_freq), _ptr(positions), _ptr(slot_mapping), _ptr(cos_sin), T, q_heads, kv_heads, head_dim,
                   rotary_dim, eps, page_size, pages, 1 if write_kv else 0, dtype_code(qkv.dtype), wd, _stream())
        return q

    def paged_attention_generic(self, q, k_pool, v_pool, positions, token_row, kv_indptr, kv_indices, scale: float,
                                window: int | None) -> torch.Tensor:
        _need(q, "q"); _need(k_pool, "k_pool", q.dtype); _need(v_pool, "v_pool", q.dtype)
        for n, t in (("positions", positions), ("token_row", token_row), ("kv_indptr", kv_indptr), ("kv_indices", kv_indices)):
            _need(t, n, torch.int32)
        T, nq, d = q.shape
        _, nkv, page, d2 = k_pool.shape
        if d2 != d:
            raise KernelError("paged_attention: head_dim of q and of the pool differ")
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
        self._call("roost_paged_attention_generic", _ptr(q), _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(positions),
                   _ptr(token_row), _ptr(kv_indptr), _ptr(kv_indices), T, nq, nkv, d, page, scale,
                   int(window) if window else 0, dtype_code(q.dtype), _stream())
        return out

    def attention_mma_supported(self, head_dim: int) -> bool:
        return bool(self._lib.roost_attention_mma_supported(int(head_dim)))

    def attention_prefill_tile_rows(self, q_heads: int, k_pool: torch.Tensor, v_pool: torch.Tensor, packed_rows: int = 0,
                                    tensor_memory: bool = True) -> int:
        """Packed rows of a prefill work item (64 or 128) for these pools [pages, kv_heads, page_size, head_dim] and a step
        that brings ``packed_rows`` packed rows in all to the prefill kernels."""
        pages, nkv, page, d = k_pool.shape
        if not tensor_memory:       # the mma.sync kernels' items (a caller that wants wide weights)
            return int(self._lib.roost_attention_prefill_tile_rows_mma(d, nkv, int(packed_rows)))
        return int(self._lib.roost_attention_prefill_tile_rows(d, int(q_heads), nkv, page, pages, _ptr(k_pool), _ptr(v_pool), int(packed_rows)))

    def attention_set_prefill_tc(self, on: bool) -> None:
        """Prompt portions run the tcgen05 attention kernel where the sizes allow (the default), or never."""
        self._lib.roost_attention_set_prefill_tc(1 if on else 0)

    attention_mma_sink = True    # the tensor-core kernels take a softmax with one added to its denominator (``sink``)
    attention_mma_softcap = True  # ... and their prompt kernels a cap on the scores (``softcap``)
    ATTENTION_SINK = 1 << 30     # ROOST_ATTENTION_SINK of csrc/roost_kernels.h
    ATTENTION_WIDE_WEIGHTS = 1 << 29

    def attention_mma(self, q, k_pool, v_pool, q_indptr, kv_lens, kv_indptr, kv_indices, plan, scale: float,
                      window: int | None, sink: bool = False, wide_weights: bool = False, softcap: float = 0.0) -> torch.Tensor:
        """Tensor-core attention (bfloat16). ``plan``: an ``AttentionPlan`` whose work lists are on the device. ``sink``: one is
        added to the softmax's denominator (a key of score 0 that has no value). ``wide_weights``: the softmax weights enter P V as two
        bfloat16 operands (16 bits of the 32-bit weights); the plan's prefill items must then come from
        ``attention_prefill_tile_rows(..., tensor_memory=False)``. ``softcap`` c > 0: a scaled score s becomes c tanh(s / c); the
        prompt kernels on mma.sync serve it (items from ``tensor_memory=False``), the decode kernels do not: the plan must hold no
        decode items then."""
        _need(q, "q", torch.bfloat16); _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16)
        T, nq, d = q.shape
        _, nkv, page, d2 = k_pool.shape
        if d2 != d:
            raise KernelError("attention_mma: head_dim of q and of the pool differ")
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
        w = (int(window) if window else 0) | (self.ATTENTION_SINK if sink else 0) | (self.ATTENTION_WIDE_WEIGHTS if wide_weights else 0)
        if softcap and plan.decode_items:
            raise KernelError("attention_mma: the decode kernels know no cap on the scores")
        if plan.prefill_items and softcap:
            self._call("roost_attention_prefill_capped", _ptr(q), T, _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(q_indptr), _ptr(kv_lens),
                       _ptr(kv_indptr), _ptr(kv_indices), _ptr(plan.prefill_work), plan.prefill_items, plan.prefill_tile_rows, nq, nkv, d, page,
                       k_pool.shape[0], scale, w, float(softcap), _stream())
        elif plan.prefill_items:
            self._call("roost_attention_prefill", _ptr(q), T, _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(q_indptr), _ptr(kv_lens),
                       _ptr(kv_indptr), _ptr(kv_indices), _ptr(plan.prefill_work), plan.prefill_items, plan.prefill_tile_rows, nq, nkv, d, page,
                       k_pool.shape[0], scale, w, _stream())
        if plan.decode_items and plan.cluster_chunks:
            self._call("roost_attention_decode_cluster", _ptr(q), _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(q_indptr), _ptr(kv_lens),
                       _ptr(kv_indptr), _ptr(kv_indices), _ptr(plan.decode_work), plan.decode_items, plan.cluster_chunks, nq, nkv, d, page,
                       k_pool.shape[0], scale, w, _stream())
        elif plan.decode_items:
            part_o = part_ml = None
            if plan.slots:
                part_o = torch.empty((plan.slots * nkv * 16 * d,), dtype=torch.float32, device=q.device)
                part_ml = torch.empty((plan.slots * nkv * 16 * 2,), dtype=torch.float32, device=q.device)
            self._call("roost_attention_decode", _ptr(q), _ptr(out), _ptr(k_pool), _ptr(v_pool), _ptr(q_indptr), _ptr(kv_lens),
                       _ptr(kv_indptr), _ptr(kv_indices), _ptr(plan.decode_work), plan.decode_items, _ptr(plan.merge_work),
                       plan.merge_items, plan.merge_rows, _ptr(part_o), _ptr(part_ml), nq, nkv, d, page, k_pool.shape[0], scale, w, _stream(),
                       launches=2 if plan.merge_items else 1)
        return out

    def gemm_simt(self, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """a [M, K] times w [N, K] transposed, 32-bit FFMA accumulation."""
        _need(w, "w", a.dtype)
        if not a.is_cuda or a.dim() != 2 or (a.shape[1] > 1 and a.stride(1) != 1):       # rows may be strided (a column range of wider rows)
            raise KernelError("a is not a CUDA matrix with dense rows")
        M, K = a.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm: a has {K} columns, w has {K2}")
        out_dtype = out_dtype or a.dtype
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        self._call("roost_gemm_simt", _ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0),
                   dtype_code(a.dtype), dtype_code(out_dtype), _stream())
        return out

    def gemm_tcgen05_supported(self, m: int, n: int, k: int, lda: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_tcgen05_supported(m, n, k, lda, ldw))

    def gemm_tcgen05(self, a: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """a [M, K] times w [N, K] transposed on the tcgen05 tensor cores (TMA loads, accumulator in tensor memory)."""
        _need(a, "a", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = a.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_tcgen05: a has {K} columns, w has {K2}")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        self._call("roost_gemm_tcgen05", _ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _stream())
        return out

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch for the library's kernels."""
        self._lib.roost_set_pdl(1 if on else 0)
        self.pdl = bool(on)

    def gemm_stream_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_stream_supported(m, n, k, ldx, ldw))

    def _stream_workspace(self, device):
        ws = getattr(self, "_stream_ws", None)
        if ws is None or ws[0].device != device:
            # allocated once, outside any stream capture (the first decode step of a model runs eagerly)
            ws = self._stream_ws = (torch.zeros(self._lib.roost_gemm_stream_workspace_floats(), dtype=torch.float32, device=device),
                                    torch.zeros(self._lib.roost_gemm_stream_workspace_flags(), dtype=torch.int32, device=device))
        return ws

    def gemm_stream(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """x [M <= 64, K] times w [N, K] transposed: the weight-streaming tcgen05 product of decode steps."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_stream: x has {K} columns, w has {K2}")
        ws = self._stream_workspace(x.device)
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_stream", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _ptr(ws[0]), _ptr(ws[1]), _stream())
        return out

    def gemm_split_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_split_supported(m, n, k, ldx, ldw))

    def gemm_split_preferred(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        """Whether the k-split product was measured faster than the other products for this shape."""
        return bool(self._lib.roost_gemm_split_preferred(m, n, k, ldx, ldw))

    def gemm_split(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """x [M <= 64, K] times w [N, K] transposed for a weight of few 128-row tiles and a long K: K split over
        thread-block clusters, the partial sums added up through distributed shared memory."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_split: x has {K} columns, w has {K2}")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_split", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _stream())
        return out

    def gemm_split_swiglu_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_split_swiglu_supported(m, n, k, ldx, ldw))

    def gemm_split_swiglu(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for x [M <= 32, K] and w [2I, K] with gate and up rows interleaved in blocks of 128:
        the k-split product with the activation applied to the summed accumulators; returns [M, I]."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_split_swiglu: x has {K} columns, w has {K2}")
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_split_swiglu", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _stream())
        return out

    def gemm_stream_swiglu_supported(self, m: int, n: int, k: int, ldx: int, ldw: int) -> bool:
        return bool(self._lib.roost_gemm_stream_swiglu_supported(m, n, k, ldx, ldw))

    def gemm_stream_swiglu(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """silu(x Wg^T) * (x Wu^T) for x [M <= 32, K] and w [2I, K] with gate and up rows interleaved in blocks of 128:
        the weight-streaming product with the activation applied to its accumulators; returns [M, I]."""
        _need(x, "x", torch.bfloat16); _need(w, "w", torch.bfloat16)
        M, K = x.shape
        N, K2 = w.shape
        if K != K2:
            raise KernelError(f"gemm_stream_swiglu: x has {K} columns, w has {K2}")
        ws = self._stream_workspace(x.device)
        out_dtype = out_dtype or torch.bfloat16
        out = torch.empty((M, N // 2), dtype=out_dtype, device=x.device)
        self._call("roost_gemm_stream_swiglu", _ptr(x), _ptr(w), _ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
                   dtype_code(out_dtype), _ptr(ws[0]), _ptr(ws[1]), _stream())
        return out

    # ------------------------------------------------------------------ a 32-bit stream's ends and norm
    def embedding_scaled(self, table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
        """table[ids] * scale as a float32 stream."""
        _need(table, "table"); _need(ids, "ids", torch.int32)
        T, (V, H) = ids.numel(), table.shape
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
        self._call("roost_embedding_scaled", _ptr(table), _ptr(ids), _ptr(out), T, H, V, scale, dtype_code(table.dtype), _stream())
        return out

    def layer_norm(self, stream: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float, out_dtype: torch.dtype,
                   addend: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
        """Layer norm of the float32 ``stream`` (plus ``addend``, added in 32-bit and written back unless ``rows`` gathers)
        into ``out_dtype``."""
        _need(stream, "stream", torch.float32); _need(w, "w", torch.float32); _need(b, "b", torch.float32)
        H = stream.shape[-1]
        if w.numel() != H or b.numel() != H:
            raise KernelError(f"layer_norm: weight and bias must have {H} elements")
        if addend is not None:
            _need(addend, "addend", out_dtype)
            if addend.shape != stream.shape:
                raise KernelError("layer_norm: the addend and the stream differ in shape")
        if rows is not None:
            _need(rows, "rows", torch.int32)
        n = stream.numel() // H if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=out_dtype, device=stream.device)
        self._call("roost_layer_norm", _ptr(stream), _ptr(addend), _ptr(w), _ptr(b), _ptr(out), _ptr(rows), n, H, eps, dtype_code(out_dtype),
                   _stream())
        return out

    def softcap_(self, logits: torch.Tensor, cap: float) -> torch.Tensor:
        _need(logits, "logits", torch.float32)
        self._call("roost_softcap", _ptr(logits), logits.numel(), cap, _stream())
        return logits

    def gemm_simt_batched(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out[b] = a[b] w[b]^T on FFMA; a [B, M, K], w [B, N, K] and out [B, M, N] may be strided views with a dense last
        dimension."""
        B, M, K = a.shape
        _, N, _ = w.shape
        if w.shape != (B, N, K) or out.shape != (B, M, N) or a.dtype != w.dtype:
            raise KernelError(f"gemm_simt_batched: shapes {tuple(a.shape)}, {tuple(w.shape)}, {tuple(out.shape)} do not fit")
        for n, t in (("a", a), ("w", w), ("out", out)):
            if not t.is_cuda or t.stride(2) != 1:
                raise KernelError(f"gemm_simt_batched: {n} must be on the device with a dense last dimension")
        self._call("roost_gemm_simt_batched", _ptr(a), _ptr(w), _ptr(out), B, M, N, K, a.stride(1), w.stride(1), out.stride(1), a.stride(0),
                   w.stride(0), out.stride(0), dtype_code(a.dtype), dtype_code(out.dtype), _stream())
        return out

    # ------------------------------------------------------------------ latent attention
    def latent_prepare(self, q, down, pool, latent_w, inv_freq, rotary_dim, positions, slot_mapping, heads, nope, rope, rank, eps, page_size) -> None:
        """Rotates the heads' rotated query parts in place and, when ``down`` is given, writes the tokens' cache entries."""
        _need(q, "q"); _need(positions, "positions", torch.int32)
        if rotary_dim:
            _need(inv_freq, "inv_freq", torch.float64)
        T = q.shape[0]
        if q.shape[1] != heads * (nope + rope) or (rotary_dim and inv_freq.numel() != rotary_dim // 2):
            raise KernelError("latent_prepare: q or inv_freq do not fit the sizes")
        if down is not None:
            _need(down, "down", q.dtype); _need(pool, "pool", q.dtype); _need(latent_w, "latent_w", torch.float32)
            _need(slot_mapping, "slot_mapping", torch.int32)
            if tuple(down.shape) != (T, rank + rope) or tuple(pool.shape[1:]) != (1, page_size, rank + rope) or latent_w.numel() != rank:
                raise KernelError("latent_prepare: down, pool or the latent's weight do not fit the sizes")
        self._call("roost_latent_prepare", _ptr(q), _ptr(down), _ptr(pool), _ptr(latent_w), _ptr(inv_freq) if rotary_dim else None, _ptr(positions), _ptr(slot_mapping),
                   T, heads, nope, rope, rotary_dim, rank, eps, dtype_code(q.dtype), _stream())

    def latent_splits_for(self, tokens: int, heads: int, window: int | None, kv_cap: int) -> int:
        """Blocks a token's keys are dealt to: 1 when the step's (token, 8 heads) blocks fill the device by themselves, else as
        many as give two blocks an SM, up to the tiles a token can have (from the window and the bound on the requests'
        lengths, so that every replay of a captured step agrees) and to 32."""
        if not self._decode_ctas:
            self._decode_ctas = 2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        blocks = tokens * (-(-heads // 8))
        reach = min(window, kv_cap) if window else kv_cap
        tiles = -(-max(reach, 1) // 32) + 1
        return max(1, min(self._decode_ctas // max(blocks, 1), tiles, 32))

    LATENT_TC_MIN_ROWS = 128    # packed (token, head) rows from which a bfloat16 step runs the tensor-core form

    def latent_attention(self, q_latent, q, pool, positions, token_row, kv_indptr, kv_indices, heads, nope, rope, rank, scale, window,
                         kv_cap: int = 0, few_rows: bool = False, q_indptr: torch.Tensor | None = None) -> torch.Tensor:
        """Attention in the latent space: out [heads, tokens, rank]. bfloat16 steps of many tokens (prompt portions) run on
        the tensor cores where the sizes allow; steps of few rows (decode) and float32 run the 32-bit form, a token's keys
        dealt to several blocks when the step alone would not fill the device."""
        _need(q_latent, "q_latent"); _need(q, "q", q_latent.dtype); _need(pool, "pool", q.dtype)
        for n, t in (("positions", positions), ("token_row", token_row), ("kv_indptr", kv_indptr), ("kv_indices", kv_indices)):
            _need(t, n, torch.int32)
        T = q.shape[0]
        if tuple(q_latent.shape) != (heads, T, rank) or pool.shape[-1] != rank + rope or pool.shape[1] != 1:
            raise KernelError("latent_attention: q_latent or the pool do not fit the sizes")
        out = torch.empty((heads, T, rank), dtype=q.dtype, device=q.device)
        if (q.dtype == torch.bfloat16 and q_indptr is not None and not few_rows and T * heads >= self.LATENT_TC_MIN_ROWS
                and self._lib.roost_latent_attention_tc_supported(nope, rope, rank)):
            _need(q_indptr, "q_indptr", torch.int32)
            self._call("roost_latent_attention_tc", _ptr(q_latent), _ptr(q), _ptr(out), _ptr(pool), _ptr(positions), _ptr(q_indptr),
                       _ptr(kv_indptr), _ptr(kv_indices), T, q_indptr.numel() - 1, heads, nope, rope, rank, pool.shape[2], scale,
                       int(window) if window else 0, _stream())
            return out
        splits = self.latent_splits_for(T, heads, window, kv_cap) if kv_cap else 1
        part = torch.empty((T * heads * splits * (rank + 2),), dtype=torch.float32, device=q.device) if splits > 1 else None
        self._call("roost_latent_attention", _ptr(q_latent), _ptr(q), _ptr(out), _ptr(part), _ptr(pool), _ptr(positions), _ptr(token_row),
                   _ptr(kv_indptr), _ptr(kv_indices), T, heads, nope, rope, rank, pool.shape[2], scale, int(window) if window else 0, splits,
                   dtype_code(q.dtype), _stream(), launches=2 if splits > 1 else 1)
        return out

    # ------------------------------------------------------------------ prompt portions over keys and values carried out of a latent cache
    def latent_gather(self, pool, kv_lens, kv_indptr, kv_indices, rows: int, stride: int) -> torch.Tensor:
        """[rows * stride, width]: entry r * stride + j is the cached vector of row r's token at position j (zeros beyond the row)."""
        _need(pool, "pool", torch.bfloat16)
        for n, t in (("kv_lens", kv_lens), ("kv_indptr", kv_indptr), ("kv_indices", kv_indices)):
            _need(t, n, torch.int32)
        if pool.shape[1] != 1 or kv_lens.numel() < rows:
            raise KernelError("latent_gather: a pool of one vector a token and a length a row")
        out = torch.empty((rows * stride, pool.shape[3]), dtype=pool.dtype, device=pool.device)
        self._call("roost_latent_gather", _ptr(pool), _ptr(out), _ptr(kv_lens), _ptr(kv_indptr), _ptr(kv_indices), rows, stride, pool.shape[3],
                   pool.shape[2], _stream())
        return out

    def carried_attention_supported(self, dim: int, vdim: int) -> bool:
        return bool(self._lib.roost_carried_attention_supported(int(dim), int(vdim)))

    def carried_attention(self, q, keys, values, positions, q_indptr, heads: int, dim: int, vdim: int, stride: int, scale: float) -> torch.Tensor:
        """Causal softmax attention of the step's queries q [T, >= heads * dim] over keys [rows * stride, heads * dim] and values
        [rows * stride, heads * vdim] (entry r * stride + j: row r's token at position j): [T, heads * vdim], bfloat16 on the tensor cores."""
        _need(q, "q", torch.bfloat16); _need(keys, "keys", torch.bfloat16); _need(values, "values", torch.bfloat16)
        _need(positions, "positions", torch.int32); _need(q_indptr, "q_indptr", torch.int32)
        T, rows = q.shape[0], q_indptr.numel() - 1
        if q.shape[1] < heads * dim or tuple(keys.shape) != (rows * stride, heads * dim) or tuple(values.shape) != (rows * stride, heads * vdim):
            raise KernelError("carried_attention: the queries, keys or values do not fit the sizes")
        out = torch.empty((T, heads * vdim), dtype=q.dtype, device=q.device)
        self._call("roost_carried_attention", _ptr(q), q.stride(0), _ptr(out), _ptr(keys), _ptr(values), _ptr(positions), _ptr(q_indptr), T, rows, heads,
                   dim, vdim, stride, float(scale), _stream())
        return out

    # ------------------------------------------------------------------ the Mamba-2 recurrence
    def mamba2_conv(self, u, col, channels, w, b, state, conv_off, token_row, q_indptr, slots, activation: str = "silu") -> torch.Tensor:
        """``activation``: "silu" of the sum, or "none"."""
        if activation not in ("silu", "none"):
            raise KernelError(f"mamba2_conv: activation '{activation}' is neither silu nor none")
        _need(u, "u"); _need(w, "w", torch.float32); _need(b, "b", torch.float32); _need(state, "state", torch.float32)
        T = u.shape[0]
        out = torch.empty((T, channels), dtype=u.dtype, device=u.device)
        self._call("roost_mamba2_conv", _ptr(u), u.stride(0), col, _ptr(out), _ptr(w), _ptr(b), _ptr(state), state.stride(0), conv_off,
                   _ptr(token_row), _ptr(q_indptr), _ptr(slots), T, channels, w.shape[1], 1 if activation == "silu" else 0, dtype_code(u.dtype),
                   _stream())
        return out

    def mamba2_conv_state(self, u, col, channels, taps, state, conv_off, q_indptr, slots) -> None:
        _need(u, "u"); _need(state, "state", torch.float32)
        self._call("roost_mamba2_conv_state", _ptr(u), u.stride(0), col, _ptr(state), state.stride(0), conv_off, _ptr(q_indptr), _ptr(slots),
                   slots.numel(), channels, taps, dtype_code(u.dtype), _stream(), launches=1 if taps > 1 else 0)

    SCAN_CHUNKED_MIN_TOKENS = 512

    def mamba2_scan(self, xbc, u, dt_col, dt_bias, a_log, d, state, q_indptr, slots, heads, head_dim, state_rows, groups) -> torch.Tensor:
        _need(xbc, "xbc"); _need(u, "u", xbc.dtype); _need(state, "state", torch.float32)
        for n, t in (("dt_bias", dt_bias), ("A_log", a_log), ("D", d)):
            _need(t, n, torch.float32)
        T = xbc.shape[0]
        y = torch.empty((T, heads * head_dim), dtype=torch.float32, device=xbc.device)
        ws_state = ws_decay = None
        if T >= self.SCAN_CHUNKED_MIN_TOKENS:       # long rows are cut into chunks that run side by side
            chunks = self._lib.roost_mamba2_scan_chunks(T, slots.numel())
            ws_state = torch.empty((chunks * heads * head_dim * state_rows,), dtype=torch.float32, device=xbc.device)
            ws_decay = torch.empty((chunks * heads,), dtype=torch.float32, device=xbc.device)
        self._call("roost_mamba2_scan", _ptr(xbc), _ptr(u), u.stride(0), dt_col, _ptr(y), _ptr(dt_bias), _ptr(a_log), _ptr(d), _ptr(state),
                   state.stride(0), _ptr(q_indptr), _ptr(slots), slots.numel(), T, heads, head_dim, state_rows, groups, _ptr(ws_state),
                   _ptr(ws_decay), dtype_code(xbc.dtype), _stream(), launches=3 if ws_state is not None else 1)
        return y

    def gated_group_norm(self, y, u, w, groups, eps, out_dtype) -> torch.Tensor:
        _need(y, "y", torch.float32); _need(u, "u", out_dtype); _need(w, "w", torch.float32)
        T, inner = y.shape
        out = torch.empty((T, inner), dtype=out_dtype, device=y.device)
        self._call("roost_gated_group_norm", _ptr(y), _ptr(u), u.stride(0), _ptr(w), _ptr(out), T, inner, groups, eps, dtype_code(out_dtype),
                   _stream())
        return out

    # ------------------------------------------------------------------ routed experts
    def moe_router_logits(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """x W^T as 32-bit sums, float32 [tokens, experts]."""
        _need(x, "x"); _need(w, "w", x.dtype)
        T, H = x.shape
        E = w.shape[0]
        if w.shape[1] != H:
            raise KernelError("moe_router_logits: x and the router's weight differ in width")
        out = torch.empty((T, E), dtype=torch.float32, device=x.device)
        self._call("roost_moe_router_logits", _ptr(x), _ptr(w), _ptr(out), T, H, E, dtype_code(x.dtype), _stream())
        return out

    def moe_route(self, logits: torch.Tensor, top: int, score: str = "sigmoid", correction: torch.Tensor | None = None, scale: float = 1.0,
                  routed: int | None = None, real: int | None = None) -> MoeRoute:
        """``score`` "sigmoid": the weights are the sigmoid of the chosen logits. "softmax": scores are the softmax over the first
        ``routed`` columns (default all), ``correction`` is added for the choice only, the weights are score * ``scale``; experts
        from ``real`` on are identity experts (sorted rows, no tiles)."""
        _need(logits, "logits", torch.float32)
        T, columns = logits.shape
        E = columns if routed is None else routed
        real = E if real is None else real
        if score not in ("sigmoid", "softmax"):
            raise KernelError(f"moe_route: score '{score}' is neither sigmoid nor softmax")
        if correction is not None:
            _need(correction, "correction", torch.float32)
            if correction.numel() != E:
                raise KernelError("moe_route: the correction does not have one number a routed expert")
        counts = getattr(self, "_moe_counts", None)
        if counts is None or counts.device != logits.device:
            # the experts' running counts: zero between calls (the sorting kernel leaves them so), allocated once, outside any capture
            counts = self._moe_counts = torch.zeros(4096, dtype=torch.int32, device=logits.device)
        rows = T * top
        tile = self._lib.roost_moe_tile_rows()
        max_tiles = -(-rows // tile) + E
        dev = logits.device
        wide = self._lib.roost_moe_wide_tile_rows()
        max_wide = (-(-rows // wide) + E) if rows >= MOE_TCGEN05_MIN_ROWS else 0
        ints = torch.empty((4 * rows + (E + 1) + 3 * max_tiles + 3 * max_wide + 3 * rows,), dtype=torch.int32, device=dev)
        token, expert, inverse = ints[:rows], ints[rows : 2 * rows], ints[2 * rows : 3 * rows]
        at = 3 * rows
        offsets, at = ints[at : at + E + 1], at + E + 1
        tiles, at = ints[at : at + 3 * max_tiles], at + 3 * max_tiles
        wide_tiles, at = (ints[at : at + 3 * max_wide] if max_wide else None), at + 3 * max_wide
        scratch = ints[at : at + 3 * rows]
        weight = torch.empty((rows,), dtype=torch.float32, device=dev)
        self._call("roost_moe_route", _ptr(logits), T, columns, E, real, top, 1 if score == "softmax" else 0, _ptr(correction), float(scale),
                   _ptr(token), _ptr(weight), _ptr(expert), _ptr(inverse), _ptr(offsets), _ptr(tiles), max_tiles, _ptr(wide_tiles), max_wide,
                   _ptr(scratch), _ptr(counts), _stream(), launches=2)
        return MoeRoute(top=top, rows=rows, token=token, weight=weight, expert=expert, inverse=inverse, offsets=offsets, tiles=tiles,
                        max_tiles=max_tiles, form=0, real=real, wide_tiles=wide_tiles, max_wide_tiles=max_wide)

    def moe_gather_scale(self, x: torch.Tensor, route: MoeRoute, scale: bool = True) -> torch.Tensor:
        """The tokens' rows in the order of the sorted pairs, times the pair's weight (``scale``) or as they are."""
        _need(x, "x")
        xs = torch.empty((route.rows, x.shape[1]), dtype=x.dtype, device=x.device)
        self._call("roost_moe_gather_scale", _ptr(x), _ptr(xs), _ptr(route.token), _ptr(route.weight), route.rows, x.shape[1], 1 if scale else 0,
                   dtype_code(x.dtype), _stream())
        return xs

    def _moe_gemm(self, a, w1, w2, route: MoeRoute, block: int = 0, activation: str = "silu", limit: float = 0.0) -> torch.Tensor:
        """The experts' product on tiles of rows or a warp an output. ``block`` > 0: ``w1`` is [experts, 2 n, k] with gate and
        up rows interleaved in blocks of ``block`` and ``w2`` is not looked at."""
        _need(a, "a"); _need(w1, "w1", a.dtype)
        E, N, K = w1.shape
        if block:
            N, w2 = N // 2, w1
        if a.shape != (route.rows, K) or (w2 is not None and not block and w2.shape != w1.shape):
            raise KernelError(f"moe_expert_gemm: rows {tuple(a.shape)} against weights {tuple(w1.shape)}")
        form = 1 if (a.dtype == torch.bfloat16 and route.rows <= MOE_ROW_FORM_MAX_ROWS) else 0
        out = torch.empty((route.rows, N), dtype=a.dtype, device=a.device)
        self._call("roost_moe_expert_gemm", _ptr(a), _ptr(w1), _ptr(w2), _ptr(out), _ptr(route.tiles), route.max_tiles, _ptr(route.expert),
                   route.rows, N, K, form, block, GATE_FUNCTIONS[activation], float(limit), min(route.real, E), dtype_code(a.dtype), _stream())
        return out

    def _moe_gemm_tcgen05(self, a, w, route: MoeRoute, swiglu: bool, activation: str = "silu", limit: float = 0.0) -> torch.Tensor:
        E, N, K = w.shape
        out = torch.empty((route.rows, N // 2 if swiglu else N), dtype=a.dtype, device=a.device)
        self._call("roost_gemm_tcgen05_grouped", _ptr(a), _ptr(w), _ptr(out), _ptr(route.wide_tiles), route.max_wide_tiles, route.rows, E, N, K,
                   1 if swiglu else 0, GATE_FUNCTIONS[activation], float(limit), _stream())
        return out

    def moe_expert_gate_up(self, xs, gate, up, route: MoeRoute, gate_up: torch.Tensor | None = None, activation: str = "silu",
                           limit: float = 0.0) -> torch.Tensor:
        """silu(xs Wg[e]^T) * (xs Wu[e]^T) over the sorted rows, e the row's expert. The weights come as ``gate`` and ``up``
        [experts, ff, k], or as ``gate_up`` [experts, 2 ff, k] with an expert's gate and up rows interleaved in blocks of
        128: the layout in which the tcgen05 product of steps of many rows applies the activation to its accumulator, and
        which the other forms read as well."""
        if gate_up is None:
            return self._moe_gemm(xs, gate, up, route, activation=activation, limit=limit)
        if route.wide_tiles is not None and xs.dtype == torch.bfloat16 and xs.shape[1] % 8 == 0:
            _need(xs, "xs"); _need(gate_up, "gate_up", torch.bfloat16)
            return self._moe_gemm_tcgen05(xs, gate_up, route, True, activation, limit)
        return self._moe_gemm(xs, gate_up, None, route, block=128, activation=activation, limit=limit)

    def moe_expert_down(self, act, down, route: MoeRoute) -> torch.Tensor:
        if route.wide_tiles is not None and act.dtype == torch.bfloat16 and act.shape[1] % 8 == 0 and down.shape[1] % 8 == 0:
            _need(act, "act"); _need(down, "down", torch.bfloat16)
            return self._moe_gemm_tcgen05(act, down, route, False)
        return self._moe_gemm(act, down, None, route)

    def moe_combine(self, ys: torch.Tensor, route: MoeRoute, shared: torch.Tensor | None = None) -> torch.Tensor:
        _need(ys, "ys")
        T, H = route.rows // route.top, ys.shape[1]
        if shared is not None:
            _need(shared, "shared", ys.dtype)
        out = torch.empty((T, H), dtype=ys.dtype, device=ys.device)
        self._call("roost_moe_combine", _ptr(ys), _ptr(route.inverse), _ptr(shared), _ptr(out), T, H, route.top, dtype_code(ys.dtype), _stream())
        return out

    def moe_combine_weighted(self, ys: torch.Tensor, route: MoeRoute, x: torch.Tensor, shared: torch.Tensor | None = None,
                             gate_logits: torch.Tensor | None = None) -> torch.Tensor:
        """out[t] = sum_k weight_k * (the k-th chosen expert's output, or x[t] for an identity expert) + sigmoid(gate) * shared[t];
        ``gate_logits``: float32 [T, columns] whose last column is the shared expert's gate logit (None: the gate is 1)."""
        _need(ys, "ys"); _need(x, "x", ys.dtype)
        T, H = x.shape
        if shared is not None:
            _need(shared, "shared", ys.dtype)
        gate, stride = None, 0
        if gate_logits is not None:
            _need(gate_logits, "gate_logits", torch.float32)
            gate, stride = gate_logits.data_ptr() + 4 * (gate_logits.shape[1] - 1), gate_logits.shape[1]
        out = torch.empty((T, H), dtype=ys.dtype, device=ys.device)
        self._call("roost_moe_combine_weighted", _ptr(ys), _ptr(route.inverse), _ptr(route.weight), _ptr(route.expert), _ptr(x), _ptr(shared),
                   gate, stride, _ptr(out), T, H, route.top, route.real, dtype_code(ys.dtype), _stream())
        return out

    # ------------------------------------------------------------------ residual streams, gate functions
    def stream_step(self, streams, norm_w, eps, out_dtype, read=None, y=None, mix=None, write=None, init_from=None, rows=None) -> torch.Tensor:
        """One pass over the tokens' residual streams (float32 [T, S, width], updated in place): fresh streams from
        ``init_from``, or the write-back x'_r = sum_s mix[s, r] x_s + write[r] y of the sublayer before (not stored when ``rows``
        selects tokens); then the read u = sum_s read[s] x'_s (None: the plain sum) and its root-mean-square norm times
        ``norm_w`` (float32, any offset folded in), in ``out_dtype``."""
        _need(streams, "streams", torch.float32); _need(norm_w, "norm_w", torch.float32)
        T, S, W = streams.shape
        for n, t in (("read", read), ("mix", mix), ("write", write)):
            if t is not None:
                _need(t, n, torch.float32)
        for n, t in (("y", y), ("init_from", init_from)):
            if t is not None:
                _need(t, n, out_dtype)
                if tuple(t.shape) != (T, W):
                    raise KernelError(f"stream_step: {n} is {tuple(t.shape)}; the streams hold {T} tokens of width {W}")
        n_out = T
        if rows is not None:
            _need(rows, "rows", torch.int32)
            n_out = rows.numel()
        out = torch.empty((n_out, W), dtype=out_dtype, device=streams.device)
        self._call("roost_stream_step", _ptr(streams), _ptr(y), _ptr(init_from), _ptr(mix), _ptr(write), _ptr(read), _ptr(norm_w), _ptr(rows),
                   _ptr(out), n_out, S, W, float(eps), dtype_code(out_dtype), _stream())
        return out

    def gated_act_mul(self, x: torch.Tensor, activation: str, limit: float = 0.0, block: int = 0) -> torch.Tensor:
        """fn(gate) * up over rows [gate | up] for the gate function ``activation`` (see ``GATE_FUNCTIONS``)."""
        _need(x, "x")
        T, two_i = x.shape
        out = torch.empty((T, two_i // 2), dtype=x.dtype, device=x.device)
        self._call("roost_gated_act_mul", _ptr(x), _ptr(out), T, two_i // 2, block, GATE_FUNCTIONS[activation], float(limit), dtype_code(x.dtype),
                   _stream())
        return out

    # ------------------------------------------------------------------ attention with a sink
    @staticmethod
    def _sink_cache(k_pool, v_pool, dim, vdim):
        """(keys' base address, values' base address, numbers between two entries) of a cache of two planes or of one."""
        if v_pool is None:
            if k_pool.shape[3] != dim + vdim:
                raise KernelError("sink_attention: a cache of one plane holds entries of dim + vdim numbers")
            return k_pool.data_ptr(), k_pool.data_ptr() + dim * k_pool.element_size(), dim + vdim
        if k_pool.shape[3] != dim or v_pool.shape[3] != vdim or dim != vdim:
            raise KernelError("sink_attention: a cache of two planes holds keys and values of one size")
        return k_pool.data_ptr(), v_pool.data_ptr(), dim

    def sink_attention_prepare(self, qkv, k_pool, v_pool, inv_freq, rotary_dim, positions, slot_mapping, heads, kv_heads, dim, vdim, eps,
                               page_size, q_out: torch.Tensor | None = None, halves: bool = False) -> None:
        """``q_out`` [tokens, heads, dim]: where the prepared queries go instead of back into ``qkv``. ``halves``: element i of the
        rotated part is paired with element i + rotary_dim / 2 instead of its neighbour."""
        if q_out is not None:
            _need(q_out, "q_out", qkv.dtype)
            if tuple(q_out.shape) != (qkv.shape[0], heads, dim):
                raise KernelError("sink_attention_prepare: q_out is not [tokens, heads, dim]")
        _need(qkv, "qkv"); _need(k_pool, "k_pool", qkv.dtype); _need(positions, "positions", torch.int32); _need(slot_mapping, "slot_mapping", torch.int32)
        if v_pool is not None:
            _need(v_pool, "v_pool", qkv.dtype)
        if rotary_dim:
            _need(inv_freq, "inv_freq", torch.float64)
        if qkv.shape[1] != (heads + kv_heads) * dim + kv_heads * vdim or k_pool.shape[1] != kv_heads or k_pool.shape[2] != page_size:
            raise KernelError("sink_attention_prepare: qkv or the pool do not fit the sizes")
        kb, vb, entry = self._sink_cache(k_pool, v_pool, dim, vdim)
        self._call("roost_sink_attention_prepare", _ptr(qkv), qkv.stride(0), _ptr(q_out), kb, vb, entry, _ptr(inv_freq) if rotary_dim else None, _ptr(positions),
                   _ptr(slot_mapping), qkv.shape[0], heads, kv_heads, dim, vdim, rotary_dim, float(eps) if eps else 0.0, page_size,
                   1 if halves else 0, dtype_code(qkv.dtype), _stream())

    def sink_splits_for(self, tokens: int, gy: int, kv_cap: int) -> tuple[int, int]:
        """(blocks a token's key tiles are dealt to, tiles a block): 1 when the step's blocks fill the device by themselves,
        else as many as give two blocks an SM, up to 32 and to the tiles the bound on the requests' lengths allows, so that
        every replay of a captured step agrees."""
        if not self._decode_ctas:
            self._decode_ctas = 2 * torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        tiles = -(-max(kv_cap, 1) // 32)
        splits = max(1, min(self._decode_ctas // max(tokens * gy, 1), -(-tiles // 4), 32))
        per = -(-tiles // splits)
        return -(-tiles // per), per

    def sink_attention(self, qkv, k_pool, v_pool, positions, token_row, kv_indptr, kv_indices, heads, kv_heads, dim, vdim, scale, sink,
                       kv_cap: int = 0, window: int | None = None, softcap: float = 0.0) -> torch.Tensor:
        """Attention of the step's (prepared) queries over the paged cache in 32-bit arithmetic: out [T, heads * vdim]. ``window``:
        the keys a query sees, its own included (None: all); ``softcap`` c > 0: a scaled score s becomes c tanh(s / c)."""
        _need(qkv, "qkv"); _need(k_pool, "k_pool", qkv.dtype)
        for n, t in (("positions", positions), ("token_row", token_row), ("kv_indptr", kv_indptr), ("kv_indices", kv_indices)):
            _need(t, n, torch.int32)
        T = qkv.shape[0]
        kb, vb, entry = self._sink_cache(k_pool, v_pool, dim, vdim)
        out = torch.empty((T, heads * vdim), dtype=qkv.dtype, device=qkv.device)
        gy = kv_heads * (-(-(heads // kv_heads) // 8))
        # a window's keys span at most window + 31 positions' worth of tiles, whatever the requests' lengths are
        span = min(kv_cap, window + 62) if (window and kv_cap) else kv_cap
        splits, per = self.sink_splits_for(T, gy, span) if span else (1, 1 << 24)
        part = torch.empty((T * heads * splits * (vdim + 2),), dtype=torch.float32, device=qkv.device) if splits > 1 else None
        self._call("roost_sink_attention", _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(part), kb, vb, entry, _ptr(positions), _ptr(token_row),
                   _ptr(kv_indptr), _ptr(kv_indices), T, heads, kv_heads, dim, vdim, k_pool.shape[2], float(scale), 1 if sink else 0, splits, per,
                   int(window or 0), float(softcap or 0.0), dtype_code(qkv.dtype), _stream(), launches=2 if splits > 1 else 1)
        return out

    # ------------------------------------------------------------------ a 32-bit stream with root-mean-square norms
    def wide_rms_norm(self, stream: torch.Tensor, w: torch.Tensor | None, eps: float, out_dtype: torch.dtype, addend: torch.Tensor | None = None,
                      extra: torch.Tensor | None = None, rows: torch.Tensor | None = None) -> torch.Tensor:
        """Root-mean-square norm of the float32 ``stream`` plus ``addend`` (activation dtype) plus ``extra`` (float32), the sums
        formed in 32-bit and written back unless ``rows`` gathers, into ``out_dtype``; without ``w`` the sum itself, rounded."""
        _need(stream, "stream", torch.float32)
        H = stream.shape[-1]
        if w is not None:
            _need(w, "w", torch.float32)
            if w.numel() != H:
                raise KernelError(f"wide_rms_norm: the weight must have {H} elements")
        if addend is not None:
            _need(addend, "addend", out_dtype)
            if addend.shape != stream.shape:
                raise KernelError("wide_rms_norm: the addend and the stream differ in shape")
        if extra is not None:
            _need(extra, "extra", torch.float32)
            if extra.shape != stream.shape:
                raise KernelError("wide_rms_norm: the second addend and the stream differ in shape")
        if rows is not None:
            _need(rows, "rows", torch.int32)
        n = stream.numel() // H if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=out_dtype, device=stream.device)
        self._call("roost_wide_rms_norm", _ptr(stream), _ptr(addend), _ptr(extra), _ptr(w), _ptr(out), _ptr(rows), n, H, eps, dtype_code(out_dtype),
                   _stream())
        return out

    def normed_mean(self, xs: list, ws: list, eps: float) -> torch.Tensor:
        """The mean of the branches ``xs`` [T, H], each divided by its root mean square over a row and multiplied by its weight."""
        n = len(xs)
        if not 1 <= n <= 4 or len(ws) != n:
            raise KernelError("normed_mean: one to four branches with a weight each")
        for x, w in zip(xs, ws):
            _need(x, "x", xs[0].dtype); _need(w, "w", torch.float32)
            if x.shape != xs[0].shape or w.numel() != x.shape[1]:
                raise KernelError("normed_mean: the branches and their weights differ in shape")
        T, H = xs[0].shape
        out = torch.empty((T, H), dtype=xs[0].dtype, device=xs[0].device)
        xp = (c_void_p * n)(*[x.data_ptr() for x in xs])
        wp = (c_void_p * n)(*[w.data_ptr() for w in ws])
        self._call("roost_normed_mean", xp, wp, n, _ptr(out), T, H, eps, dtype_code(out.dtype), _stream())
        return out

    def pair_embedding(self, table, pairs, ids, positions, token_row, q_indptr, slots, state, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
        """table[ids] + pairs[(previous id * mul_prev + id * mul_cur) mod buckets] as a float32 stream; ``state`` int32 [slots, 1] holds
        the id before each request's next token."""
        _need(table, "table"); _need(pairs, "pairs", table.dtype); _need(ids, "ids", torch.int32); _need(state, "state", torch.int32)
        for n, t in (("positions", positions), ("token_row", token_row), ("q_indptr", q_indptr), ("slots", slots)):
            _need(t, n, torch.int32)
        T, (V, H) = ids.numel(), table.shape
        if tuple(pairs.shape) != (buckets + 1, H):
            raise KernelError(f"pair_embedding: the pair table must be [{buckets + 1}, {H}]")
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
        self._call("roost_pair_embedding", _ptr(table), _ptr(pairs), _ptr(ids), _ptr(positions), _ptr(token_row), _ptr(q_indptr), _ptr(slots),
                   _ptr(state), _ptr(out), T, H, V, buckets, mul_prev, mul_cur, dtype_code(table.dtype), _stream())
        return out

    def last_token_store(self, ids, q_indptr, slots, state) -> None:
        _need(ids, "ids", torch.int32); _need(state, "state", torch.int32)
        self._call("roost_last_token_store", _ptr(ids), _ptr(q_indptr), _ptr(slots), _ptr(state), slots.numel(), _stream())

    def add_bias_(self, y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
        _need(y, "y", torch.float32); _need(bias, "bias", torch.float32)
        if y.dim() != 2 or bias.numel() != y.shape[1]:
            raise KernelError("add_bias: one bias a column of a [rows, width] tensor")
        self._call("roost_add_bias", _ptr(y), _ptr(bias), y.shape[0], y.shape[1], _stream())
        return y

    def gelu_mul_rows(self, gate: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        """gelu_tanh(gate) * table[ids], the function on the 32-bit values."""
        _need(gate, "gate"); _need(table, "table", gate.dtype); _need(ids, "ids", torch.int32)
        T, D = gate.shape
        if table.shape[1] != D or ids.numel() != T:
            raise KernelError("gelu_mul_rows: the table's rows and the gate's differ in width")
        out = torch.empty_like(gate)
        self._call("roost_gelu_mul_rows", _ptr(gate), _ptr(table), _ptr(ids), _ptr(out), T, D, table.shape[0], dtype_code(gate.dtype), _stream())
        return out

    # ------------------------------------------------------------------ the gated linear recurrence, the matrix memory
    def gated_recurrence_scan(self, u, gates, yx, gate_bias, decay, state, q_indptr, slots, width: int, blocks: int, chunked: bool | None = None) -> torch.Tensor:
        """S <- a S + sqrt(1 - a^2) i u a channel, out = S gelu_tanh(y): see csrc/gated_recurrence.cu. ``chunked`` None: steps of
        ``SCAN_CHUNKED_MIN_TOKENS`` tokens or more cut their rows into chunks that run side by side."""
        _need(u, "u"); _need(gates, "gates", torch.float32); _need(yx, "yx", u.dtype); _need(state, "state", torch.float32)
        _need(gate_bias, "gate_bias", torch.float32); _need(decay, "decay", torch.float32)
        T = u.shape[0]
        if tuple(u.shape) != (T, width) or tuple(gates.shape) != (blocks, T, 2 * (width // blocks)) or gate_bias.numel() != 2 * width or decay.numel() != width:
            raise KernelError("gated_recurrence_scan: the gates, biases or decays do not fit the sizes")
        out = torch.empty((T, width), dtype=u.dtype, device=u.device)
        ws_state = ws_decay = None
        if (T >= self.SCAN_CHUNKED_MIN_TOKENS) if chunked is None else chunked:
            chunks = self._lib.roost_gated_recurrence_scan_chunks(T, slots.numel())
            ws_state = torch.empty((chunks * width,), dtype=torch.float32, device=u.device)
            ws_decay = torch.empty((chunks * width,), dtype=torch.float32, device=u.device)
        self._call("roost_gated_recurrence_scan", _ptr(u), _ptr(gates), _ptr(yx), yx.stride(0), _ptr(out), _ptr(gate_bias), _ptr(decay), _ptr(state),
                   state.stride(0), _ptr(q_indptr), _ptr(slots), slots.numel(), T, width, blocks, _ptr(ws_state), _ptr(ws_decay), dtype_code(u.dtype),
                   _stream(), launches=3 if ws_state is not None else 1)
        return out

    def matrix_memory_scan(self, qkv, gates, state, q_indptr, slots, heads: int, dim: int, vdim: int, cap: float, floor: float,
                           chunked: bool | None = None) -> torch.Tensor:
        """The matrix memory's outputs a head before their norm, float32 [T, heads * vdim]: see csrc/matrix_memory.cu. ``chunked``
        None: steps of ``SCAN_CHUNKED_MIN_TOKENS`` tokens or more cut their rows into chunks that run side by side."""
        _need(qkv, "qkv"); _need(gates, "gates", torch.float32); _need(state, "state", torch.float32)
        T = qkv.shape[0]
        if tuple(gates.shape) != (T, 2 * heads) or qkv.shape[1] < heads * (2 * dim + vdim):
            raise KernelError("matrix_memory_scan: the gates or the projection's rows do not fit the sizes")
        out = torch.empty((T, heads * vdim), dtype=torch.float32, device=qkv.device)
        ws = None
        if (T >= self.SCAN_CHUNKED_MIN_TOKENS) if chunked is None else chunked:
            chunks = self._lib.roost_matrix_memory_scan_chunks(T, slots.numel())
            ws = torch.empty((chunks * heads * (dim * vdim + dim + 3),), dtype=torch.float32, device=qkv.device)
        self._call("roost_matrix_memory_scan", _ptr(qkv), qkv.stride(0), _ptr(gates), _ptr(out), _ptr(state), state.stride(0), _ptr(q_indptr),
                   _ptr(slots), slots.numel(), T, heads, dim, vdim, float(cap), float(floor), _ptr(ws), dtype_code(qkv.dtype), _stream(),
                   launches=3 if ws is not None else 1)
        return out

    def head_norm_gate(self, o, u, col: int, w, heads: int, eps: float, out_dtype, gate: str = "sigmoid") -> torch.Tensor:
        """o / sqrt(mean over a head of o^2 + eps) * w * sigmoid(u[:, col : col + width]) into ``out_dtype``; ``w`` None: no weight;
        ``gate`` "silu": the gate is g sigmoid(g) of g = u[:, col : col + width]."""
        if gate not in ("sigmoid", "silu"):
            raise KernelError(f"head_norm_gate: gate '{gate}' is neither sigmoid nor silu")
        _need(o, "o", torch.float32); _need(u, "u", out_dtype)
        if w is not None:
            _need(w, "w", torch.float32)
        T, V = o.shape
        out = torch.empty((T, V), dtype=out_dtype, device=o.device)
        self._call("roost_head_norm_gate", _ptr(o), _ptr(u), u.stride(0), col, _ptr(w), _ptr(out), T, heads, V // heads, eps,
                   1 if gate == "silu" else 0, dtype_code(out_dtype), _stream())
        return out

    # ------------------------------------------------------------------ retention
    def retention_prepare(self, u, inv_freq, rotary_dim: int, positions, heads: int, dim: int, k_scale: float) -> torch.Tensor:
        """The rotated query heads and the rotated, scaled key heads of rows [q heads | k heads | ...] as float32 [T, 2 * heads * dim]."""
        _need(u, "u"); _need(positions, "positions", torch.int32)
        if rotary_dim:
            _need(inv_freq, "inv_freq", torch.float64)
            if inv_freq.numel() != rotary_dim // 2:
                raise KernelError("retention_prepare: inv_freq must have rotary_dim / 2 entries")
        T = u.shape[0]
        if u.shape[1] < 2 * heads * dim:
            raise KernelError("retention_prepare: the rows do not hold the query and key heads")
        qk = torch.empty((T, 2 * heads * dim), dtype=torch.float32, device=u.device)
        self._call("roost_retention_prepare", _ptr(u), u.stride(0), _ptr(qk), _ptr(inv_freq) if rotary_dim else None, _ptr(positions), T, heads, dim,
                   rotary_dim, float(k_scale), dtype_code(u.dtype), _stream())
        return qk

    def retention_scan(self, qk, u, v_col: int, state, decay, q_indptr, slots, heads: int, dim: int, vdim: int, chunked: bool | None = None) -> torch.Tensor:
        """S <- decay_h S + k v^T, o = S^T q a head: float32 [T, heads * vdim]; see csrc/retention.cu. The values are the columns
        from ``v_col`` on of ``u``. ``chunked`` None: steps of ``SCAN_CHUNKED_MIN_TOKENS`` tokens or more cut their rows into chunks."""
        _need(qk, "qk", torch.float32); _need(u, "u"); _need(state, "state", torch.float32); _need(decay, "decay", torch.float32)
        _need(q_indptr, "q_indptr", torch.int32); _need(slots, "slots", torch.int32)
        T = u.shape[0]
        if tuple(qk.shape) != (T, 2 * heads * dim) or u.shape[1] < v_col + heads * vdim or decay.numel() != heads:
            raise KernelError("retention_scan: the queries and keys, the values or the decays do not fit the sizes")
        out = torch.empty((T, heads * vdim), dtype=torch.float32, device=u.device)
        ws = None
        if (T >= self.SCAN_CHUNKED_MIN_TOKENS) if chunked is None else chunked:
            chunks = self._lib.roost_retention_scan_chunks(T, slots.numel())
            ws = torch.empty((chunks * heads * dim * vdim,), dtype=torch.float32, device=u.device)
        self._call("roost_retention_scan", _ptr(qk), u.data_ptr() + v_col * u.element_size(), u.stride(0), _ptr(out), _ptr(state), state.stride(0),
                   _ptr(decay), _ptr(q_indptr), _ptr(slots), slots.numel(), T, heads, dim, vdim, _ptr(ws), dtype_code(u.dtype), _stream(),
                   launches=3 if ws is not None else 1)
        return out

    # ------------------------------------------------------------------ attention with sigmoid weights
    def sigmoid_attention_prepare(self, qkv, k_pool, v_pool, q_w, k_w, positions, slot_mapping, heads, kv_heads, dim, vdim, eps, temp_coef,
                                  temp_every, page_size) -> torch.Tensor:
        """Normed (and, for the queries, temperature-scaled) heads: the queries come back as [T, heads, dim], keys and values go to the cache."""
        _need(qkv, "qkv"); _need(k_pool, "k_pool", qkv.dtype); _need(positions, "positions", torch.int32); _need(slot_mapping, "slot_mapping", torch.int32)
        _need(q_w, "q_w", torch.float32); _need(k_w, "k_w", torch.float32)
        if v_pool is not None:
            _need(v_pool, "v_pool", qkv.dtype)
        if qkv.shape[1] < (heads + kv_heads) * dim + kv_heads * vdim or k_pool.shape[1] != kv_heads or k_pool.shape[2] != page_size:
            raise KernelError("sigmoid_attention_prepare: qkv or the pool do not fit the sizes")
        if q_w.numel() != dim or k_w.numel() != dim:
            raise KernelError("sigmoid_attention_prepare: the norms' weights must have dim entries")
        kb, vb, entry = self._sink_cache(k_pool, v_pool, dim, vdim)
        q = torch.empty((qkv.shape[0], heads, dim), dtype=qkv.dtype, device=qkv.device)
        self._call("roost_sigmoid_attention_prepare", _ptr(qkv), qkv.stride(0), _ptr(q), kb, vb, entry, _ptr(q_w), _ptr(k_w), _ptr(positions),
                   _ptr(slot_mapping), qkv.shape[0], heads, kv_heads, dim, vdim, float(eps), float(temp_coef), int(temp_every), page_size,
                   dtype_code(qkv.dtype), _stream())
        return q

    SIGMOID_MMA_MIN_TOKENS = 32     # tokens from which a bfloat16 step that brings prompt portions runs the tensor-core form
    SIGMOID_MMA_CHUNK_TILES = 8     # tiles of 64 keys a block of the tensor-core form takes of a long row

    def sigmoid_attention_mma_supported(self, dim: int, vdim: int, two_planes: bool) -> bool:
        return bool(self._lib.roost_sigmoid_attention_mma_supported(int(dim), int(vdim), int(dim if two_planes else dim + vdim)))

    def sigmoid_attention(self, q, k_pool, v_pool, gate_rows, gate_col, slopes, head_bias, positions, token_row, kv_indptr, kv_indices, kv_heads, vdim,
                          scale, kv_cap: int = 0, q_indptr: torch.Tensor | None = None) -> torch.Tensor:
        """out[t, h] = sum over visible keys j of sigmoid((q . k_j) scale - slopes[h] (p - j) + head_bias[h]) v_j, times
        sigmoid(gate_rows[t, gate_col + h * vdim : ...]) when ``gate_col`` is not None: [T, heads * vdim]. With ``q_indptr`` (the rows'
        token ranges) a bfloat16 step runs on the tensor cores where the sizes allow; without, the 32-bit form, a token's keys dealt to
        several blocks when the step alone would not fill the device."""
        _need(q, "q"); _need(k_pool, "k_pool", q.dtype); _need(slopes, "slopes", torch.float32); _need(head_bias, "head_bias", torch.float32)
        for n, t in (("positions", positions), ("token_row", token_row), ("kv_indptr", kv_indptr), ("kv_indices", kv_indices)):
            _need(t, n, torch.int32)
        T, heads, dim = q.shape
        if slopes.numel() != heads or head_bias.numel() != heads:
            raise KernelError("sigmoid_attention: one slope and one bias a query head")
        gate_ptr, ld_gate = None, 0
        if gate_col is not None:
            _need(gate_rows, "gate_rows", q.dtype)
            if gate_rows.shape[0] != T or gate_rows.shape[1] < gate_col + heads * vdim:
                raise KernelError("sigmoid_attention: the gate's rows do not fit the sizes")
            gate_ptr, ld_gate = gate_rows.data_ptr() + gate_col * gate_rows.element_size(), gate_rows.stride(0)
        kb, vb, entry = self._sink_cache(k_pool, v_pool, dim, vdim)
        out = torch.empty((T, heads * vdim), dtype=q.dtype, device=q.device)
        if q_indptr is not None and q.dtype == torch.bfloat16 and self.sigmoid_attention_mma_supported(dim, vdim, v_pool is not None):
            _need(q_indptr, "q_indptr", torch.int32)
            # rows of more than SIGMOID_MMA_CHUNK_TILES tiles of 64 keys have the keys of their later queries dealt to several blocks;
            # the bound on the requests' lengths says how many (every replay of a captured step agrees)
            per = self.SIGMOID_MMA_CHUNK_TILES
            chunks = -(-(kv_cap // 64 + 1) // per) if kv_cap else 1
            if chunks == 1:
                per = 1 << 24
            ws = torch.empty((T * heads * chunks * vdim,), dtype=torch.float32, device=q.device) if chunks > 1 else None
            self._call("roost_sigmoid_attention_mma", _ptr(q), _ptr(out), kb, vb, entry, gate_ptr, ld_gate, _ptr(slopes), _ptr(head_bias), _ptr(positions),
                       _ptr(q_indptr), _ptr(token_row), _ptr(kv_indptr), _ptr(kv_indices), T, q_indptr.numel() - 1, heads, kv_heads, dim, vdim,
                       k_pool.shape[2], float(scale), _ptr(ws), per, chunks, _stream(), launches=2 if chunks > 1 else 1)
            return out
        gy = kv_heads * (-(-(heads // kv_heads) // 8))
        splits, per = self.sink_splits_for(T, gy, kv_cap) if kv_cap else (1, 1 << 24)
        part = torch.empty((T * heads * splits * vdim,), dtype=torch.float32, device=q.device) if splits > 1 else None
        self._call("roost_sigmoid_attention", _ptr(q), _ptr(out), _ptr(part), kb, vb, entry, gate_ptr, ld_gate, _ptr(slopes), _ptr(head_bias),
                   _ptr(positions), _ptr(token_row), _ptr(kv_indptr), _ptr(kv_indices), T, heads, kv_heads, dim, vdim, k_pool.shape[2], float(scale),
                   splits, per, dtype_code(q.dtype), _stream(), launches=2 if splits > 1 else 1)
        return out

    # ------------------------------------------------------------------ activations, gates, scaled sums
    def xielu(self, x: torch.Tensor, a_pos: float, a_neg: float) -> torch.Tensor:
        """a_pos z^2 + z / 2 for z > 0, a_neg (exp(z) - 1 - z) + z / 2 for z <= 0."""
        _need(x, "x")
        out = torch.empty_like(x)
        self._call("roost_xielu", _ptr(x), _ptr(out), x.numel(), float(a_pos), float(a_neg), dtype_code(x.dtype), _stream())
        return out

    def head_gate_mul_(self, x: torch.Tensor, g: torch.Tensor, col: int, heads: int) -> torch.Tensor:
        """x[t, h, :] *= sigmoid(g[t, col + h]) in place, for x [T, heads * vdim]."""
        _need(x, "x"); _need(g, "g", x.dtype)
        T, V = x.shape
        if V % heads or g.shape[0] != T or g.shape[1] < col + heads:
            raise KernelError("head_gate_mul: one gate a token and head")
        self._call("roost_head_gate_mul", _ptr(x), _ptr(g), g.stride(0), col, T, heads, V // heads, dtype_code(x.dtype), _stream())
        return x

    def wide_rms_norm_gated(self, stream, w, eps: float, out_dtype, addend, gate, gate_bias, rows=None) -> torch.Tensor:
        """``wide_rms_norm`` with the addend multiplied by sigmoid(gate + gate_bias) first (gate float32 like the stream, bias [hidden])."""
        _need(stream, "stream", torch.float32); _need(addend, "addend", out_dtype); _need(gate, "gate", torch.float32)
        _need(gate_bias, "gate_bias", torch.float32)
        H = stream.shape[-1]
        if w is not None:
            _need(w, "w", torch.float32)
        if addend.shape != stream.shape or gate.shape != stream.shape or gate_bias.numel() != H or (w is not None and w.numel() != H):
            raise KernelError("wide_rms_norm_gated: the addend, the gate, its bias or the weight do not fit the stream")
        if rows is not None:
            _need(rows, "rows", torch.int32)
        n = stream.numel() // H if rows is None else rows.numel()
        out = torch.empty((n, H), dtype=out_dtype, device=stream.device)
        self._call("roost_wide_rms_norm_gated", _ptr(stream), _ptr(addend), _ptr(gate), _ptr(gate_bias), _ptr(w), _ptr(out), _ptr(rows), n, H, eps,
                   dtype_code(out_dtype), _stream())
        return out

    def scale_(self, x: torch.Tensor, factor: float) -> torch.Tensor:
        _need(x, "x", torch.float32)
        self._call("roost_scale", _ptr(x), x.numel(), float(factor), _stream())
        return x

    # ------------------------------------------------------------------ the selective scan
    def mamba1_scan(self, xc, dt, dbc, xz, dt_bias, a, d, state, q_indptr, slots, inner, n_state, dt_rank, chunked: bool | None = None) -> torch.Tensor:
        """``chunked`` None: steps of ``SCAN_CHUNKED_MIN_TOKENS`` tokens or more cut their rows into chunks that run side by side."""
        _need(xc, "xc"); _need(dt, "dt", torch.float32); _need(dbc, "dbc", xc.dtype); _need(xz, "xz", xc.dtype); _need(state, "state", torch.float32)
        for n, t in (("dt_bias", dt_bias), ("A", a), ("D", d)):
            _need(t, n, torch.float32)
        T = xc.shape[0]
        if tuple(dt.shape) != (T, inner) or tuple(a.shape) != (inner, n_state) or xc.shape[1] != inner:
            raise KernelError("mamba1_scan: the step sizes, the decays or the convolution's output do not fit")
        out = torch.empty((T, inner), dtype=xc.dtype, device=xc.device)
        ws_state = ws_dt = None
        if (T >= self.SCAN_CHUNKED_MIN_TOKENS) if chunked is None else chunked:
            chunks = self._lib.roost_mamba1_scan_chunks(T, slots.numel())
            ws_state = torch.empty((chunks * inner * n_state,), dtype=torch.float32, device=xc.device)
            ws_dt = torch.empty((chunks * inner,), dtype=torch.float32, device=xc.device)
        self._call("roost_mamba1_scan", _ptr(xc), _ptr(dt), _ptr(dbc), dbc.stride(0), _ptr(xz), xz.stride(0), _ptr(out), _ptr(dt_bias), _ptr(a),
                   _ptr(d), _ptr(state), state.stride(0), _ptr(q_indptr), _ptr(slots), slots.numel(), T, inner, n_state, dt_rank,
                   _ptr(ws_state), _ptr(ws_dt), dtype_code(xc.dtype), _stream(), launches=3 if ws_state is not None else 1)
        return out

    def attention_set_decode_tma(self, on: bool) -> None:
        """Decode rows stream keys and values through the copy engine where the sizes allow (the default), or never."""
        self._lib.roost_attention_set_decode_tma(1 if on else 0)

    def attention_status(self) -> int:
        """The code of a bounded wait the copy-engine decode kernel gave up since the last call (0: none); synchronises."""
        return int(self._lib.roost_attention_status())

    def status_snapshot(self, out: torch.Tensor) -> None:
        """Writes the kernels' error words into ``out`` (four int32: three codes, then 1) in stream order, without
        synchronising. ``out`` is on the device or in pinned host memory: an engine that copies a step's tokens to the
        host puts the words beside them and reads both after the one wait it makes anyway."""
        if out.dtype != torch.int32 or out.numel() < 4 or not out.is_contiguous():
            raise KernelError("status_snapshot: four contiguous int32 are needed")
        if not out.is_cuda and not out.is_pinned():
            raise KernelError("status_snapshot: a host destination must be pinned memory")
        self._call("roost_status_snapshot", _ptr(out), 0 if out.is_cuda else 1, _stream())

    def check_device_status(self) -> None:
        """Raises when a kernel gave up one of its bounded waits since the last call (its results are then not valid).
        Synchronises, clears the error words and lowers the flags a weight-streaming product that gave up may have left
        raised, so that the launches after the error start clean."""
        gemm, attn = self.gemm_tcgen05_status(), self.attention_status()
        if gemm or attn:
            ws = getattr(self, "_stream_ws", None)
            if ws is not None:
                ws[1].zero_()
            raise KernelError(f"a kernel gave up a bounded wait (tcgen05 product: code {gemm}, decode attention: code {attn}); "
                              "the step's results are not valid")

    def gemm_tcgen05_set_pairs(self, on: bool) -> None:
        """Tiles on pairs of CTAs (cta_group::2, the default) or on single CTAs."""
        self._lib.roost_gemm_tcgen05_set_pairs(1 if on else 0)

    def gemm_tcgen05_status(self) -> int:
        """The code of a bounded wait the tcgen05 product gave up since the last call (0: none); synchronises."""
        return int(self._lib.roost_gemm_tcgen05_status())

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        _need(logits, "logits", torch.float32)
        R, V = logits.shape
        ids = torch.empty((R,), dtype=torch.int32, device=logits.device)
        splits = min(16, V // 8192)     # a block a span of 8192 logits or more, up to 16 blocks a row
        if splits > 1:
            ws = getattr(self, "_argmax_ws", None)
            if ws is None or ws[2].numel() < R or ws[2].device != logits.device:
                cap = max(64, R)
                ws = self._argmax_ws = (torch.empty(cap * 16, dtype=torch.float32, device=logits.device),
                                        torch.empty(cap * 16, dtype=torch.int32, device=logits.device),
                                        torch.zeros(cap, dtype=torch.int32, device=logits.device))
            self._call("roost_argmax_split", _ptr(logits), logits.stride(0), R, V, _ptr(ids), splits, _ptr(ws[0]), _ptr(ws[1]), _ptr(ws[2]),
                       _stream())
            return ids
        self._call("roost_argmax", _ptr(logits), logits.stride(0), R, V, _ptr(ids), _stream())
        return ids

    def sample(self, logits, temperature, top_k, top_p, min_p, seeds, offsets, workspace=None) -> torch.Tensor:
        _need(logits, "logits", torch.float32)
        R, V = logits.shape
        for n, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32), ("top_p", top_p, torch.float32),
                         ("min_p", min_p, torch.float32), ("seeds", seeds, torch.int64), ("offsets", offsets, torch.int64)):
            _need(t, n, dt)
            if t.numel() != R:
                raise KernelError(f"sample: {n} has {t.numel()} entries for {R} rows")
        if workspace is None:
            workspace = torch.empty((R, V), dtype=torch.float32, device=logits.device)
        ids = torch.empty((R,), dtype=torch.int32, device=logits.device)
        self._call("roost_sample", _ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k), _ptr(top_p),
                   _ptr(min_p), _ptr(seeds), _ptr(offsets), _ptr(workspace), _ptr(ids), _stream())
        return ids

    def sample_penalise(self, logits, counts, prompt_bits, row_slot, repetition, presence, frequency, mask_bits=None) -> torch.Tensor:
        """The rows of ``logits`` with the reference's repetition, frequency and presence penalties applied: counts
        [slots, vocab] int32 (the requests' output tokens so far), prompt_bits [slots, (vocab + 31) // 32] int32 (the
        prompts' tokens), row_slot [rows] int32 (-1: the row is copied as it is), the penalties float32 [rows]; then
        -inf where a token's bit in mask_bits (shaped as prompt_bits; None: every token stays) is 0."""
        _need(logits, "logits", torch.float32); _need(counts, "counts", torch.int32); _need(prompt_bits, "prompt_bits", torch.int32)
        R, V = logits.shape
        if counts.shape[1] != V or prompt_bits.shape != (counts.shape[0], (V + 31) // 32):
            raise KernelError(f"sample_penalise: counts {tuple(counts.shape)} and prompt_bits {tuple(prompt_bits.shape)} do not fit a vocabulary of {V}")
        for n, t, dt in (("row_slot", row_slot, torch.int32), ("repetition", repetition, torch.float32), ("presence", presence, torch.float32),
                         ("frequency", frequency, torch.float32)):
            _need(t, n, dt)
            if t.numel() != R:
                raise KernelError(f"sample_penalise: {n} has {t.numel()} entries for {R} rows")
        out = torch.empty((R, V), dtype=torch.float32, device=logits.device)
        if mask_bits is not None:
            _need(mask_bits, "mask_bits", torch.int32)
            if mask_bits.shape != prompt_bits.shape:
                raise KernelError("sample_penalise: mask_bits must be shaped as prompt_bits")
        self._call("roost_sample_penalise", _ptr(logits), logits.stride(0), R, V, _ptr(out), _ptr(counts), _ptr(prompt_bits), _ptr(mask_bits),
                   _ptr(row_slot), _ptr(repetition), _ptr(presence), _ptr(frequency), _stream())
        return out

    def sample_count_tokens(self, counts, row_slot, ids) -> None:
        """counts[row_slot[r], ids[r]] += 1 for the rows with a slot and a token."""
        _need(counts, "counts", torch.int32); _need(row_slot, "row_slot", torch.int32); _need(ids, "ids", torch.int32)
        if row_slot.numel() != ids.numel():
            raise KernelError("sample_count_tokens: one slot a token id is needed")
        self._call("roost_sample_count_tokens", _ptr(counts), counts.shape[1], _ptr(row_slot), _ptr(ids), ids.numel(), _stream())

    def sample_prompt_bits(self, bits_of_slot, ids) -> None:
        """Sets the bits of the token ids ``ids`` in one slot's words (int32 [(vocab + 31) // 32], a view into the table)."""
        _need(bits_of_slot, "bits", torch.int32); _need(ids, "ids", torch.int32)
        self._call("roost_sample_prompt_bits", _ptr(bits_of_slot), _ptr(ids), ids.numel(), bits_of_slot.numel() * 32, _stream())

    def sample_logprobs(self, logits, ids, top: int = 0):
        """(log-softmax of the raw logits at ids [rows] float32, the ``top`` highest raw logits' ids [rows, top] int32 and
        their log-softmax [rows, top] float32), all on the device."""
        _need(logits, "logits", torch.float32); _need(ids, "ids", torch.int32)
        R, V = logits.shape
        if ids.numel() != R or not 0 <= top <= V:
            raise KernelError(f"sample_logprobs: {ids.numel()} ids for {R} rows, or top {top} outside [0, {V}]")
        lp = torch.empty((R,), dtype=torch.float32, device=logits.device)
        top_ids = torch.empty((R, top), dtype=torch.int32, device=logits.device)
        top_vals = torch.empty((R, top), dtype=torch.float32, device=logits.device)
        self._call("roost_sample_logprobs", _ptr(logits), logits.stride(0), R, V, _ptr(ids), _ptr(lp), top, _ptr(top_ids) if top else None,
                   _ptr(top_vals) if top else None, _stream())
        return lp, top_ids, top_vals


_LIB: KernelLibrary | None = None


def load() -> KernelLibrary:
    """The process-wide library handle. Raises when no CUDA device is present or the library cannot be built."""
    global _LIB
    if _LIB is None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: roost_b200 runs on an sm_100a GPU only and has no CPU path")
        major, minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelError(f"the GPU has compute capability {major}.{minor}; the kernel library is built for sm_100a only")
        _LIB = KernelLibrary(build.library_path())
        import os
        # The bfloat16 products that go to cuBLAS through torch accumulate in 32-bit, as the reference asks of its library
        # (CUBLAS_COMPUTE_32F, kernels/src/gemm.cu:247-249). torch's default also lets a split-k product add its partial
        # sums up in bfloat16; that is switched off here, so that every sum of the bfloat16 path is a 32-bit sum.
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        # programmatic dependent launch is on unless ROOST_PDL=0: the library's kernels overlap their preambles, and the
        # weight-streaming product its first loads of weights, with the tail of the kernel before them
        _LIB.set_pdl(os.environ.get("ROOST_PDL", "1") != "0")
        _LIB.decode_cluster = os.environ.get("ROOST_DECODE_CLUSTER", "1") != "0"
    return _LIB
