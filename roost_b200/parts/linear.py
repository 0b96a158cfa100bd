"""y = x W^T for a weight stored [out, in] (src/Starlings.Roost.Ops/CpuOps.cs:395-437), with a bias where a part asks for one.

float32 runs the library's FFMA product (true 32-bit, the same bits for a row whatever the batch). bfloat16
with 32-bit accumulation goes to cuBLAS through torch, the place where the reference's engine also calls a
library (kernels/src/gemm.cu:235), except where a kernel of this library is faster. ``Runtime.small_gemm`` decides for
products of at most 64 rows (decode steps): "auto" takes this library's TMA/tcgen05 kernels where they were measured
faster than cuBLAS on a B200 (the product with k split over thread-block clusters for weights of few tiles and a long k:
output and down projections of at most 8 rows; the weight-streaming product for at most 16 rows and a reduction length
of 8192 or more, or the vocabulary-sized head) and leaves the rest to cuBLAS; "stream" and "split" force those kernels
wherever they serve, "library" forces cuBLAS.
"""
from __future__ import annotations

import torch

from .base import Runtime

_MM_OUT_DTYPE = None  # does torch.mm take out_dtype on this build? decided at first use


class Linear:
    def __init__(self, runtime: Runtime, out_features: int, in_features: int):
        self.rt = runtime
        self.out_features = out_features
        self.in_features = in_features
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def load(self, weight: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        if tuple(weight.shape) != (self.out_features, self.in_features):
            raise ValueError(f"linear: weight is {tuple(weight.shape)}; expected {(self.out_features, self.in_features)}")
        self.weight = weight.to(self.rt.dtype).contiguous()
        if bias is not None:
            if bias.numel() != self.out_features:
                raise ValueError(f"linear: bias has {bias.numel()} elements; expected {self.out_features}")
            self.bias = bias.to(self.rt.dtype).contiguous()
            self.bias32 = bias.float().contiguous()

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        if self.bias is None:
            return self._product(x, out_dtype)
        # the bias joins the 32-bit sums before the one rounding: the library product's epilogue in bfloat16, a kernel over
        # the 32-bit product otherwise
        k = self.rt.kernels
        if self.rt.full_precision or (out_dtype or self.rt.dtype) != self.rt.dtype:
            return k.add_bias_(self._product(x, torch.float32), self.bias32)
        k.library_launches += 1
        return torch.addmm(self.bias, x, self.weight.t())

    def _product(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        global _MM_OUT_DTYPE
        k = self.rt.kernels
        out_dtype = out_dtype or self.rt.dtype
        if self.rt.full_precision:
            return k.gemm_simt(x, self.weight, torch.float32)
        M = x.shape[0]
        if M <= 64 and x.is_contiguous():
            policy = self.rt.small_gemm
            if policy in ("auto", "split") and getattr(k, "gemm_split_supported", None):
                choose = k.gemm_split_supported if policy == "split" else k.gemm_split_preferred
                if choose(M, self.out_features, self.in_features, x.stride(0), self.weight.stride(0)):
                    return k.gemm_split(x, self.weight, out_dtype)    # k split over thread-block clusters, tcgen05 products
            if policy == "stream" or (policy == "auto" and M <= 16 and (self.in_features >= 8192 or self.out_features >= 65536)):
                if k.gemm_stream_supported(M, self.out_features, self.in_features, x.stride(0), self.weight.stride(0)):
                    return k.gemm_stream(x, self.weight, out_dtype)   # weights streamed once by TMA, tcgen05 products
        if out_dtype == torch.bfloat16:
            k.library_launches += 1
            return torch.matmul(x, self.weight.t())
        if _MM_OUT_DTYPE is None:
            try:
                torch.mm(x[:1], self.weight[:8].t(), out_dtype=torch.float32)
                _MM_OUT_DTYPE = True
            except (TypeError, RuntimeError):
                _MM_OUT_DTYPE = False
        if _MM_OUT_DTYPE:
            k.library_launches += 1
            return torch.mm(x, self.weight.t(), out_dtype=torch.float32)
        return k.gemm_simt(x, self.weight, torch.float32)


def batched_linear_f32(rt: Runtime, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a[b] w[b]^T as 32-bit sums, [B, M, N] float32 contiguous, for a [B, M, K] (a view with a dense last dimension) and
    w [B, N, K]: what enters a recurrence's gates is not rounded to the activation dtype on its way."""
    global _BMM_OUT_DTYPE
    B, M, _ = a.shape
    out = torch.empty((B, M, w.shape[1]), dtype=torch.float32, device=a.device)
    if rt.full_precision:
        return rt.kernels.gemm_simt_batched(a, w, out)
    if _BMM_OUT_DTYPE is None:
        try:
            torch.bmm(a[:, :1], w[:, :8].transpose(1, 2), out_dtype=torch.float32)
            _BMM_OUT_DTYPE = True
        except (TypeError, RuntimeError):
            _BMM_OUT_DTYPE = False
    if _BMM_OUT_DTYPE:
        rt.kernels.library_launches += 1
        return torch.bmm(a, w.transpose(1, 2), out_dtype=torch.float32)
    return rt.kernels.gemm_simt_batched(a, w, out)


_BMM_OUT_DTYPE = None  # does torch.bmm take out_dtype on this build? decided at first use


def batched_linear(rt: Runtime, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[b] = a[b] w[b]^T for a [B, M, K], w [B, N, K] (contiguous) and out [B, M, N]; ``a`` and ``out`` may be views whose
    rows and batches are strided (heads side by side in a token's row) as long as their last dimension is dense: no
    operand is copied. float32 runs the library's FFMA product over the batch, bfloat16 cuBLAS's strided batched product
    with 32-bit accumulation."""
    if rt.full_precision:
        return rt.kernels.gemm_simt_batched(a, w, out)
    rt.kernels.library_launches += 1
    return torch.bmm(a, w.transpose(1, 2), out=out)
