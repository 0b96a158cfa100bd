// Activation functions of feed-forwards that are not gated, and gates that scale whole heads.
//
// xielu:          y = a_pos z^2 + z / 2 for z > 0, y = a_neg (exp(z) - 1 - z) + z / 2 for z <= 0, on the 32-bit value, rounded once.
//                 Vector form: 16 bytes a thread where the pointers and the count allow.
// head_gate_mul:  x[t, h, :] *= sigmoid(g[t, col + h]), one gate a token and head, in place.
#include "common.cuh"

namespace roost {

__device__ __forceinline__ float xielu_f(float z, float a_pos, float a_neg) {
  return z > 0.f ? fmaf(a_pos * z, z, 0.5f * z) : fmaf(a_neg, expm1f(z) - z, 0.5f * z);
}

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n, float a_pos, float a_neg) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_float<T>(xielu_f(to_float(x[i]), a_pos, a_neg));
}

template <typename T>
__global__ void xielu_vec_kernel(const T* __restrict__ x, T* __restrict__ out, size_t nvec, float a_pos, float a_neg) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  float v[Vec<T>::N];
  Vec<T>::load(x + i * Vec<T>::N, v);
#pragma unroll
  for (int j = 0; j < Vec<T>::N; ++j) v[j] = xielu_f(v[j], a_pos, a_neg);
  Vec<T>::store(out + i * Vec<T>::N, v);
}

template <typename T>
__global__ void head_gate_mul_kernel(T* __restrict__ x, const T* __restrict__ g, int64_t ld_g, int col, int heads, int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int n = heads * vdim;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float gate = 1.0f / (1.0f + expf(-to_float(g[t * ld_g + col + i / vdim])));
    x[t * n + i] = from_float<T>(to_float(x[t * n + i]) * gate);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_xielu(const void* x, void* out, int64_t n, float a_pos, float a_neg, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(n >= 0 && (n == 0 || (x && out)), "xielu: a pointer is null");
  if (n == 0) return ROOST_OK;
  const int vec = dtype == ROOST_F32 ? 4 : 8;
  if (n % vec == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0) {
    const int64_t nvec = n / vec, blocks = (nvec + 255) / 256;
    if (blocks > 2147483647LL) return fail(ROOST_ERR_UNSUPPORTED, "xielu: too many numbers for one launch");
    ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(xielu_vec_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)x, (T*)out,
                                                 (size_t)nvec, a_pos, a_neg));
    return check_launch("xielu");
  }
  const int64_t blocks = (n + 255) / 256;
  if (blocks > 2147483647LL) return fail(ROOST_ERR_UNSUPPORTED, "xielu: too many numbers for one launch");
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(xielu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const T*)x, (T*)out, (size_t)n,
                                               a_pos, a_neg));
  return check_launch("xielu");
}

extern "C" int roost_head_gate_mul(void* x, const void* g, int64_t ld_g, int col, int tokens, int heads, int vdim, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0 && col >= 0 && ld_g >= col + heads, "head_gate_mul: sizes do not fit");
  ROOST_REQUIRE(x && g, "head_gate_mul: a pointer is null");
  if (tokens == 0) return ROOST_OK;
  const int threads = heads * vdim >= 1024 ? 256 : 128;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(head_gate_mul_kernel<T>, dim3(tokens), dim3(threads), 0, (cudaStream_t)stream, (T*)x, (const T*)g, ld_g, col,
                                               heads, vdim));
  return check_launch("head_gate_mul");
}
