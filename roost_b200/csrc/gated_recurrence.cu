// The gated linear recurrence a channel (the real-gated linear recurrent unit), in 32-bit arithmetic.
//
// Per (row, channel c), for the row's tokens in order, with the two gates' arguments given as 32-bit sums
// gates[block][token][r of the block's channels | i of the block's channels] (a batched product over the blocks of u):
//   r = sigmoid(gates_r + bias_r), i = sigmoid(gates_i + bias_i), x = decay[c] r (decay = rate softplus(lam), formed at load),
//   a = exp(-x), S <- a S + sqrt(1 - a^2) i u  with 1 - a^2 formed as -expm1(-2x) (no cancellation where a is near one),
//   out = S gelu_tanh(y), rounded once; y is column c of the row [y | x] of the input projection.
// S is read from and written back to the row's state slot. A thread a channel; the loads of a token do not depend on the
// recurrence, so the loop is unrolled and the loads of the next tokens are in flight while S advances.
#include "common.cuh"

namespace roost {

template <typename T>
__device__ __forceinline__ float recurrence_exp(float x) { return expf(x); }
template <>
__device__ __forceinline__ float recurrence_exp<float>(float x) { return exp_nearest(x); }

template <typename T>
__global__ void __launch_bounds__(128) gated_recurrence_scan_kernel(const T* __restrict__ u, const float* __restrict__ gates, const T* __restrict__ yx,
                                                                   int64_t ld_yx, T* __restrict__ out, const float* __restrict__ gate_bias,
                                                                   const float* __restrict__ decay, float* state, int64_t state_stride,
                                                                   const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots,
                                                                   int tokens, int width, int block_width) {
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int b = c / block_width, j = c % block_width;
  const float bias_r = gate_bias[(size_t)b * 2 * block_width + j], bias_i = gate_bias[(size_t)b * 2 * block_width + block_width + j];
  const float rate = decay[c];
  const int start = q_indptr[r], end = q_indptr[r + 1];
  float* sp = state + (size_t)slots[r] * state_stride + c;
  pdl_wait();
  if (end <= start) return;
  float S = *sp;
  const float* g = gates + ((size_t)b * tokens) * 2 * block_width + j;
#pragma unroll 4
  for (int t = start; t < end; ++t) {
    const float gr = g[(size_t)t * 2 * block_width] + bias_r;
    const float gi = g[(size_t)t * 2 * block_width + block_width] + bias_i;
    const float uv = to_float(u[(size_t)t * width + c]);
    const float yv = to_float(yx[(size_t)t * ld_yx + c]);
    const float x = rate / (1.0f + expf(-gr));
    const float a = recurrence_exp<T>(-x);
    const float drive = sqrtf(-expm1f(-2.0f * x)) * (uv / (1.0f + expf(-gi)));
    S = fmaf(a, S, drive);
    out[(size_t)t * width + c] = from_float<T>(S * gelu_tanh_f(yv));
  }
  *sp = S;
}

}  // namespace roost

using namespace roost;

extern "C" int roost_gated_recurrence_scan(const void* u, const float* gates, const void* yx, int64_t ld_yx, void* out, const float* gate_bias,
                                           const float* decay, float* state, int64_t state_stride, const int32_t* q_indptr,
                                           const int32_t* slots, int rows, int tokens, int width, int blocks, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && tokens >= 0 && width > 0 && blocks > 0 && width % blocks == 0, "gated_recurrence_scan: sizes do not fit");
  ROOST_REQUIRE(u && gates && yx && out && gate_bias && decay && state && q_indptr && slots, "gated_recurrence_scan: a pointer is null");
  ROOST_REQUIRE(ld_yx >= width && state_stride >= width, "gated_recurrence_scan: a row or a slot is too narrow");
  if (rows == 0 || tokens == 0) return ROOST_OK;
  dim3 grid(rows, (width + 127) / 128);
  if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "gated_recurrence_scan: too many channels");
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(gated_recurrence_scan_kernel<T>, grid, dim3(128), 0, (cudaStream_t)stream, (const T*)u, gates,
                                               (const T*)yx, ld_yx, (T*)out, gate_bias, decay, state, state_stride, q_indptr, slots, tokens, width,
                                               width / blocks));
  return check_launch("gated_recurrence_scan");
}
