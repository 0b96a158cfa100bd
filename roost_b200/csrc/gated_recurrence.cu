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

constexpr int kGrChunkTokens = 16;   // a thread a channel: short chunks give the device enough threads (2,048 tokens x 1,024 channels: 131 k)

// Which (row, chunk) the block `b` of a chunked launch takes: rows in order, each with ceil(tokens / 16) chunks. False beyond
// the step's chunks.
__device__ __forceinline__ bool recurrence_chunk_of_block(const int32_t* __restrict__ q_indptr, int rows, int b, int& r, int& k, int& chunks_of_row) {
  for (r = 0; r < rows; ++r) {
    const int n = q_indptr[r + 1] - q_indptr[r];
    chunks_of_row = (n + kGrChunkTokens - 1) / kGrChunkTokens;
    if (b < chunks_of_row) {
      k = b;
      return true;
    }
    b -= chunks_of_row;
  }
  return false;
}

// MODE 0: a thread walks its row's tokens from the slot's state and writes the state back. MODE 1: a thread walks one chunk
// from an empty state and leaves the state (ws_state[chunk][width]) and the chunk's sum of -log a (ws_decay[chunk][width]); a
// row's last chunk is skipped. MODE 2: a thread walks one chunk from ws_state[chunk] (the carry kernel put the chunk's true
// starting state there) and writes the outputs; a row's last chunk leaves the row's state in the slot.
template <typename T, int MODE>
__global__ void __launch_bounds__(128) gated_recurrence_scan_kernel(const T* __restrict__ u, const float* __restrict__ gates, const T* __restrict__ yx,
                                                                   int64_t ld_yx, T* __restrict__ out, const float* __restrict__ gate_bias,
                                                                   const float* __restrict__ decay, float* state, int64_t state_stride,
                                                                   const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots,
                                                                   int rows, int tokens, int width, int block_width, float* ws_state, float* ws_decay) {
  pdl_launch_dependents();
  int r = blockIdx.x, k = 0, chunks_of_row = 1;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  if (MODE != 0 && !recurrence_chunk_of_block(q_indptr, rows, blockIdx.x, r, k, chunks_of_row)) return;
  if (MODE == 1 && k == chunks_of_row - 1) return;       // nobody starts from the state a row's last chunk ends with
  const int b = c / block_width, j = c % block_width;
  const float bias_r = gate_bias[(size_t)b * 2 * block_width + j], bias_i = gate_bias[(size_t)b * 2 * block_width + block_width + j];
  const float rate = decay[c];
  int start = q_indptr[r], end = q_indptr[r + 1];
  if (MODE != 0) {
    start += k * kGrChunkTokens;
    end = min(end, start + kGrChunkTokens);
  }
  float* sp = state + (size_t)slots[r] * state_stride + c;
  pdl_wait();
  if (end <= start) return;
  float S = MODE == 0 ? *sp : (MODE == 1 ? 0.f : ws_state[(size_t)blockIdx.x * width + c]);
  float x_sum = 0.f;
  const float* g = gates + ((size_t)b * tokens) * 2 * block_width + j;
#pragma unroll 4
  for (int t = start; t < end; ++t) {
    const float gr = g[(size_t)t * 2 * block_width] + bias_r;
    const float gi = g[(size_t)t * 2 * block_width + block_width] + bias_i;
    const float uv = to_float(u[(size_t)t * width + c]);
    const float x = rate / (1.0f + expf(-gr));
    const float a = recurrence_exp<T>(-x);
    const float drive = sqrtf(-expm1f(-2.0f * x)) * (uv / (1.0f + expf(-gi)));
    S = fmaf(a, S, drive);
    if (MODE == 1) {
      x_sum += x;
    } else {
      const float yv = to_float(yx[(size_t)t * ld_yx + c]);
      out[(size_t)t * width + c] = from_float<T>(S * gelu_tanh_f(yv));
    }
  }
  if (MODE == 1) {
    ws_state[(size_t)blockIdx.x * width + c] = S;
    ws_decay[(size_t)blockIdx.x * width + c] = x_sum;
  } else if (MODE == 0 || k == chunks_of_row - 1) {
    *sp = S;
  }
}

// One thread a (row, channel): the row's state through its chunks in order. ws_state[chunk] holds the chunk's own state on entry
// (all but a row's last chunk) and the state the chunk starts from on exit. The slot is read, not written: the second walk of
// the row's last chunk leaves the row's final state there.
template <typename T>
__global__ void gated_recurrence_carry_kernel(const float* state, int64_t state_stride, float* __restrict__ ws_state, const float* __restrict__ ws_decay,
                                              const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= width) return;
  int first = 0;
  for (int rr = 0; rr < r; ++rr) first += (q_indptr[rr + 1] - q_indptr[rr] + kGrChunkTokens - 1) / kGrChunkTokens;
  const int chunks = (q_indptr[r + 1] - q_indptr[r] + kGrChunkTokens - 1) / kGrChunkTokens;
  if (chunks == 0) return;
  float S = state[(size_t)slots[r] * state_stride + c];
  constexpr int kBatch = 16;      // the chunks' own states and decays do not depend on S: a batch of loads in flight, then the chain
  for (int k0 = 0; k0 < chunks; k0 += kBatch) {
    float own[kBatch], dec[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const bool has = k0 + j < chunks - 1;
      own[j] = has ? ws_state[(size_t)(first + k0 + j) * width + c] : 0.f;
      dec[j] = has ? ws_decay[(size_t)(first + k0 + j) * width + c] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (k0 + j < chunks) {
        ws_state[(size_t)(first + k0 + j) * width + c] = S;                  // what chunk k0 + j starts from
        if (k0 + j < chunks - 1) S = fmaf(recurrence_exp<T>(-dec[j]), S, own[j]);
      }
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_gated_recurrence_scan_chunks(int tokens, int rows) { return (tokens + kGrChunkTokens - 1) / kGrChunkTokens + rows; }

// ws_state and ws_decay (float[chunks * width] each, chunks = roost_gated_recurrence_scan_chunks(tokens, rows)): rows are cut into
// chunks of 16 tokens that run side by side (three launches); null: every row is walked in one pass.
extern "C" int roost_gated_recurrence_scan(const void* u, const float* gates, const void* yx, int64_t ld_yx, void* out, const float* gate_bias,
                                           const float* decay, float* state, int64_t state_stride, const int32_t* q_indptr,
                                           const int32_t* slots, int rows, int tokens, int width, int blocks, float* ws_state, float* ws_decay,
                                           int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && tokens >= 0 && width > 0 && blocks > 0 && width % blocks == 0, "gated_recurrence_scan: sizes do not fit");
  ROOST_REQUIRE(u && gates && yx && out && gate_bias && decay && state && q_indptr && slots, "gated_recurrence_scan: a pointer is null");
  ROOST_REQUIRE(ld_yx >= width && state_stride >= width, "gated_recurrence_scan: a row or a slot is too narrow");
  ROOST_REQUIRE((ws_state == nullptr) == (ws_decay == nullptr), "gated_recurrence_scan: the chunked form needs both workspaces");
  if (rows == 0 || tokens == 0) return ROOST_OK;
  const int gy = (width + 127) / 128;
  if (gy > 65535) return fail(ROOST_ERR_UNSUPPORTED, "gated_recurrence_scan: too many channels");
  cudaStream_t s = (cudaStream_t)stream;
  const int bw = width / blocks;
  ROOST_DISPATCH_DTYPE(dtype, T, {
    if (ws_state == nullptr) {
      launch_kernel(gated_recurrence_scan_kernel<T, 0>, dim3(rows, gy), dim3(128), 0, s, (const T*)u, gates, (const T*)yx, ld_yx, (T*)out, gate_bias,
                    decay, state, state_stride, q_indptr, slots, rows, tokens, width, bw, ws_state, ws_decay);
    } else {
      const int chunks = roost_gated_recurrence_scan_chunks(tokens, rows);
      launch_kernel(gated_recurrence_scan_kernel<T, 1>, dim3(chunks, gy), dim3(128), 0, s, (const T*)u, gates, (const T*)yx, ld_yx, (T*)out, gate_bias,
                    decay, state, state_stride, q_indptr, slots, rows, tokens, width, bw, ws_state, ws_decay);
      launch_kernel(gated_recurrence_carry_kernel<T>, dim3(rows, gy), dim3(128), 0, s, (const float*)state, state_stride, ws_state,
                    (const float*)ws_decay, q_indptr, slots, width);
      launch_kernel(gated_recurrence_scan_kernel<T, 2>, dim3(chunks, gy), dim3(128), 0, s, (const T*)u, gates, (const T*)yx, ld_yx, (T*)out, gate_bias,
                    decay, state, state_stride, q_indptr, slots, rows, tokens, width, bw, ws_state, ws_decay);
    }
  });
  return check_launch("gated_recurrence_scan");
}
