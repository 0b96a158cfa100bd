// The Mamba selective scan over a step's rows, with the state of every request in a slot of 32-bit floats:
// [S: inner x state with the state index fastest | the convolution's last taps-1 inputs] (the convolution and its state are the
// kernels of mamba2.cu, which take any channel range).
//
//   scan: per (row, channel c), for the row's tokens in order: dt = softplus(dt_raw[t, c] + dt_bias[c]);
//         S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x[t, c] B[t, n];  y = sum_n S[c, n] C[t, n] + D[c] x[t, c];
//         out[t, c] = y * silu(z[t, c]), rounded once. A is given as it enters the decay (negative), dt_raw is the step
//         projection's 32-bit output, x the convolution's output, [dt | B | C] rows of the projection of x, z the second half
//         of the input projection's rows. S is read from and written to the row's slot. 32-bit throughout.
// A channel's state is shared by L adjacent lanes (L a power of two, each lane keeps 8 state indices in registers); a block
// of 128 threads takes 128 / L channels and stages 8 (decode steps) or 32 tokens of B, C, dt and x at a time. The float32 form computes the decay
// exp(dt A) with a reduced-argument polynomial rounded to nearest instead of the special-function unit's exponential: that
// unit's error (up to 2 units in the last place) leans one way for the small arguments of slow decays, and a state multiplied by
// it a thousand times in a row drifts by that lean times a thousand, far above the rounding of everything else. Rows are given by q_indptr (token
// range) and slots; the padding rows of a captured step name a scratch slot. Every sum's order depends on the sizes only.
//
// Steps of many tokens cut every row into chunks of 64 tokens that run side by side (three launches): each chunk but a row's
// last walks its tokens from an empty state and leaves that state and the sum of its step sizes a channel; one thread a
// (row, channel, state index) then carries the row's state from chunk to chunk, S <- exp(A sum dt) S + chunk's state, leaving every
// chunk's true starting state in its place and the row's final state in the slot; a second walk of every chunk from its
// starting state writes the outputs.
#include "common.cuh"

namespace roost {

constexpr int kM1Threads = 128;
constexpr int kM1Chunk = 8;          // tokens staged at once by a block that walks a decode step's rows
constexpr int kM1ChunkLong = 32;     // ... and by a block that walks many tokens: four times fewer waits for the staged loads
constexpr int kM1PerLane = 8;

template <typename T>
__device__ __forceinline__ float decay_exp(float x) { return expf(x); }
template <>
__device__ __forceinline__ float decay_exp<float>(float x) { return exp_nearest(x); }

constexpr int kM1ChunkTokens = 64;

// Which (row, chunk) the block `b` of a chunked launch takes: rows in order, each with ceil(tokens / 64) chunks. False beyond
// the step's chunks.
__device__ __forceinline__ bool chunk_of_block(const int32_t* __restrict__ q_indptr, int rows, int b, int& r, int& k, int& chunks_of_row) {
  for (r = 0; r < rows; ++r) {
    const int n = q_indptr[r + 1] - q_indptr[r];
    chunks_of_row = (n + kM1ChunkTokens - 1) / kM1ChunkTokens;
    if (b < chunks_of_row) {
      k = b;
      return true;
    }
    b -= chunks_of_row;
  }
  return false;
}

// MODE 0: a block walks its row's tokens from the slot's state and writes the state back. MODE 1: a block walks one chunk from
// an empty state and leaves the state (ws_state[chunk][inner][N]) and the chunk's sum of step sizes (ws_dt[chunk][inner]); a
// row's last chunk is skipped. MODE 2: a block walks one chunk from ws_state[chunk] and writes the outputs; a row's last chunk
// also writes the state it ends with to the slot.
template <typename T, int MODE>
__global__ void __launch_bounds__(kM1Threads) mamba1_scan_kernel(const T* __restrict__ xc, const float* __restrict__ dt_raw, const T* __restrict__ dbc,
                                                                int64_t ld_dbc, const T* __restrict__ xz, int64_t ld_xz, T* __restrict__ out,
                                                                const float* __restrict__ dt_bias, const float* __restrict__ a_neg,
                                                                const float* __restrict__ d_skip, float* state, int64_t state_stride,
                                                                const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, int inner,
                                                                int N, int R, int L, int rows, float* __restrict__ ws_state,
                                                                float* __restrict__ ws_dt, int stage_tokens) {
  extern __shared__ float sm[];
  const int NP = L * kM1PerLane;                 // state indices, padded
  const int CPB = kM1Threads / L;                // channels a block
  float* sB = sm;                                // [chunk][NP]
  float* sC = sB + stage_tokens * NP;            // [chunk][NP]
  float* sdt = sC + stage_tokens * NP;           // [chunk][CPB]
  float* sx = sdt + stage_tokens * CPB;          // [chunk][CPB]
  float* sy = sx + stage_tokens * CPB;           // [chunk][CPB]
  pdl_launch_dependents();
  int r = blockIdx.x, k = 0, chunks_of_row = 1;
  if (MODE != 0 && !chunk_of_block(q_indptr, rows, blockIdx.x, r, k, chunks_of_row)) return;
  if (MODE == 1 && k == chunks_of_row - 1) return;       // nobody starts from the state a row's last chunk ends with
  const int c0 = blockIdx.y * CPB;
  const int cl = threadIdx.x / L, j = threadIdx.x % L;
  const int c = c0 + cl;
  const bool live = c < inner;
  const int n0 = j * kM1PerLane;
  const int start = q_indptr[r] + (MODE != 0 ? k * kM1ChunkTokens : 0);
  const int end = MODE != 0 ? min(start + kM1ChunkTokens, q_indptr[r + 1]) : q_indptr[r + 1];
  float a[kM1PerLane], S[kM1PerLane];
#pragma unroll
  for (int i = 0; i < kM1PerLane; ++i) a[i] = (live && n0 + i < N) ? a_neg[(size_t)c * N + n0 + i] : 0.f;
  const float skip = live ? d_skip[c] : 0.f;
  float* Sg = MODE == 0 ? state + (size_t)slots[r] * state_stride + (size_t)(live ? c : 0) * N
                        : ws_state + ((size_t)blockIdx.x * inner + (live ? c : 0)) * N;
  pdl_wait();
  if (end <= start) return;
  float dt_sum = 0.f;
#pragma unroll
  for (int i = 0; i < kM1PerLane; ++i) S[i] = (MODE != 1 && live && n0 + i < N) ? Sg[n0 + i] : 0.f;
  for (int t0 = start; t0 < end; t0 += stage_tokens) {
    const int nt = min(stage_tokens, end - t0);
    __syncthreads();
#pragma unroll 4      // several loads in flight a thread: a stage's time is its loads' latency
    for (int idx = threadIdx.x; idx < nt * NP; idx += kM1Threads) {
      const int tt = idx / NP, n = idx % NP;
      const T* row = dbc + (size_t)(t0 + tt) * ld_dbc + R;
      sB[idx] = n < N ? to_float(row[n]) : 0.f;
      sC[idx] = n < N ? to_float(row[N + n]) : 0.f;
    }
#pragma unroll 4
    for (int idx = threadIdx.x; idx < nt * CPB; idx += kM1Threads) {
      const int tt = idx / CPB, cc = c0 + idx % CPB;
      float dt = 0.f, x = 0.f;
      if (cc < inner) {
        const float zdt = dt_raw[(size_t)(t0 + tt) * inner + cc] + dt_bias[cc];
        dt = zdt > 20.f ? zdt : log1pf(expf(zdt));
        x = to_float(xc[(size_t)(t0 + tt) * inner + cc]);
      }
      sdt[idx] = dt;
      sx[idx] = x;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = sdt[tt * CPB + cl], x = sx[tt * CPB + cl];
      const float dx = dt * x;
      if (MODE == 1) dt_sum += dt;
      const float* B = sB + tt * NP + n0;
      const float* C = sC + tt * NP + n0;
      float y = 0.f;
#pragma unroll
      for (int i = 0; i < kM1PerLane; ++i) {
        S[i] = fmaf(decay_exp<T>(dt * a[i]), S[i], dx * B[i]);
        y = fmaf(S[i], C[i], y);
      }
      if (MODE == 1) continue;
      for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (j == 0) sy[tt * CPB + cl] = fmaf(skip, x, y);
    }
    if (MODE == 1) continue;
    __syncthreads();
#pragma unroll 4
    for (int idx = threadIdx.x; idx < nt * CPB; idx += kM1Threads) {
      const int tt = idx / CPB, cc = c0 + idx % CPB;
      if (cc < inner) {
        const float z = to_float(xz[(size_t)(t0 + tt) * ld_xz + inner + cc]);
        out[(size_t)(t0 + tt) * inner + cc] = from_float<T>(sy[idx] * (z / (1.0f + expf(-z))));
      }
    }
  }
  if (live && (MODE != 2 || k == chunks_of_row - 1)) {      // the second walk of a row's last chunk ends with the row's state
    float* dst = MODE == 2 ? state + (size_t)slots[r] * state_stride + (size_t)c * N : Sg;
#pragma unroll
    for (int i = 0; i < kM1PerLane; ++i)
      if (n0 + i < N) dst[n0 + i] = S[i];
    if (MODE == 1 && j == 0) ws_dt[(size_t)blockIdx.x * inner + c] = dt_sum;
  }
}

// One thread a (row, channel, state index): the row's state through its chunks in order. ws_state[chunk] holds the chunk's own
// state on entry (all but a row's last chunk) and the state the chunk starts from on exit. The slot is read, not written: the
// second walk of the row's last chunk leaves the row's final state there.
template <typename T>
__global__ void mamba1_carry_kernel(float* state, int64_t state_stride, float* __restrict__ ws_state, const float* __restrict__ ws_dt,
                                    const float* __restrict__ a_neg, const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots,
                                    int inner, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int idx = blockIdx.y * blockDim.x + threadIdx.x;
  if (idx >= inner * N) return;
  const int c = idx / N;
  int first = 0;
  for (int rr = 0; rr < r; ++rr) first += (q_indptr[rr + 1] - q_indptr[rr] + kM1ChunkTokens - 1) / kM1ChunkTokens;
  const int chunks = (q_indptr[r + 1] - q_indptr[r] + kM1ChunkTokens - 1) / kM1ChunkTokens;
  if (chunks == 0) return;
  const float a = a_neg[idx];
  float S = state[(size_t)slots[r] * state_stride + idx];
#pragma unroll 4      // the chunks' own states and step sums do not depend on S: several loads in flight
  for (int k = 0; k < chunks; ++k) {
    float* w = ws_state + ((size_t)(first + k) * inner) * N + idx;
    const float own = k < chunks - 1 ? *w : 0.f;
    *w = S;                                                                  // what chunk k starts from
    if (k < chunks - 1) S = fmaf(decay_exp<T>(a * ws_dt[(size_t)(first + k) * inner + c]), S, own);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_mamba1_scan_chunks(int tokens, int rows) { return (tokens + kM1ChunkTokens - 1) / kM1ChunkTokens + rows; }

// ws_state (float[chunks * inner * n_state]) and ws_dt (float[chunks * inner]), chunks = roost_mamba1_scan_chunks(tokens, rows):
// rows are cut into chunks that run side by side; null: every row is walked in one pass.
extern "C" int roost_mamba1_scan(const void* xc, const float* dt_raw, const void* dbc, int64_t ld_dbc, const void* xz, int64_t ld_xz, void* out,
                                 const float* dt_bias, const float* a_neg, const float* d_skip, float* state, int64_t state_stride,
                                 const int32_t* q_indptr, const int32_t* slots, int rows, int tokens, int inner, int n_state, int dt_rank,
                                 float* ws_state, float* ws_dt, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && tokens >= 0 && inner > 0 && n_state > 0 && dt_rank > 0, "mamba1_scan: sizes must be positive");
  ROOST_REQUIRE(xc && dt_raw && dbc && xz && out && dt_bias && a_neg && d_skip && state && q_indptr && slots, "mamba1_scan: a pointer is null");
  ROOST_REQUIRE(ld_dbc >= dt_rank + 2 * n_state && ld_xz >= 2 * inner && state_stride >= (int64_t)inner * n_state,
                "mamba1_scan: a row or a slot is too narrow");
  ROOST_REQUIRE((ws_state == nullptr) == (ws_dt == nullptr), "mamba1_scan: the chunked form needs both workspaces");
  if (n_state > 32 * kM1PerLane) return fail(ROOST_ERR_UNSUPPORTED, "mamba1_scan: a state beyond 256 numbers a channel");
  if (rows == 0 || tokens == 0) return ROOST_OK;
  int L = 1;
  while (L * kM1PerLane < n_state) L *= 2;
  const int cpb = kM1Threads / L;
  const int gy = (inner + cpb - 1) / cpb;
  if (gy > 65535 || rows > 65535) return fail(ROOST_ERR_UNSUPPORTED, "mamba1_scan: too many channels or rows");
  // steps of more tokens than rows stage 32 tokens at a time where that fits the default shared memory
  int stage = kM1Chunk;
  if (tokens > rows && ((size_t)2 * kM1ChunkLong * L * kM1PerLane + (size_t)3 * kM1ChunkLong * cpb) * sizeof(float) <= 48 * 1024) stage = kM1ChunkLong;
  const size_t smem = ((size_t)2 * stage * L * kM1PerLane + (size_t)3 * stage * cpb) * sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
  if (ws_state != nullptr) {
    const int chunks = roost_mamba1_scan_chunks(tokens, rows);
    ROOST_DISPATCH_DTYPE(dtype, T, {
      launch_kernel(mamba1_scan_kernel<T, 1>, dim3(chunks, gy), dim3(kM1Threads), smem, s, (const T*)xc, dt_raw, (const T*)dbc, ld_dbc, (const T*)xz,
                    ld_xz, (T*)out, dt_bias, a_neg, d_skip, state, state_stride, q_indptr, slots, inner, n_state, dt_rank, L, rows, ws_state, ws_dt, stage);
      launch_kernel(mamba1_carry_kernel<T>, dim3(rows, (inner * n_state + 255) / 256), dim3(256), 0, s, state, state_stride, ws_state,
                    (const float*)ws_dt, a_neg, q_indptr, slots, inner, n_state);
      launch_kernel(mamba1_scan_kernel<T, 2>, dim3(chunks, gy), dim3(kM1Threads), smem, s, (const T*)xc, dt_raw, (const T*)dbc, ld_dbc, (const T*)xz,
                    ld_xz, (T*)out, dt_bias, a_neg, d_skip, state, state_stride, q_indptr, slots, inner, n_state, dt_rank, L, rows, ws_state, ws_dt, stage);
    });
    return check_launch("mamba1_scan");
  }
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(mamba1_scan_kernel<T, 0>, dim3(rows, gy), dim3(kM1Threads), smem, s, (const T*)xc,
                                               dt_raw, (const T*)dbc, ld_dbc, (const T*)xz, ld_xz, (T*)out, dt_bias, a_neg, d_skip, state,
                                               state_stride, q_indptr, slots, inner, n_state, dt_rank, L, rows, (float*)nullptr, (float*)nullptr, stage));
  return check_launch("mamba1_scan");
}
