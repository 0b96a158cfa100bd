// The Mamba-2 recurrence over a step's rows, with the state of every request in a slot of 32-bit floats:
// [S of head 0 .. heads-1, each head_dim x state with the state index fastest | the convolution's last taps-1 inputs, each
// `channels` wide, oldest first].
//
// u is the input projection's output, a row [z (inner) | x (inner) | B (groups*state) | C (groups*state) | dt (heads)].
//   conv:       xbc[t, c] = silu(bias[c] + sum_k w[c, k] * in[t - (taps-1) + k, c]) over the channels [x | B | C]; inputs before
//               a row's first token of this step come from the request's slot (zeros for a fresh request).
//   conv_state: the slot's inputs become the last taps-1 of (old inputs, this step's inputs).
//   scan:       per (row, head): dt = softplus(dt + dt_bias), a = exp(-exp(A_log) dt); for the row's tokens in order
//               S <- a S + dt B x^T, y = S^T C + D x; head h reads group h / (heads / groups). S is read from and written to
//               the slot. 32-bit throughout; x, B, C are read in the activation dtype, y is written in 32-bit.
//   gated_group_norm: g = y * silu(z); each of `groups` equal parts of a token's g is divided by its root mean square (eps
//               inside the root) and multiplied by the weight; the output has the activation dtype.
// Rows are given by q_indptr (token range) and state_slots (slot per row); the padding rows of a captured step name a scratch
// slot. Every sum's order depends on the sizes only, never on the batch.
#include "common.cuh"

namespace roost {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

template <typename T>
__global__ void mamba2_conv_kernel(const T* __restrict__ u, int64_t ld, int col, T* __restrict__ out, const float* __restrict__ w,
                                   const float* __restrict__ bias, const float* __restrict__ state, int64_t state_stride, int conv_off,
                                   const int32_t* __restrict__ token_row, const int32_t* __restrict__ q_indptr,
                                   const int32_t* __restrict__ slots, int channels, int taps, int act) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int r = token_row[t];
  const int start = q_indptr[r];
  const float* st = state + (size_t)slots[r] * state_stride + conv_off;
  float acc = bias[c];
  pdl_wait();
  for (int k = 0; k < taps; ++k) {
    const int i = t - (taps - 1) + k;
    const float v = i >= start ? to_float(u[(size_t)i * ld + col + c]) : st[(size_t)(i - start + taps - 1) * channels + c];
    acc = fmaf(w[(size_t)c * taps + k], v, acc);
  }
  out[(size_t)t * channels + c] = from_float<T>(act ? silu_f(acc) : acc);
}

template <typename T>
__global__ void mamba2_conv_state_kernel(const T* __restrict__ u, int64_t ld, int col, float* state, int64_t state_stride, int conv_off,
                                         const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, int channels, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int start = q_indptr[r], n = q_indptr[r + 1] - start;
  if (n <= 0) return;
  const int keep = taps - 1;
  float* st = state + (size_t)slots[r] * state_stride + conv_off;
  // entry j of the new list is entry n + j of (old list, this step's inputs): a thread reads ahead of where it writes
  for (int j = 0; j < keep; ++j) {
    const int i = n + j;
    st[(size_t)j * channels + c] = i < keep ? st[(size_t)i * channels + c] : to_float(u[(size_t)(start + i - keep) * ld + col + c]);
  }
}

constexpr int kScanSlices = 4;     // threads that share a column of S: each keeps every fourth state index
constexpr int kScanChunk = 8;      // tokens whose B, C, x and dt a block stages at once

// One block per (row, head). Thread (p, s) keeps S[n][p] for n = s + 4 i in registers.
template <typename T, int NI>
__global__ void mamba2_scan_kernel(const T* __restrict__ xbc, const T* __restrict__ u, int64_t ld_u, int dt_col, float* __restrict__ y,
                                   const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                                   float* state, int64_t state_stride, const int32_t* __restrict__ q_indptr,
                                   const int32_t* __restrict__ slots, int heads, int P, int N, int groups) {
  extern __shared__ float sm[];
  constexpr int NP = NI * kScanSlices;            // state indices, padded
  float* sB = sm;                                 // [chunk][NP]
  float* sC = sB + kScanChunk * NP;               // [chunk][NP]
  float* sx = sC + kScanChunk * NP;               // [chunk][P]
  float* sdt = sx + kScanChunk * P;               // [chunk] dt, then [chunk] decay
  pdl_launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y;
  const int g = h / (heads / groups);
  const int inner = heads * P, channels = inner + 2 * groups * N;
  const int p = threadIdx.x / kScanSlices, s = threadIdx.x % kScanSlices;
  const bool live = p < P;
  const int start = q_indptr[r], end = q_indptr[r + 1];
  const float bias = dt_bias[h], rate = -expf(a_log[h]), skip = d_skip[h];
  float* Sg = state + (size_t)slots[r] * state_stride + ((size_t)h * P + (live ? p : 0)) * N;
  pdl_wait();
  if (end <= start) return;
  float S[NI];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int n = s + kScanSlices * i;
    S[i] = (live && n < N) ? Sg[n] : 0.f;
  }
  for (int t0 = start; t0 < end; t0 += kScanChunk) {
    const int nt = min(kScanChunk, end - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nt * NP; idx += blockDim.x) {
      const int tt = idx / NP, n = idx % NP;
      const T* row = xbc + (size_t)(t0 + tt) * channels + inner + (size_t)g * N;
      sB[idx] = n < N ? to_float(row[n]) : 0.f;
      sC[idx] = n < N ? to_float(row[(size_t)groups * N + n]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < nt * P; idx += blockDim.x) {
      const int tt = idx / P, pp = idx % P;
      sx[idx] = to_float(xbc[(size_t)(t0 + tt) * channels + (size_t)h * P + pp]);
    }
    if (threadIdx.x < nt) {
      const float zdt = to_float(u[(size_t)(t0 + threadIdx.x) * ld_u + dt_col + h]) + bias;
      const float dt = zdt > 20.f ? zdt : log1pf(expf(zdt));
      sdt[threadIdx.x] = dt;
      sdt[kScanChunk + threadIdx.x] = expf(rate * dt);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = sdt[tt], a = sdt[kScanChunk + tt];
      const float xv = live ? sx[tt * P + p] : 0.f;
      const float dx = dt * xv;
      const float* B = sB + tt * NP + s;
      const float* C = sC + tt * NP + s;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        S[i] = fmaf(a, S[i], dx * B[kScanSlices * i]);
        acc = fmaf(S[i], C[kScanSlices * i], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (live && s == 0) y[(size_t)(t0 + tt) * inner + (size_t)h * P + p] = fmaf(skip, xv, acc);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int n = s + kScanSlices * i;
      if (n < N) Sg[n] = S[i];
    }
  }
}

// The same walk for sizes of whole 16-byte vectors (state, head size, channel offsets), which is every model of real size:
// a block takes 16 values of a head (64 threads), thread (p, s) keeps the s-th quarter of S[.][p], a contiguous run of
// state indices, so B and C are read from shared memory 16 bytes at a time; the next 8 tokens' B, C and x arrive by
// cp.async in the activation dtype while the current 8 are walked, and are widened when read.
constexpr int kScanVecP = 16;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

//
// Long rows are cut into chunks of kScanChunkTokens tokens that run side by side (a single row of a prompt would keep two
// warps an SM busy otherwise): MODE 1 walks every chunk from a zero state and leaves the chunk's own state and the product
// of its decays; a carry kernel then gives every chunk the state it starts from, S_in(c+1) = (product of c's decays) S_in(c)
// + S_own(c), and the slot its new state; MODE 2 walks the chunks again from those states and writes y. MODE 0 is the
// walk of whole rows in one pass (decode steps and short portions). A block of MODE 1 or 2 finds its (row, chunk) by
// walking q_indptr; blocks beyond the step's chunks leave at once.
constexpr int kScanChunkTokens = 128;

template <typename T, int NI, int MODE>
__global__ void __launch_bounds__(64) mamba2_scan_vec_kernel(const T* __restrict__ xbc, const T* __restrict__ u, int64_t ld_u, int dt_col,
                                                            float* __restrict__ y, const float* __restrict__ dt_bias,
                                                            const float* __restrict__ a_log, const float* __restrict__ d_skip, float* state,
                                                            int64_t state_stride, const int32_t* __restrict__ q_indptr,
                                                            const int32_t* __restrict__ slots, int heads, int P, int N, int groups,
                                                            float* __restrict__ ws_state, float* __restrict__ ws_decay, int batch_rows) {
  constexpr int V = Vec<T>::N;                    // elements of a 16-byte piece
  constexpr int PAD = V;                          // a quarter's run is followed by one piece: the quarters fall in different banks
  constexpr int ROW = kScanSlices * (NI + PAD);   // elements of a token's B (or C) in shared memory
  __shared__ __align__(16) T sB[2][kScanChunk][ROW];
  __shared__ __align__(16) T sC[2][kScanChunk][ROW];
  __shared__ __align__(16) T sx[2][kScanChunk][kScanVecP];
  __shared__ float sdt[2][2][kScanChunk];
  __shared__ int item[2];
  pdl_launch_dependents();
  const int h = blockIdx.y, p0 = blockIdx.z * kScanVecP;
  const int g = h / (heads / groups);
  const int inner = heads * P, channels = inner + 2 * groups * N;
  const int tid = threadIdx.x;
  const int pl = tid / kScanSlices, s = tid % kScanSlices;     // the thread's value within the block, and its quarter
  const int p = p0 + pl;
  const bool live = p < P;
  int r = blockIdx.x, start, end;
  if (MODE == 0) {
    start = q_indptr[r];
    end = q_indptr[r + 1];
  } else {
    if (tid == 0) {
      int at = 0, found = -1, c = 0;
      for (int b = 0; b < batch_rows; ++b) {
        const int n = (q_indptr[b + 1] - q_indptr[b] + kScanChunkTokens - 1) / kScanChunkTokens;
        if ((int)blockIdx.x < at + n) {
          found = b;
          c = (int)blockIdx.x - at;
          break;
        }
        at += n;
      }
      item[0] = found;
      item[1] = c;
    }
    __syncthreads();
    r = item[0];
    if (r < 0) return;
    start = q_indptr[r] + item[1] * kScanChunkTokens;
    end = min(start + kScanChunkTokens, q_indptr[r + 1]);
  }
  float* Win = MODE == 0 ? nullptr : ws_state + (((size_t)blockIdx.x * heads + h) * P + (live ? p : 0)) * N;
  const float bias = dt_bias[h], rate = -expf(a_log[h]), skip = d_skip[h];
  float* Sg = state + (size_t)slots[r] * state_stride + ((size_t)h * P + (live ? p : 0)) * N;
  // pieces beyond the state's rows stay zero for the whole walk
  for (int i = tid; i < 2 * kScanChunk * ROW; i += 64) {
    (&sB[0][0][0])[i] = from_float<T>(0.f);
    (&sC[0][0][0])[i] = from_float<T>(0.f);
  }
  pdl_wait();
  if (end <= start) return;
  float S[NI];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int n = s * NI + i;
    S[i] = (MODE != 1 && live && n < N) ? (MODE == 0 ? Sg[n] : Win[n]) : 0.f;
  }
  float decays = 1.0f;
  __syncthreads();
  const int pieces_n = N / V;                      // pieces of a token's B
  const int pieces_x = kScanVecP / V;
  auto issue = [&](int t0, int buf) {
    const int nt = min(kScanChunk, end - t0);
    for (int idx = tid; idx < nt * pieces_n; idx += 64) {
      const int tt = idx / pieces_n, j = idx % pieces_n;
      const int n = j * V;
      const T* row = xbc + (size_t)(t0 + tt) * channels + inner + (size_t)g * N + n;
      const int at = (n / NI) * (NI + PAD) + n % NI;
      cp_async_16(&sB[buf][tt][at], row);
      cp_async_16(&sC[buf][tt][at], row + (size_t)groups * N);
    }
    for (int idx = tid; idx < nt * pieces_x; idx += 64) {
      const int tt = idx / pieces_x, j = idx % pieces_x;
      if (p0 + j * V < P) cp_async_16(&sx[buf][tt][j * V], xbc + (size_t)(t0 + tt) * channels + (size_t)h * P + p0 + j * V);
    }
    cp_async_commit();
  };
  auto step_sizes = [&](int t0, int buf) {
    if (tid < min(kScanChunk, end - t0)) {
      const float zdt = to_float(u[(size_t)(t0 + tid) * ld_u + dt_col + h]) + bias;
      const float dt = zdt > 20.f ? zdt : log1pf(expf(zdt));
      sdt[buf][0][tid] = dt;
      sdt[buf][1][tid] = expf(rate * dt);
    }
  };
  issue(start, 0);
  step_sizes(start, 0);
  int buf = 0;
  for (int t0 = start; t0 < end; t0 += kScanChunk, buf ^= 1) {
    const int nt = min(kScanChunk, end - t0);
    if (t0 + kScanChunk < end) {
      issue(t0 + kScanChunk, buf ^ 1);
      step_sizes(t0 + kScanChunk, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dt = sdt[buf][0][tt], a = sdt[buf][1][tt];
      const float xv = live ? to_float(sx[buf][tt][pl]) : 0.f;
      const float dx = dt * xv;
      if (MODE == 1) decays *= a;
      const T* B = &sB[buf][tt][s * (NI + PAD)];
      const T* C = &sC[buf][tt][s * (NI + PAD)];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < NI; i += V) {
        float bv[V], cv[V];
        Vec<T>::load(B + i, bv);
        Vec<T>::load(C + i, cv);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          S[i + e] = fmaf(a, S[i + e], dx * bv[e]);
          acc[e & 3] = fmaf(S[i + e], cv[e], acc[e & 3]);
        }
      }
      if (MODE != 1) {
        float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (live && s == 0) y[(size_t)(t0 + tt) * inner + (size_t)h * P + p] = fmaf(skip, xv, sum);
      }
    }
    __syncthreads();      // the buffer may be filled again
  }
  if (MODE == 2) return;
  float* dst = MODE == 0 ? Sg : Win;
  if (live) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int n = s * NI + i;
      if (n < N) dst[n] = S[i];
    }
  }
  if (MODE == 1 && tid == 0 && blockIdx.z == 0) ws_decay[(size_t)blockIdx.x * heads + h] = decays;
}

// Between the two walks of the chunks: per row and element of the state, in chunk order, the state a chunk starts from
// replaces the chunk's own in the workspace; the row's slot gets the state after its last chunk.
__global__ void mamba2_chunk_carry_kernel(float* __restrict__ ws_state, const float* __restrict__ ws_decay, float* state, int64_t state_stride,
                                          const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, int heads, int P, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const size_t per = (size_t)heads * P * N;
  const size_t e = (size_t)blockIdx.y * blockDim.x + threadIdx.x;
  if (e >= per) return;
  int first = 0;
  for (int i = 0; i < b; ++i) first += (q_indptr[i + 1] - q_indptr[i] + kScanChunkTokens - 1) / kScanChunkTokens;
  const int chunks = (q_indptr[b + 1] - q_indptr[b] + kScanChunkTokens - 1) / kScanChunkTokens;
  if (chunks == 0) return;
  const int h = (int)(e / ((size_t)P * N));
  float* slot = state + (size_t)slots[b] * state_stride + e;
  float run = *slot;
  for (int c0 = 0; c0 < chunks; c0 += 8) {        // eight chunks' values are loaded before the first is needed
    float own[8], decay[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = c0 + j < chunks;
      own[j] = in ? ws_state[(size_t)(first + c0 + j) * per + e] : 0.f;
      decay[j] = in ? ws_decay[(size_t)(first + c0 + j) * heads + h] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (c0 + j < chunks) {
        ws_state[(size_t)(first + c0 + j) * per + e] = run;
        run = fmaf(decay[j], run, own[j]);
      }
    }
  }
  *slot = run;
}

template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ u, int64_t ld_u, const float* __restrict__ w,
                                        T* __restrict__ out, int inner, int groups, float eps) {
  extern __shared__ float sm[];     // a group's values, then 32 floats of scratch
  const int gs = inner / groups;
  float* vals = sm;
  float* scratch = sm + gs;
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const int c = g * gs + i;
    const float v = y[(size_t)t * inner + c] * silu_f(to_float(u[(size_t)t * ld_u + c]));
    vals[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)gs + eps);
  for (int i = threadIdx.x; i < gs; i += blockDim.x) {
    const int c = g * gs + i;
    out[(size_t)t * inner + c] = from_float<T>(vals[i] * inv * w[c]);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_mamba2_conv(const void* u, int64_t ld, int col, void* out, const float* w, const float* bias, const float* state,
                                 int64_t state_stride, int conv_off, const int32_t* token_row, const int32_t* q_indptr, const int32_t* slots,
                                 int tokens, int channels, int taps, int act, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && channels > 0 && taps > 0 && col >= 0 && ld >= col + channels, "mamba2_conv: sizes do not fit");
  if (tokens == 0) return ROOST_OK;
  dim3 grid(tokens, (channels + 255) / 256);
  if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "mamba2_conv: too many channels");
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(mamba2_conv_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)u, ld, col, (T*)out, w,
                                               bias, state, state_stride, conv_off, token_row, q_indptr, slots, channels, taps, act));
  return check_launch("mamba2_conv");
}

extern "C" int roost_mamba2_conv_state(const void* u, int64_t ld, int col, float* state, int64_t state_stride, int conv_off,
                                       const int32_t* q_indptr, const int32_t* slots, int rows, int channels, int taps, int dtype,
                                       roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && channels > 0 && taps > 0 && col >= 0 && ld >= col + channels, "mamba2_conv_state: sizes do not fit");
  if (rows == 0 || taps == 1) return ROOST_OK;
  dim3 grid(rows, (channels + 255) / 256);
  if (grid.y > 65535) return fail(ROOST_ERR_UNSUPPORTED, "mamba2_conv_state: too many channels");
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(mamba2_conv_state_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (const T*)u, ld, col, state,
                                               state_stride, conv_off, q_indptr, slots, channels, taps));
  return check_launch("mamba2_conv_state");
}

template <typename T, int NI>
static void launch_scan(const void* xbc, const void* u, int64_t ld_u, int dt_col, float* y, const float* dt_bias, const float* a_log,
                        const float* d_skip, float* state, int64_t state_stride, const int32_t* q_indptr, const int32_t* slots, int rows,
                        int heads, int P, int N, int groups, cudaStream_t stream) {
  const int threads = ((P * kScanSlices + 31) / 32) * 32;
  const size_t smem = ((size_t)2 * kScanChunk * NI * kScanSlices + (size_t)kScanChunk * P + 2 * kScanChunk) * sizeof(float);
  launch_kernel(mamba2_scan_kernel<T, NI>, dim3(rows, heads), dim3(threads), smem, stream, (const T*)xbc, (const T*)u, ld_u, dt_col, y, dt_bias,
                a_log, d_skip, state, state_stride, q_indptr, slots, heads, P, N, groups);
}

extern "C" int roost_mamba2_scan(const void* xbc, const void* u, int64_t ld_u, int dt_col, float* y, const float* dt_bias, const float* a_log,
                                 const float* d_skip, float* state, int64_t state_stride, const int32_t* q_indptr, const int32_t* slots,
                                 int rows, int tokens, int heads, int head_dim, int state_rows, int groups, float* ws_state, float* ws_decay,
                                 int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && heads > 0 && head_dim > 0 && state_rows > 0 && groups > 0 && heads % groups == 0, "mamba2_scan: sizes do not fit");
  if (state_rows > 256) return fail(ROOST_ERR_UNSUPPORTED, "mamba2_scan: a state of more than 256 rows");
  if (head_dim > 128) return fail(ROOST_ERR_UNSUPPORTED, "mamba2_scan: heads of more than 128 values");
  if (heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "mamba2_scan: too many heads");
  if (rows == 0) return ROOST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  {
    // whole 16-byte pieces everywhere: the form that reads shared memory in vectors and prefetches
    const int vec = dtype == ROOST_F32 ? 4 : 8;
    const int inner = heads * head_dim;
    if (state_rows % vec == 0 && head_dim % vec == 0 && inner % vec == 0 && (groups * state_rows) % vec == 0 && (uintptr_t)xbc % 16 == 0 &&
        (dtype == ROOST_F32 || dtype == ROOST_BF16) && (head_dim + kScanVecP - 1) / kScanVecP <= 65535 && rows <= 65535) {
      const int zdim = (head_dim + kScanVecP - 1) / kScanVecP;
      const long long chunks = (long long)(tokens + kScanChunkTokens - 1) / kScanChunkTokens + rows;     // an upper bound
      const bool chunked = ws_state != nullptr && tokens >= 4 * kScanChunkTokens && chunks <= 65535 * 32;
#define ROOST_SCAN_VEC(NI, MODE, GRIDX)                                                                                                     \
  launch_kernel(mamba2_scan_vec_kernel<T, NI, MODE>, dim3((unsigned)(GRIDX), heads, zdim), dim3(64), 0, s, (const T*)xbc, (const T*)u, ld_u, \
                dt_col, y, dt_bias, a_log, d_skip, state, state_stride, q_indptr, slots, heads, head_dim, state_rows, groups, ws_state, ws_decay, rows)
      ROOST_DISPATCH_DTYPE(dtype, T, {
        if (!chunked) {
          if (state_rows <= 64) ROOST_SCAN_VEC(16, 0, rows);
          else if (state_rows <= 128) ROOST_SCAN_VEC(32, 0, rows);
          else ROOST_SCAN_VEC(64, 0, rows);
        } else {
          if (state_rows <= 64) ROOST_SCAN_VEC(16, 1, chunks);
          else if (state_rows <= 128) ROOST_SCAN_VEC(32, 1, chunks);
          else ROOST_SCAN_VEC(64, 1, chunks);
          const size_t per = (size_t)heads * head_dim * state_rows;
          launch_kernel(mamba2_chunk_carry_kernel, dim3(rows, (unsigned)((per + 255) / 256)), dim3(256), 0, s, ws_state, (const float*)ws_decay,
                        state, state_stride, q_indptr, slots, heads, head_dim, state_rows);
          if (state_rows <= 64) ROOST_SCAN_VEC(16, 2, chunks);
          else if (state_rows <= 128) ROOST_SCAN_VEC(32, 2, chunks);
          else ROOST_SCAN_VEC(64, 2, chunks);
        }
      });
#undef ROOST_SCAN_VEC
      return check_launch("mamba2_scan");
    }
  }
  ROOST_DISPATCH_DTYPE(dtype, T, {
    if (state_rows <= 64)
      launch_scan<T, 16>(xbc, u, ld_u, dt_col, y, dt_bias, a_log, d_skip, state, state_stride, q_indptr, slots, rows, heads, head_dim, state_rows, groups, s);
    else if (state_rows <= 128)
      launch_scan<T, 32>(xbc, u, ld_u, dt_col, y, dt_bias, a_log, d_skip, state, state_stride, q_indptr, slots, rows, heads, head_dim, state_rows, groups, s);
    else
      launch_scan<T, 64>(xbc, u, ld_u, dt_col, y, dt_bias, a_log, d_skip, state, state_stride, q_indptr, slots, rows, heads, head_dim, state_rows, groups, s);
  });
  return check_launch("mamba2_scan");
}

extern "C" int roost_mamba2_scan_chunks(int tokens, int rows) { return (tokens + kScanChunkTokens - 1) / kScanChunkTokens + rows; }

extern "C" int roost_gated_group_norm(const float* y, const void* u, int64_t ld_u, const float* w, void* out, int tokens, int inner, int groups,
                                      float eps, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && inner > 0 && groups > 0 && inner % groups == 0 && eps > 0.f && ld_u >= inner, "gated_group_norm: sizes do not fit");
  if (tokens == 0) return ROOST_OK;
  if (groups > 65535) return fail(ROOST_ERR_UNSUPPORTED, "gated_group_norm: too many groups");
  const int gs = inner / groups;
  const size_t smem = ((size_t)gs + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "gated_group_norm: a group too long for shared memory");
  const int threads = gs >= 1024 ? 512 : (gs >= 256 ? 256 : 64);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = gated_group_norm_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, dim3(tokens, groups), dim3(threads), smem, (cudaStream_t)stream, y, (const T*)u, ld_u, w, (T*)out, inner, groups, eps);
  });
  return check_launch("gated_group_norm");
}
