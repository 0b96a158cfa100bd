// A matrix memory a head with exponential gates (the mLSTM cell), in 32-bit arithmetic.
//
// Per (row, head), for the row's tokens in order, with q, k (dim numbers) and v (vdim numbers) from the row [q | k | v | ...] of
// the input projection and the two gates' arguments a head as 32-bit sums [i of every head | f of every head]:
//   i = c tanh(gi / c), f = logsigmoid(c tanh(gf / c)), m' = max(f + m, i), keep = exp(f + m - m'), take = exp(i - m'),
//   S <- keep S + take k v^T, n <- keep n + take k, o = S^T (q / sqrt(dim)) / (max(|n . q / sqrt(dim)|, exp(-m')) + floor).
// The slot holds, head after head, [S: dim x vdim | n: dim | m].
//
// scan: one warp (a block) per (row, head, 32 columns of S). A lane keeps its column of S in registers (dim up to 128) or in
// shared memory (beyond), and the entries lane, lane + 32, ... of n; a token's (take k, q) are staged in shared memory once
// and read by all lanes; n . q is a warp sum. The next token's q, k, v and gates are loaded while the current one is
// multiplied. Every warp of a head keeps n and m for itself; the first writes them back.
//
// Steps of many tokens cut every row into chunks of 64 tokens that run side by side (three launches). With F the sum of a chunk's
// f, a chunk walked from an empty memory (S = 0, n = 0, m = -inf) ends with (S', n', m'), and a memory (S, n, m) before the chunk
// is (e^(F + m - M) S + e^(m' - M) S', likewise n, M = max(F + m, m')) after it: the first walk leaves every chunk's own
// (S', n', m', F), one thread an entry then carries the row's memory from chunk to chunk leaving every chunk's true starting
// memory in its place, and a second walk of every chunk from there writes the outputs and, from a row's last chunk, the slot.
//
// head_norm_gate: per token and head, o / sqrt(mean(o^2) + eps) * w * sigmoid(g) (w may be absent; with gate_silu the gate is
// g sigmoid(g)), rounded once.
#include "common.cuh"

namespace roost {

template <typename T>
__device__ __forceinline__ float memory_exp(float x) { return expf(x); }
template <>
__device__ __forceinline__ float memory_exp<float>(float x) { return exp_nearest(x); }

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

constexpr int kMmChunkTokens = 64;

// Which (row, chunk) the block `b` of a chunked launch takes: rows in order, each with ceil(tokens / 64) chunks. False beyond
// the step's chunks.
__device__ __forceinline__ bool memory_chunk_of_block(const int32_t* __restrict__ q_indptr, int rows, int b, int& r, int& k, int& chunks_of_row) {
  for (r = 0; r < rows; ++r) {
    const int n = q_indptr[r + 1] - q_indptr[r];
    chunks_of_row = (n + kMmChunkTokens - 1) / kMmChunkTokens;
    if (b < chunks_of_row) {
      k = b;
      return true;
    }
    b -= chunks_of_row;
  }
  return false;
}

// A chunk's place in the workspace, head after head: [S: dim x vdim | n: dim | m' | F | the m the chunk starts from].
__device__ __forceinline__ size_t memory_ws_head(int dim, int vdim) { return (size_t)dim * vdim + dim + 3; }

// DREG > 0: S in registers, dim <= DREG. DREG == 0: S in shared memory after the staging area, [dim][32].
// MODE 0: a warp walks its row's tokens from the slot and writes the slot back. MODE 1: a warp walks one chunk from an empty
// memory and leaves (S', n', m', F) in ws[chunk]; a row's last chunk is skipped. MODE 2: a warp walks one chunk from ws[chunk]
// (the carry kernel put the chunk's true starting memory there) and writes the outputs; a row's last chunk writes the slot.
template <typename T, int DREG, int MODE>
__global__ void __launch_bounds__(32) matrix_memory_scan_kernel(const T* __restrict__ qkv, int64_t ld, const float* __restrict__ gates,
                                                               float* __restrict__ out, float* state, int64_t state_stride,
                                                               const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, int rows,
                                                               int heads, int dim, int vdim, float cap, float floor_, float* ws) {
  extern __shared__ float sm[];      // two staging slots of dim (take k, q) pairs; then S when it does not live in registers
  constexpr int NREG = DREG > 0 ? DREG : 1;
  constexpr int NN = DREG > 0 ? DREG / 32 : 32;          // entries of n a lane keeps (dim <= 1024 in shared-memory form)
  pdl_launch_dependents();
  int r = blockIdx.x, k = 0, chunks_of_row = 1;
  const int h = blockIdx.y, slice = blockIdx.z;
  const int lane = threadIdx.x;
  const int col = slice * 32 + lane;
  const bool live = col < vdim;
  if (MODE != 0 && !memory_chunk_of_block(q_indptr, rows, blockIdx.x, r, k, chunks_of_row)) return;
  if (MODE == 1 && k == chunks_of_row - 1) return;       // nobody starts from the memory a row's last chunk ends with
  int start = q_indptr[r], end = q_indptr[r + 1];
  if (MODE != 0) {
    start += k * kMmChunkTokens;
    end = min(end, start + kMmChunkTokens);
  }
  float* slot = state + (size_t)slots[r] * state_stride + (size_t)h * ((size_t)dim * vdim + dim + 1);
  float* wsh = MODE != 0 ? ws + ((size_t)blockIdx.x * heads + h) * memory_ws_head(dim, vdim) : nullptr;
  const float* hs = MODE == 0 ? slot : wsh;               // where the walk starts from (MODE 1 starts empty)
  float* S_sm = sm + 4 * dim + lane;                       // [dim][32], used when DREG == 0
  const float inv_cap = 1.0f / cap, q_scale = rsqrtf((float)dim);
  const int QK = heads * dim;
  pdl_wait();
  if (end <= start) return;
  float S[NREG], n[NN];
  if (DREG > 0) {
#pragma unroll
    for (int d = 0; d < NREG; ++d) S[d] = (MODE != 1 && live && d < dim) ? hs[(size_t)d * vdim + col] : 0.f;
  } else {
    for (int d = 0; d < dim; ++d) S_sm[(size_t)d * 32] = (MODE != 1 && live) ? hs[(size_t)d * vdim + col] : 0.f;
  }
#pragma unroll
  for (int i = 0; i < NN; ++i) {
    const int d = lane + 32 * i;
    n[i] = (MODE != 1 && d < dim) ? hs[(size_t)dim * vdim + d] : 0.f;
  }
  float m = MODE == 0 ? hs[(size_t)dim * vdim + dim] : (MODE == 1 ? -INFINITY : hs[(size_t)dim * vdim + dim + 2]);
  float f_sum = 0.f;

  // the next token's inputs, loaded one token ahead
  float nk[NN], nq[NN], nv, ngi, ngf;
  auto load = [&](int t) {
    const T* row = qkv + (size_t)t * ld;
#pragma unroll
    for (int i = 0; i < NN; ++i) {
      const int d = lane + 32 * i;
      nq[i] = d < dim ? to_float(row[(size_t)h * dim + d]) * q_scale : 0.f;
      nk[i] = d < dim ? to_float(row[QK + (size_t)h * dim + d]) : 0.f;
    }
    nv = live ? to_float(row[2 * QK + (size_t)h * vdim + col]) : 0.f;
    ngi = gates[(size_t)t * 2 * heads + h];
    ngf = gates[(size_t)t * 2 * heads + heads + h];
  };
  load(start);
  for (int t = start; t < end; ++t) {
    const float gi = cap * tanhf(ngi * inv_cap);
    const float gf = log_sigmoid_f(cap * tanhf(ngf * inv_cap));
    const float m_new = fmaxf(gf + m, gi);
    const float keep = memory_exp<T>(gf + m - m_new), take = memory_exp<T>(gi - m_new);
    m = m_new;
    if (MODE == 1) f_sum += gf;
    float2* stage = reinterpret_cast<float2*>(sm) + (size_t)(t & 1) * dim;
    float nq_part = 0.f;
#pragma unroll
    for (int i = 0; i < NN; ++i) {
      const int d = lane + 32 * i;
      if (d < dim) {
        const float tk = take * nk[i];
        stage[d] = make_float2(tk, nq[i]);
        n[i] = fmaf(keep, n[i], tk);
        nq_part = fmaf(n[i], nq[i], nq_part);
      }
    }
    const float v = nv;
    if (t + 1 < end) load(t + 1);
    __syncwarp();
    float num = 0.f;
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < NREG; ++d) {
        if (d < dim) {
          const float2 kq = stage[d];
          S[d] = fmaf(keep, S[d], kq.x * v);
          num = fmaf(S[d], kq.y, num);
        }
      }
    } else {
      for (int d = 0; d < dim; ++d) {
        const float2 kq = stage[d];
        const float s = fmaf(keep, S_sm[(size_t)d * 32], kq.x * v);
        S_sm[(size_t)d * 32] = s;
        num = fmaf(s, kq.y, num);
      }
    }
    if (MODE != 1) {
      const float den = fmaxf(fabsf(warp_sum(nq_part)), memory_exp<T>(-m)) + floor_;
      if (live) out[(size_t)t * heads * vdim + (size_t)h * vdim + col] = num / den;
    }
  }
  if (MODE == 2 && k != chunks_of_row - 1) return;
  float* hd = MODE == 1 ? wsh : slot;                     // where the walk's end goes
  if (live) {
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < NREG; ++d)
        if (d < dim) hd[(size_t)d * vdim + col] = S[d];
    } else {
      for (int d = 0; d < dim; ++d) hd[(size_t)d * vdim + col] = S_sm[(size_t)d * 32];
    }
  }
  if (slice == 0) {
#pragma unroll
    for (int i = 0; i < NN; ++i) {
      const int d = lane + 32 * i;
      if (d < dim) hd[(size_t)dim * vdim + d] = n[i];
    }
    if (lane == 0) {
      hd[(size_t)dim * vdim + dim] = m;
      if (MODE == 1) hd[(size_t)dim * vdim + dim + 1] = f_sum;
    }
  }
}

// One thread an entry of S or n of a (row, head): the row's memory through its chunks in order. ws[chunk] holds the chunk's own
// (S', n', m', F) on entry (all but a row's last chunk) and the memory the chunk starts from on exit (its m in a place of its
// own: the other threads still read m'). The slot is read, not written: the second walk of the row's last chunk writes it.
template <typename T>
__global__ void matrix_memory_carry_kernel(const float* state, int64_t state_stride, float* ws, const int32_t* __restrict__ q_indptr,
                                           const int32_t* __restrict__ slots, int heads, int dim, int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int idx = blockIdx.z * blockDim.x + threadIdx.x;
  const int entries = dim * vdim + dim;
  if (idx >= entries) return;
  int first = 0;
  for (int rr = 0; rr < r; ++rr) first += (q_indptr[rr + 1] - q_indptr[rr] + kMmChunkTokens - 1) / kMmChunkTokens;
  const int chunks = (q_indptr[r + 1] - q_indptr[r] + kMmChunkTokens - 1) / kMmChunkTokens;
  if (chunks == 0) return;
  const float* slot = state + (size_t)slots[r] * state_stride + (size_t)h * ((size_t)entries + 1);
  float e = slot[idx], m = slot[entries];
  constexpr int kBatch = 8;       // the chunks' own entries, maxima and sums do not depend on e: a batch of loads in flight, then the chain
  const size_t stride = (size_t)heads * memory_ws_head(dim, vdim);
  float* w0 = ws + ((size_t)first * heads + h) * memory_ws_head(dim, vdim);
  for (int k0 = 0; k0 < chunks; k0 += kBatch) {
    float own[kBatch], m_own[kBatch], f[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const bool has = k0 + j < chunks - 1;
      const float* w = w0 + (size_t)(k0 + j) * stride;
      own[j] = has ? w[idx] : 0.f;
      m_own[j] = has ? w[entries] : 0.f;
      f[j] = has ? w[entries + 1] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (k0 + j < chunks) {
        float* w = w0 + (size_t)(k0 + j) * stride;
        w[idx] = e;                                                          // what chunk k0 + j starts from
        if (idx == 0) w[entries + 2] = m;
        if (k0 + j < chunks - 1) {
          const float m_new = fmaxf(f[j] + m, m_own[j]);
          e = fmaf(memory_exp<T>(f[j] + m - m_new), e, memory_exp<T>(m_own[j] - m_new) * own[j]);
          m = m_new;
        }
      }
    }
  }
}

template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ u, int64_t ld_u, int col, const float* __restrict__ w,
                                      T* __restrict__ out, int heads, int vdim, float eps, int gate_silu) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int h = warp; h < heads; h += nwarps) {
    const float* x = o + (t * heads + h) * vdim;
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
      const size_t c = (size_t)h * vdim + i;
      const float g = to_float(u[t * ld_u + col + c]);
      const float y = x[i] * inv * (w != nullptr ? w[c] : 1.0f) / (1.0f + expf(-g));
      out[t * heads * vdim + c] = from_float<T>(gate_silu ? y * g : y);
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_matrix_memory_scan_chunks(int tokens, int rows) { return (tokens + kMmChunkTokens - 1) / kMmChunkTokens + rows; }

// ws (float[chunks * heads * (dim * vdim + dim + 3)], chunks = roost_matrix_memory_scan_chunks(tokens, rows)): rows are cut into chunks
// that run side by side (three launches); null: every row is walked in one pass.
extern "C" int roost_matrix_memory_scan(const void* qkv, int64_t ld, const float* gates, float* out, float* state, int64_t state_stride,
                                        const int32_t* q_indptr, const int32_t* slots, int rows, int tokens, int heads, int dim, int vdim,
                                        float cap, float floor_, float* ws, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && tokens >= 0 && heads > 0 && dim > 0 && vdim > 0 && cap > 0.f && floor_ >= 0.f,
                "matrix_memory_scan: sizes and the cap must be positive");
  ROOST_REQUIRE(qkv && gates && out && state && q_indptr && slots, "matrix_memory_scan: a pointer is null");
  ROOST_REQUIRE(ld >= (int64_t)heads * (2 * dim + vdim) && state_stride >= (int64_t)heads * ((int64_t)dim * vdim + dim + 1),
                "matrix_memory_scan: a row or a slot is too narrow");
  if (dim > 1024) return fail(ROOST_ERR_UNSUPPORTED, "matrix_memory_scan: heads of more than 1024 keys");
  const int slices = (vdim + 31) / 32;
  if (heads > 65535 || slices > 65535) return fail(ROOST_ERR_UNSUPPORTED, "matrix_memory_scan: too many heads or values");
  if (rows == 0 || tokens == 0) return ROOST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t stage = (size_t)4 * dim * sizeof(float);
  const int chunks = roost_matrix_memory_scan_chunks(tokens, rows);
#define ROOST_MM_LAUNCH(DREG, MODE, SMEM, GX)                                                                                                     \
  do {                                                                                                                                            \
    auto kernel = matrix_memory_scan_kernel<T, DREG, MODE>;                                                                                       \
    if ((SMEM) > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM));                               \
    launch_kernel(kernel, dim3((GX), heads, slices), dim3(32), (SMEM), s, (const T*)qkv, ld, gates, out, state, state_stride, q_indptr, slots,   \
                  rows, heads, dim, vdim, cap, floor_, ws);                                                                                       \
  } while (0)
#define ROOST_MM_SCAN(DREG, SMEM)                                                                                                                 \
  do {                                                                                                                                            \
    if (ws == nullptr) {                                                                                                                          \
      ROOST_MM_LAUNCH(DREG, 0, SMEM, rows);                                                                                                       \
    } else {                                                                                                                                      \
      ROOST_MM_LAUNCH(DREG, 1, SMEM, chunks);                                                                                                     \
      launch_kernel(matrix_memory_carry_kernel<T>, dim3(rows, heads, (dim * vdim + dim + 255) / 256), dim3(256), 0, s, (const float*)state,       \
                    state_stride, ws, q_indptr, slots, heads, dim, vdim);                                                                         \
      ROOST_MM_LAUNCH(DREG, 2, SMEM, chunks);                                                                                                     \
    }                                                                                                                                             \
  } while (0)
  ROOST_DISPATCH_DTYPE(dtype, T, {
    if (dim <= 32) ROOST_MM_SCAN(32, stage);
    else if (dim <= 64) ROOST_MM_SCAN(64, stage);
    else if (dim <= 128) ROOST_MM_SCAN(128, stage);
    else ROOST_MM_SCAN(0, stage + (size_t)dim * 32 * sizeof(float));
  });
#undef ROOST_MM_SCAN
#undef ROOST_MM_LAUNCH
  return check_launch("matrix_memory_scan");
}

extern "C" int roost_head_norm_gate(const float* o, const void* u, int64_t ld_u, int col, const float* w, void* out, int tokens, int heads, int vdim,
                                    float eps, int gate_silu, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0 && eps > 0.f && col >= 0 && ld_u >= col + (int64_t)heads * vdim, "head_norm_gate: sizes do not fit");
  ROOST_REQUIRE(o && u && out, "head_norm_gate: a pointer is null");
  if (tokens == 0) return ROOST_OK;
  const int threads = heads >= 8 ? 256 : (heads >= 4 ? 128 : 32 * heads);
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(head_norm_gate_kernel<T>, dim3(tokens), dim3(threads), 0, (cudaStream_t)stream, o, (const T*)u, ld_u, col,
                                               w, (T*)out, heads, vdim, eps, gate_silu));
  return check_launch("head_norm_gate");
}
