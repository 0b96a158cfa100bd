// Retention: a matrix state a head that fades by a constant factor a token and is read by the query as it is, in 32-bit arithmetic.
//
// Per (row, head), for the row's tokens in order, with q, k (dim numbers) and v (vdim numbers):
//   S <- decay_h S + k v^T,   o = S^T q.
// The slot holds, head after head, S: dim x vdim.
//
// prepare: per token, every query and key head of the row [q heads | k heads | ...] of the input projection has its first
// rot_dims elements turned in pairs (i, i + rot_dims / 2): (u, v) -> (u cos a - v sin a, v cos a + u sin a) with
// a = position * inv_freq[i] formed in double and reduced to [-pi, pi]; the keys are then multiplied by k_scale. Both go to a
// float32 tensor [tokens, 2 * heads * dim] of their own: what enters the recurrence is not rounded to the activation dtype.
//
// scan: one warp (a block) per (row, head, 32 columns of S). A lane keeps its column of S in registers (dim up to 128) or in
// shared memory (beyond); a token's (k, q) are staged in shared memory once and read by all lanes; the next token's inputs are
// loaded while the current one is multiplied.
//
// Steps of many tokens cut every row into chunks of 64 tokens that run side by side (three launches): a chunk of n tokens walked
// from S = 0 ends with S'; a state S before the chunk is decay^n S + S' after it. The first walk leaves every chunk's own S', one
// thread an entry then carries the row's state from chunk to chunk leaving every chunk's true starting state in its place, and a
// second walk of every chunk from there writes the outputs and, from a row's last chunk, the slot.
#include "common.cuh"

namespace roost {

constexpr int kRtChunkTokens = 64;

template <typename T>
__global__ void __launch_bounds__(128) retention_prepare_kernel(const T* __restrict__ u, int64_t ld, float* __restrict__ qk,
                                                               const double* __restrict__ inv_freq, const int32_t* __restrict__ positions,
                                                               int heads, int dim, int rot_dims, float k_scale) {
  extern __shared__ float sm[];      // rot_dims/2 cosines, rot_dims/2 sines
  const int half = rot_dims / 2;
  float* cs = sm;
  float* sn = sm + half;
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double ang = (double)pos * inv_freq[i];
    ang -= 6.283185307179586476925286766559 * rint(ang * 0.15915494309189533576888376337251);
    sincosf((float)ang, &sn[i], &cs[i]);
  }
  pdl_wait();
  __syncthreads();
  const T* row = u + (size_t)t * ld;
  float* dst = qk + (size_t)t * 2 * heads * dim;
  const int n = 2 * heads * dim;
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int j = idx % dim;
    const float x = to_float(row[idx]);
    float y = x;
    if (j < half) {
      y = x * cs[j] - to_float(row[idx + half]) * sn[j];
    } else if (j < rot_dims) {
      y = x * cs[j - half] + to_float(row[idx - half]) * sn[j - half];
    }
    dst[idx] = idx >= heads * dim ? y * k_scale : y;
  }
}

// Which (row, chunk) the block `b` of a chunked launch takes: rows in order, each with ceil(tokens / 64) chunks.
__device__ __forceinline__ bool retention_chunk_of_block(const int32_t* __restrict__ q_indptr, int rows, int b, int& r, int& k, int& chunks_of_row) {
  for (r = 0; r < rows; ++r) {
    const int n = q_indptr[r + 1] - q_indptr[r];
    chunks_of_row = (n + kRtChunkTokens - 1) / kRtChunkTokens;
    if (b < chunks_of_row) {
      k = b;
      return true;
    }
    b -= chunks_of_row;
  }
  return false;
}

// DREG > 0: S in registers, dim <= DREG. DREG == 0: S in shared memory after the staging area, [dim][32].
// MODE 0: a warp walks its row's tokens from the slot and writes the slot back. MODE 1: a warp walks one chunk from S = 0 and
// leaves S' in ws[chunk]; a row's last chunk is skipped. MODE 2: a warp walks one chunk from ws[chunk] (the carry kernel put the
// chunk's true starting state there) and writes the outputs; a row's last chunk writes the slot.
template <typename T, int DREG, int MODE>
__global__ void __launch_bounds__(32) retention_scan_kernel(const float* __restrict__ qk, const T* __restrict__ v, int64_t ldv,
                                                           float* __restrict__ out, float* state, int64_t state_stride,
                                                           const float* __restrict__ decay, const int32_t* __restrict__ q_indptr,
                                                           const int32_t* __restrict__ slots, int rows, int heads, int dim, int vdim, float* ws) {
  extern __shared__ float sm[];      // two staging slots of dim (k, q) pairs; then S when it does not live in registers
  constexpr int NREG = DREG > 0 ? DREG : 1;
  constexpr int NN = DREG > 0 ? DREG / 32 : 32;          // entries of q and k a lane loads (dim <= 1024 in shared-memory form)
  pdl_launch_dependents();
  int r = blockIdx.x, k = 0, chunks_of_row = 1;
  const int h = blockIdx.y, slice = blockIdx.z;
  const int lane = threadIdx.x;
  const int col = slice * 32 + lane;
  const bool live = col < vdim;
  if (MODE != 0 && !retention_chunk_of_block(q_indptr, rows, blockIdx.x, r, k, chunks_of_row)) return;
  if (MODE == 1 && k == chunks_of_row - 1) return;       // nobody starts from the state a row's last chunk ends with
  int start = q_indptr[r], end = q_indptr[r + 1];
  if (MODE != 0) {
    start += k * kRtChunkTokens;
    end = min(end, start + kRtChunkTokens);
  }
  const size_t head_state = (size_t)dim * vdim;
  float* slot = state + (size_t)slots[r] * state_stride + (size_t)h * head_state;
  float* wsh = MODE != 0 ? ws + ((size_t)blockIdx.x * heads + h) * head_state : nullptr;
  const float* hs = MODE == 0 ? slot : wsh;               // where the walk starts from (MODE 1 starts empty)
  float* S_sm = sm + 4 * dim + lane;                       // [dim][32], used when DREG == 0
  const float keep = decay[h];
  const int QK = heads * dim;
  pdl_wait();
  if (end <= start) return;
  float S[NREG];
  if (DREG > 0) {
#pragma unroll
    for (int d = 0; d < NREG; ++d) S[d] = (MODE != 1 && live && d < dim) ? hs[(size_t)d * vdim + col] : 0.f;
  } else {
    for (int d = 0; d < dim; ++d) S_sm[(size_t)d * 32] = (MODE != 1 && live) ? hs[(size_t)d * vdim + col] : 0.f;
  }
  // the next token's inputs, loaded one token ahead
  float nk[NN], nq[NN], nv;
  auto load = [&](int t) {
    const float* row = qk + (size_t)t * 2 * QK;
#pragma unroll
    for (int i = 0; i < NN; ++i) {
      const int d = lane + 32 * i;
      nq[i] = d < dim ? row[(size_t)h * dim + d] : 0.f;
      nk[i] = d < dim ? row[QK + (size_t)h * dim + d] : 0.f;
    }
    nv = live ? to_float(v[(size_t)t * ldv + (size_t)h * vdim + col]) : 0.f;
  };
  load(start);
  for (int t = start; t < end; ++t) {
    float2* stage = reinterpret_cast<float2*>(sm) + (size_t)(t & 1) * dim;
#pragma unroll
    for (int i = 0; i < NN; ++i) {
      const int d = lane + 32 * i;
      if (d < dim) stage[d] = make_float2(nk[i], nq[i]);
    }
    const float val = nv;
    if (t + 1 < end) load(t + 1);
    __syncwarp();
    float num = 0.f;
    if (DREG > 0) {
#pragma unroll
      for (int d = 0; d < NREG; ++d) {
        if (d < dim) {
          const float2 kq = stage[d];
          S[d] = fmaf(keep, S[d], kq.x * val);
          num = fmaf(S[d], kq.y, num);
        }
      }
    } else {
      for (int d = 0; d < dim; ++d) {
        const float2 kq = stage[d];
        const float s = fmaf(keep, S_sm[(size_t)d * 32], kq.x * val);
        S_sm[(size_t)d * 32] = s;
        num = fmaf(s, kq.y, num);
      }
    }
    if (MODE != 1 && live) out[(size_t)t * heads * vdim + (size_t)h * vdim + col] = num;
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
}

// One thread an entry of S of a (row, head): the row's state through its chunks in order. ws[chunk] holds the chunk's own S' on
// entry (all but a row's last chunk) and the state the chunk starts from on exit. Every chunk but a row's last has 64 tokens, so
// the state before the next chunk is decay^64 times the state before this one, plus S'. The slot is read, not written.
__global__ void retention_carry_kernel(const float* state, int64_t state_stride, float* ws, const float* __restrict__ decay,
                                       const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, int heads, int dim, int vdim) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int idx = blockIdx.z * blockDim.x + threadIdx.x;
  const int entries = dim * vdim;
  if (idx >= entries) return;
  int first = 0;
  for (int rr = 0; rr < r; ++rr) first += (q_indptr[rr + 1] - q_indptr[rr] + kRtChunkTokens - 1) / kRtChunkTokens;
  const int chunks = (q_indptr[r + 1] - q_indptr[r] + kRtChunkTokens - 1) / kRtChunkTokens;
  if (chunks == 0) return;
  float e = state[(size_t)slots[r] * state_stride + (size_t)h * entries + idx];
  float through = decay[h];                               // decay^64 by squaring: kRtChunkTokens is 2^6
#pragma unroll
  for (int i = 0; i < 6; ++i) through *= through;
  const size_t stride = (size_t)heads * entries;
  float* w0 = ws + ((size_t)first * heads + h) * entries;
  constexpr int kBatch = 8;       // the chunks' own entries do not depend on e: a batch of loads in flight, then the chain
  for (int k0 = 0; k0 < chunks; k0 += kBatch) {
    float own[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) own[j] = k0 + j < chunks - 1 ? w0[(size_t)(k0 + j) * stride + idx] : 0.f;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (k0 + j < chunks) {
        w0[(size_t)(k0 + j) * stride + idx] = e;            // what chunk k0 + j starts from
        if (k0 + j < chunks - 1) e = fmaf(through, e, own[j]);
      }
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_retention_prepare(const void* u, int64_t ld, float* qk, const double* inv_freq, const int32_t* positions, int tokens, int heads,
                                       int dim, int rot_dims, float k_scale, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && dim > 0, "retention_prepare: sizes must be positive");
  ROOST_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim, "retention_prepare: the rotated width must be even and at most dim");
  ROOST_REQUIRE(u && qk && positions && (rot_dims == 0 || inv_freq), "retention_prepare: a pointer is null");
  ROOST_REQUIRE(ld >= (int64_t)2 * heads * dim, "retention_prepare: a row is too narrow");
  if (tokens == 0) return ROOST_OK;
  const size_t smem = ((size_t)rot_dims + 2) * sizeof(float);
  if (smem > 48 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "retention_prepare: a rotation of more than 12286 elements");
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(retention_prepare_kernel<T>, dim3(tokens), dim3(128), smem, (cudaStream_t)stream, (const T*)u, ld, qk,
                                               inv_freq, positions, heads, dim, rot_dims, k_scale));
  return check_launch("retention_prepare");
}

extern "C" int roost_retention_scan_chunks(int tokens, int rows) { return (tokens + kRtChunkTokens - 1) / kRtChunkTokens + rows; }

// ws (float[chunks * heads * dim * vdim], chunks = roost_retention_scan_chunks(tokens, rows)): rows are cut into chunks that run side
// by side (three launches); null: every row is walked in one pass.
extern "C" int roost_retention_scan(const float* qk, const void* v, int64_t ldv, float* out, float* state, int64_t state_stride, const float* decay,
                                    const int32_t* q_indptr, const int32_t* slots, int rows, int tokens, int heads, int dim, int vdim, float* ws,
                                    int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && tokens >= 0 && heads > 0 && dim > 0 && vdim > 0, "retention_scan: sizes must be positive");
  ROOST_REQUIRE(qk && v && out && state && decay && q_indptr && slots, "retention_scan: a pointer is null");
  ROOST_REQUIRE(ldv >= (int64_t)heads * vdim && state_stride >= (int64_t)heads * dim * vdim, "retention_scan: a row or a slot is too narrow");
  if (dim > 1024) return fail(ROOST_ERR_UNSUPPORTED, "retention_scan: heads of more than 1024 keys");
  const int slices = (vdim + 31) / 32;
  if (heads > 65535 || slices > 65535) return fail(ROOST_ERR_UNSUPPORTED, "retention_scan: too many heads or values");
  if (rows == 0 || tokens == 0) return ROOST_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t stage = (size_t)4 * dim * sizeof(float);
  const int chunks = roost_retention_scan_chunks(tokens, rows);
#define ROOST_RT_LAUNCH(DREG, MODE, SMEM, GX)                                                                                                     \
  do {                                                                                                                                            \
    auto kernel = retention_scan_kernel<T, DREG, MODE>;                                                                                           \
    if ((SMEM) > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM));                               \
    launch_kernel(kernel, dim3((GX), heads, slices), dim3(32), (SMEM), s, qk, (const T*)v, ldv, out, state, state_stride, decay, q_indptr, slots, \
                  rows, heads, dim, vdim, ws);                                                                                                    \
  } while (0)
#define ROOST_RT_SCAN(DREG, SMEM)                                                                                                                 \
  do {                                                                                                                                            \
    if (ws == nullptr) {                                                                                                                          \
      ROOST_RT_LAUNCH(DREG, 0, SMEM, rows);                                                                                                       \
    } else {                                                                                                                                      \
      ROOST_RT_LAUNCH(DREG, 1, SMEM, chunks);                                                                                                     \
      launch_kernel(retention_carry_kernel, dim3(rows, heads, (dim * vdim + 255) / 256), dim3(256), 0, s, (const float*)state, state_stride, ws,  \
                    decay, q_indptr, slots, heads, dim, vdim);                                                                                    \
      ROOST_RT_LAUNCH(DREG, 2, SMEM, chunks);                                                                                                     \
    }                                                                                                                                             \
  } while (0)
  ROOST_DISPATCH_DTYPE(dtype, T, {
    if (dim <= 32) ROOST_RT_SCAN(32, stage);
    else if (dim <= 64) ROOST_RT_SCAN(64, stage);
    else if (dim <= 128) ROOST_RT_SCAN(128, stage);
    else ROOST_RT_SCAN(0, stage + (size_t)dim * 32 * sizeof(float));
  });
#undef ROOST_RT_SCAN
#undef ROOST_RT_LAUNCH
  return check_launch("retention_scan");
}
