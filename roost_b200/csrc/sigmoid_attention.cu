// Grouped-query causal attention without a softmax: the weight of a visible key is the sigmoid of its score, and the weights
// are used as they are (nothing divides by their sum). In 32-bit arithmetic over a paged cache of either dtype.
//
//   prepare:   per token, on a row [q heads | k heads | v heads | ...] of the fused projection: every query and key head is
//              divided by sqrt(mean(x^2) + eps) and multiplied by a weight of dim numbers (one for the queries, one for the keys,
//              shared by the heads); queries are then multiplied by the temperature of the token's position p,
//              1 + coef * ln(floor((p + 1) / every) + 1) (coef 0: none), and written to a dense [tokens, heads, dim] tensor; keys
//              and values go to the token's cache slot (slot -1: nothing is written). The cache entry of (page, kv head, offset)
//              starts at ((page * kv_heads + head) * page_size + offset) * entry from k_base (keys) and v_base (values): two planes
//              of one size, or one plane whose entries are [key | value] (v_base = k_base + dim, entry = dim + vdim).
//   attention: one block per (token, key/value head, eight of its query heads, split); a warp a query head; key tiles of 32 at
//              absolute positions staged in shared memory as float32; a lane a key for the scores, a lane a value column for
//              the sums. A query at position p gives the key at position j the weight
//              sigmoid((q . k) * scale - slope[h] * (p - j) + bias[h]); the output is the weighted sum of the values, multiplied
//              element by element by sigmoid(gate) where a gate is given (columns of the same projection row). A token's tiles
//              may be dealt to several blocks in ranges; the partial sums are then added in split order by a second kernel. A
//              padding token (position -1) is skipped.
#include "common.cuh"

namespace roost {

constexpr int kSgTile = 32;
constexpr int kSgWarps = 8;
constexpr int kSgMaxDim = 512;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(128) sigmoid_prepare_kernel(const T* __restrict__ qkv, int64_t ld, T* __restrict__ q_out, T* k_base, T* v_base, int entry,
                                                             const float* __restrict__ q_w, const float* __restrict__ k_w,
                                                             const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                                                             int heads, int kv_heads, int dim, int vdim, float eps, float temp_coef, int temp_every,
                                                             int page_size) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int slot = slot_mapping[t];
  const float temp = temp_coef != 0.f && pos >= 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1)) : 1.0f;
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const T* row = qkv + (size_t)t * ld;
  const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  for (int h = warp; h < heads + kv_heads; h += nwarps) {           // a warp a query or key head
    const T* x = row + (size_t)h * dim;
    float a[kSgMaxDim / 32];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kSgMaxDim / 32; ++c) {
      const int j = c * 32 + lane;
      a[c] = j < dim ? to_float(x[j]) : 0.f;
      ss = fmaf(a[c], a[c], ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    const bool is_q = h < heads;
    if (!is_q && slot < 0) continue;          // a padding token: no key is written
    T* dst = is_q ? q_out + ((size_t)t * heads + h) * dim : k_base + ((page * kv_heads + (h - heads)) * page_size + off) * entry;
    const float* w = is_q ? q_w : k_w;
#pragma unroll
    for (int c = 0; c < kSgMaxDim / 32; ++c) {
      const int j = c * 32 + lane;
      if (j < dim) {
        const float y = a[c] * inv * w[j];
        dst[j] = from_float<T>(is_q ? y * temp : y);
      }
    }
  }
  if (slot < 0) return;
  const T* vsrc = row + (size_t)(heads + kv_heads) * dim;
  for (int idx = threadIdx.x; idx < kv_heads * vdim; idx += blockDim.x) {
    const int g = idx / vdim, i = idx % vdim;
    v_base[((page * kv_heads + g) * page_size + off) * entry + i] = vsrc[idx];
  }
}

template <typename T>
__global__ void __launch_bounds__(kSgWarps * 32) sigmoid_attention_kernel(const T* __restrict__ q, T* __restrict__ out, float* __restrict__ part,
                                                                        const T* __restrict__ k_base, const T* __restrict__ v_base, int entry,
                                                                        const T* __restrict__ gate, int64_t ld_gate,
                                                                        const float* __restrict__ slopes, const float* __restrict__ head_bias,
                                                                        const int32_t* __restrict__ positions, const int32_t* __restrict__ token_row,
                                                                        const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_indices,
                                                                        int heads, int kv_heads, int dim, int vdim, int page_size, float scale,
                                                                        int splits, int tiles_per_split) {
  extern __shared__ float sm[];
  float* ks = sm;                                          // [tile][dim + 1]
  float* vs = ks + (size_t)kSgTile * (dim + 1);            // [tile][vdim]
  float* qs = vs + (size_t)kSgTile * vdim;                 // [warps][dim]
  float* ps = qs + (size_t)kSgWarps * dim;                 // [warps][tile]
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int group = heads / kv_heads;
  const int blocks_a_group = (group + kSgWarps - 1) / kSgWarps;
  const int g = blockIdx.y / blocks_a_group, hb = blockIdx.y % blocks_a_group;
  const int z = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hg = hb * kSgWarps + warp;                     // the warp's head within the group
  const bool active = hg < group;
  const int h = g * group + hg;
  const int pos = positions[t];
  if (pos < 0) return;                                     // a padding token
  const int r = token_row[t];
  const int32_t* pages = kv_indices + kv_indptr[r];
  const float slope = active ? slopes[h] : 0.f, bias = active ? head_bias[h] : 0.f;
  pdl_wait();
  if (active) {
    const T* qr = q + ((size_t)t * heads + h) * dim;
    for (int i = lane; i < dim; i += 32) qs[(size_t)warp * dim + i] = to_float(qr[i]);
  }
  float acc[kSgMaxDim / 32];
#pragma unroll
  for (int c = 0; c < kSgMaxDim / 32; ++c) acc[c] = 0.f;
  const int n_tiles = pos / kSgTile + 1;
  // the last split takes whatever is left: a bound on the lengths that a row exceeds costs balance, not keys
  const int first = z * tiles_per_split, last = z == splits - 1 ? n_tiles : min(n_tiles, first + tiles_per_split);
  for (int tile = first; tile < last; ++tile) {
    const int k0 = tile * kSgTile;
    __syncthreads();
    for (int kk = warp; kk < kSgTile; kk += kSgWarps) {      // a warp a key: its entry's address once, the lanes over its numbers
      const int kp = k0 + kk;
      float* kd = ks + (size_t)kk * (dim + 1);
      float* vd = vs + (size_t)kk * vdim;
      if (kp <= pos) {
        const size_t at = (((size_t)pages[kp / page_size] * kv_heads + g) * page_size + kp % page_size) * entry;
        const T* kr = k_base + at;
        const T* vr = v_base + at;
        for (int i = lane; i < dim; i += 32) kd[i] = to_float(kr[i]);
        for (int i = lane; i < vdim; i += 32) vd[i] = to_float(vr[i]);
      } else {
        for (int i = lane; i < dim; i += 32) kd[i] = 0.f;
        for (int i = lane; i < vdim; i += 32) vd[i] = 0.f;
      }
    }
    __syncthreads();
    if (!active) continue;
    const float* qw = qs + (size_t)warp * dim;
    const float* kr = ks + (size_t)lane * (dim + 1);
    float s = 0.f;
    if ((dim & 3) == 0) {        // the query four numbers a (broadcast) read; the same products in the same order
      const float4* q4 = reinterpret_cast<const float4*>(qw);
      for (int i = 0; i < dim / 4; ++i) {
        const float4 qv = q4[i];
        s = fmaf(qv.x, kr[4 * i], s);
        s = fmaf(qv.y, kr[4 * i + 1], s);
        s = fmaf(qv.z, kr[4 * i + 2], s);
        s = fmaf(qv.w, kr[4 * i + 3], s);
      }
    } else {
      for (int i = 0; i < dim; ++i) s = fmaf(qw[i], kr[i], s);
    }
    const int kp = k0 + lane;
    s = s * scale - slope * (float)(pos - kp) + bias;
    ps[warp * kSgTile + lane] = kp <= pos ? sigmoid_f(s) : 0.f;
    __syncwarp();
#pragma unroll
    for (int c = 0; c < kSgMaxDim / 32; ++c) {
      const int i = c * 32 + lane;
      if (i < vdim) {
        float a = acc[c];
        const float4* p4 = reinterpret_cast<const float4*>(ps + warp * kSgTile);
#pragma unroll
        for (int kk = 0; kk < kSgTile / 4; ++kk) {
          const float4 pv = p4[kk];
          a = fmaf(pv.x, vs[(size_t)(4 * kk) * vdim + i], a);
          a = fmaf(pv.y, vs[(size_t)(4 * kk + 1) * vdim + i], a);
          a = fmaf(pv.z, vs[(size_t)(4 * kk + 2) * vdim + i], a);
          a = fmaf(pv.w, vs[(size_t)(4 * kk + 3) * vdim + i], a);
        }
        acc[c] = a;
      }
    }
    __syncwarp();
  }
  if (!active) return;
  if (part != nullptr) {
    float* dst = part + (((size_t)t * heads + h) * splits + z) * vdim;
#pragma unroll
    for (int c = 0; c < kSgMaxDim / 32; ++c) {
      const int i = c * 32 + lane;
      if (i < vdim) dst[i] = acc[c];
    }
    return;
  }
  T* o = out + ((size_t)t * heads + h) * vdim;
#pragma unroll
  for (int c = 0; c < kSgMaxDim / 32; ++c) {
    const int i = c * 32 + lane;
    if (i < vdim) {
      const float gv = gate != nullptr ? sigmoid_f(to_float(gate[(size_t)t * ld_gate + (size_t)h * vdim + i])) : 1.0f;
      o[i] = from_float<T>(acc[c] * gv);
    }
  }
}

// The partial sums of a token's head, added in split order, then the output gate.
template <typename T>
__global__ void sigmoid_merge_kernel(const float* __restrict__ part, T* __restrict__ out, const T* __restrict__ gate, int64_t ld_gate,
                                     const int32_t* __restrict__ positions, int heads, int vdim, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = positions[t];
  if (pos < 0) return;
  const float* src = part + ((size_t)t * heads + h) * splits * vdim;
  T* o = out + ((size_t)t * heads + h) * vdim;
  for (int i = threadIdx.x; i < vdim; i += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < splits; ++z) a += src[(size_t)z * vdim + i];
    const float gv = gate != nullptr ? sigmoid_f(to_float(gate[(size_t)t * ld_gate + (size_t)h * vdim + i])) : 1.0f;
    o[i] = from_float<T>(a * gv);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_sigmoid_attention_prepare(const void* qkv, int64_t ld, void* q_out, void* k_base, void* v_base, int entry, const float* q_w,
                                               const float* k_w, const int32_t* positions, const int32_t* slot_mapping, int tokens, int heads,
                                               int kv_heads, int dim, int vdim, float eps, float temp_coef, int temp_every, int page_size, int dtype,
                                               roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && page_size > 0, "sigmoid_attention_prepare: sizes must be positive");
  ROOST_REQUIRE(qkv && q_out && k_base && v_base && q_w && k_w && positions && slot_mapping, "sigmoid_attention_prepare: a pointer is null");
  ROOST_REQUIRE(eps > 0.f && (temp_coef == 0.f || temp_every > 0), "sigmoid_attention_prepare: eps and the temperature's period must be positive");
  ROOST_REQUIRE(ld >= (int64_t)(heads + kv_heads) * dim + (int64_t)kv_heads * vdim && entry >= dim && entry >= vdim,
                "sigmoid_attention_prepare: a row or a cache entry is too narrow");
  if (dim > kSgMaxDim) return fail(ROOST_ERR_UNSUPPORTED, "sigmoid_attention_prepare: heads beyond 512 numbers");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(sigmoid_prepare_kernel<T>, dim3(tokens), dim3(128), 0, (cudaStream_t)stream, (const T*)qkv, ld, (T*)q_out,
                                               (T*)k_base, (T*)v_base, entry, q_w, k_w, positions, slot_mapping, heads, kv_heads, dim, vdim, eps,
                                               temp_coef, temp_every, page_size));
  return check_launch("sigmoid_attention_prepare");
}

extern "C" int roost_sigmoid_attention(const void* q, void* out, float* part, const void* k_base, const void* v_base, int entry, const void* gate,
                                       int64_t ld_gate, const float* slopes, const float* head_bias, const int32_t* positions,
                                       const int32_t* token_row, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens, int heads,
                                       int kv_heads, int dim, int vdim, int page_size, float scale, int splits, int tiles_per_split, int dtype,
                                       roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && page_size > 0, "sigmoid_attention: sizes must be positive");
  ROOST_REQUIRE(heads % kv_heads == 0, "sigmoid_attention: the query heads are no multiple of the key/value heads");
  ROOST_REQUIRE(q && out && k_base && v_base && slopes && head_bias && positions && token_row && kv_indptr && kv_indices,
                "sigmoid_attention: a pointer is null");
  ROOST_REQUIRE(gate == nullptr || ld_gate >= (int64_t)heads * vdim, "sigmoid_attention: a gate's row is too narrow");
  ROOST_REQUIRE(splits >= 1 && tiles_per_split >= 1 && (splits == 1 || part != nullptr), "sigmoid_attention: splits need a workspace for their partials");
  if (dim > kSgMaxDim || vdim > kSgMaxDim) return fail(ROOST_ERR_UNSUPPORTED, "sigmoid_attention: heads or values beyond 512 numbers");
  const int group = heads / kv_heads;
  const int gy = kv_heads * ((group + kSgWarps - 1) / kSgWarps);
  if (splits > 65535 || gy > 65535) return fail(ROOST_ERR_UNSUPPORTED, "sigmoid_attention: too many heads or splits");
  if (tokens == 0) return ROOST_OK;
  const size_t smem = ((size_t)kSgTile * (dim + 1 + vdim) + (size_t)kSgWarps * (dim + kSgTile)) * sizeof(float);
  dim3 grid(tokens, gy, splits);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = sigmoid_attention_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, dim3(kSgWarps * 32), smem, (cudaStream_t)stream, (const T*)q, (T*)out, splits > 1 ? part : (float*)nullptr,
                  (const T*)k_base, (const T*)v_base, entry, (const T*)gate, ld_gate, slopes, head_bias, positions, token_row, kv_indptr,
                  kv_indices, heads, kv_heads, dim, vdim, page_size, scale, splits, tiles_per_split);
    if (splits > 1)
      launch_kernel(sigmoid_merge_kernel<T>, dim3(tokens, heads), dim3(128), 0, (cudaStream_t)stream, (const float*)part, (T*)out, (const T*)gate,
                    ld_gate, positions, heads, vdim, splits);
  });
  return check_launch("sigmoid_attention");
}

// ---------------------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16, mma.sync m16n8k16), for steps that bring prompt portions.
//
// One block of four warps per (row of the step, 64 of its query tokens, query head); a warp 16 query tokens. Key tiles of 64 keys
// and their values are staged in shared memory as bfloat16 by asynchronous copies, one tile ahead; S = Q K^T in 32-bit accumulators; every score becomes its weight
// sigmoid(s scale - slope (i - j) + bias) in 32-bit, a key after the query's position none; the weights enter P V as two bfloat16
// operands, their rounding and what it left over (16 bits of the 32-bit weights), summed in 32-bit accumulators over all key tiles;
// the output gate and the one rounding come last. A tile of queries far into a long row has its keys dealt to several blocks in
// chunks of tiles_a_chunk key tiles (the sums are plain sums: a second kernel adds the chunks' in order), so that the blocks of a
// row's last tiles do not run many times as long as those of its first. Sizes: dim and vdim multiples of 16 up to 128.
namespace roost {

constexpr int kSmTile = 64;       // query tokens a block, keys a tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x, y) as two bfloat16 in one register, and what the rounding left over likewise
__device__ __forceinline__ void split_pair(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x - __bfloat162float(h.x), y - __bfloat162float(h.y));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

// Which (row, tile of 64 tokens) the block `b` takes: rows in order, each with ceil(tokens / 64) tiles. False beyond the step's.
__device__ __forceinline__ bool sigmoid_tile_of_block(const int32_t* __restrict__ q_indptr, int rows, int b, int& r, int& k) {
  for (r = 0; r < rows; ++r) {
    const int tiles = (q_indptr[r + 1] - q_indptr[r] + kSmTile - 1) / kSmTile;
    if (b < tiles) {
      k = b;
      return true;
    }
    b -= tiles;
  }
  return false;
}

template <int DMAX, int VMAX>
__global__ void __launch_bounds__(128) sigmoid_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                                                                   const __nv_bfloat16* __restrict__ k_base, const __nv_bfloat16* __restrict__ v_base,
                                                                   int entry, const __nv_bfloat16* __restrict__ gate, int64_t ld_gate,
                                                                   const float* __restrict__ slopes, const float* __restrict__ head_bias,
                                                                   const int32_t* __restrict__ positions, const int32_t* __restrict__ q_indptr,
                                                                   const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_indices,
                                                                   int rows, int heads, int kv_heads, int dim, int vdim, int page_size, float scale,
                                                                   float* __restrict__ ws, int tiles_a_chunk, int max_chunks) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  const int ldq = dim + 8, ldv = vdim + 8;                    // padded rows: 16-byte aligned, ldmatrix without bank conflicts
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sm_raw);      // [64][dim + 8]
  __nv_bfloat16* Kb = Qs + kSmTile * ldq;                            // two buffers of [64][dim + 8]
  __nv_bfloat16* Vb = Kb + 2 * kSmTile * ldq;                        // two buffers of [64][vdim + 8]
  pdl_launch_dependents();
  int r, tile;
  // the blocks with the most keys ahead of them (a row's last tiles) start first
  if (!sigmoid_tile_of_block(q_indptr, rows, (int)gridDim.x - 1 - (int)blockIdx.x, r, tile)) return;
  const int h = blockIdx.y, g = h / (heads / kv_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = q_indptr[r] + tile * kSmTile;
  const int n_valid = min(kSmTile, q_indptr[r + 1] - t0);
  const int p0 = positions[t0];
  if (p0 < 0) return;                                          // a padding row
  const int p_last = p0 + n_valid - 1;
  if ((int)blockIdx.z * tiles_a_chunk > p_last / kSmTile) return;      // the tile's keys end before this block's chunk
  const int32_t* pages = kv_indices + kv_indptr[r];
  const float slope = slopes[h], bias = head_bias[h];
  pdl_wait();
  // the block's queries
  const int qchunks = dim / 8;
  for (int idx = tid; idx < kSmTile * qchunks; idx += 128) {
    const int row = idx / qchunks, c = (idx % qchunks) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n_valid) v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + row) * heads + h) * dim + c);
    *reinterpret_cast<uint4*>(Qs + row * ldq + c) = v;
  }
  __syncthreads();
  uint32_t qa[DMAX / 16][4];
#pragma unroll
  for (int ks = 0; ks < DMAX / 16; ++ks)
    if (ks * 16 < dim) ldmatrix_x4(qa[ks], Qs + (warp * 16 + (lane & 15)) * ldq + ks * 16 + (lane >> 4) * 8);
  float o[VMAX / 8][4];
#pragma unroll
  for (int n = 0; n < VMAX / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  const int row_lo = warp * 16 + (lane >> 2);                 // the thread's two query rows within the tile: row_lo and row_lo + 8
  const int pos_lo = p0 + row_lo, pos_hi = pos_lo + 8;
  const int vchunks = vdim / 8;
  // the tile's keys in chunks of tiles_a_chunk key tiles, a chunk a block (blockIdx.z); with more than one chunk the blocks leave
  // their sums in ws and a second kernel adds them in order
  const int all_tiles = p_last / kSmTile + 1;
  const int n_chunks = min((all_tiles + tiles_a_chunk - 1) / tiles_a_chunk, max_chunks);
  const int first_tile = (int)blockIdx.z * tiles_a_chunk;
  if (first_tile >= all_tiles) return;
  // the launch's last chunk takes whatever is left: a bound on the lengths that a row exceeds costs balance, not keys
  const int n_tiles = (int)blockIdx.z == max_chunks - 1 ? all_tiles : min(all_tiles, first_tile + tiles_a_chunk);
  // a tile's keys and values come by asynchronous 16-byte copies (a key after the block's last query: zeros), one tile ahead
  auto fetch = [&](int kt) {
    const int k0 = kt * kSmTile;
    __nv_bfloat16* Kd = Kb + ((kt - first_tile) & 1) * kSmTile * ldq;
    __nv_bfloat16* Vd = Vb + ((kt - first_tile) & 1) * kSmTile * ldv;
    for (int idx = tid; idx < kSmTile * (qchunks + vchunks); idx += 128) {
      const bool is_k = idx < kSmTile * qchunks;
      const int i2 = is_k ? idx : idx - kSmTile * qchunks;
      const int per = is_k ? qchunks : vchunks;
      const int key = i2 / per, c = (i2 % per) * 8;
      const int kp = min(k0 + key, p_last);
      const size_t at = (((size_t)pages[kp / page_size] * kv_heads + g) * page_size + kp % page_size) * entry + c;
      const __nv_bfloat16* src = (is_k ? k_base : v_base) + at;
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(is_k ? Kd + key * ldq + c : Vd + key * ldv + c);
      const int bytes = k0 + key <= p_last ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  fetch(first_tile);
  for (int kt = first_tile; kt < n_tiles; ++kt) {
    const int k0 = kt * kSmTile;
    const __nv_bfloat16* Ks = Kb + ((kt - first_tile) & 1) * kSmTile * ldq;
    const __nv_bfloat16* Vs = Vb + ((kt - first_tile) & 1) * kSmTile * ldv;
    if (kt + 1 < n_tiles) {
      fetch(kt + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    if (k0 <= p0 + warp * 16 + 15) {                            // else every key of the tile lies after the warp's last query
    // S = Q K^T: 16 queries x 64 keys a warp
    float s[kSmTile / 8][4];
#pragma unroll
    for (int n = 0; n < kSmTile / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < DMAX / 16; ++ks) {
      if (ks * 16 < dim) {
#pragma unroll
        for (int np = 0; np < kSmTile / 16; ++np) {
          uint32_t b[4];
          ldmatrix_x4(b, Ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * ldq + ks * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * np], qa[ks], b[0], b[1]);
          mma_bf16(s[2 * np + 1], qa[ks], b[2], b[3]);
        }
      }
    }
    // the weights, then P V with P as two operands
    const bool diagonal = k0 + kSmTile - 1 > p0 + warp * 16;
#pragma unroll
    for (int kk = 0; kk < kSmTile / 16; ++kk) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int n = 2 * kk + half;
        const int j = k0 + n * 8 + (lane & 3) * 2;
        // bias - slope (i - j) for the thread's two rows at key j; the key after it adds one slope
        const float b_lo = fmaf(slope, (float)(j - pos_lo), bias), b_hi = fmaf(slope, (float)(j - pos_hi), bias);
        float w[4];
        w[0] = __fdividef(1.0f, 1.0f + __expf(-fmaf(s[n][0], scale, b_lo)));
        w[1] = __fdividef(1.0f, 1.0f + __expf(-fmaf(s[n][1], scale, b_lo + slope)));
        w[2] = __fdividef(1.0f, 1.0f + __expf(-fmaf(s[n][2], scale, b_hi)));
        w[3] = __fdividef(1.0f, 1.0f + __expf(-fmaf(s[n][3], scale, b_hi + slope)));
        if (diagonal) {                                          // only the tiles around the warp's own positions hold keys to hide
          if (j > pos_lo) w[0] = 0.f;
          if (j + 1 > pos_lo) w[1] = 0.f;
          if (j > pos_hi) w[2] = 0.f;
          if (j + 1 > pos_hi) w[3] = 0.f;
        }
        split_pair(w[0], w[1], hi[2 * half], lo[2 * half]);
        split_pair(w[2], w[3], hi[2 * half + 1], lo[2 * half + 1]);
      }
      // A fragment order: (rows g, keys 0-7), (rows g + 8, keys 0-7), (rows g, keys 8-15), (rows g + 8, keys 8-15)
      const uint32_t ah[4] = {hi[0], hi[1], hi[2], hi[3]}, al[4] = {lo[0], lo[1], lo[2], lo[3]};
#pragma unroll
      for (int np = 0; np < VMAX / 16; ++np) {
        if (np * 16 < vdim) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + np * 16 + (lane >> 4) * 8);
          mma_bf16(o[2 * np], ah, b[0], b[1]);
          mma_bf16(o[2 * np], al, b[0], b[1]);
          mma_bf16(o[2 * np + 1], ah, b[2], b[3]);
          mma_bf16(o[2 * np + 1], al, b[2], b[3]);
        }
      }
    }
    }
    __syncthreads();                                           // everybody is done with the buffer the next fetch fills
  }
  if (n_chunks > 1) {                                          // the chunk's sums, for the kernel that adds a tile's chunks
#pragma unroll
    for (int n = 0; n < VMAX / 8; ++n) {
      if (n * 8 < vdim) {
        const int c = n * 8 + (lane & 3) * 2;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int row = row_lo + half * 8;
          if (row < n_valid)
            *reinterpret_cast<float2*>(ws + ((((size_t)(t0 + row) * heads + h) * max_chunks + blockIdx.z) * vdim + c)) =
                make_float2(o[n][2 * half], o[n][2 * half + 1]);
        }
      }
    }
    return;
  }
  // the output gate and the one rounding
#pragma unroll
  for (int n = 0; n < VMAX / 8; ++n) {
    if (n * 8 < vdim) {
      const int c = n * 8 + (lane & 3) * 2;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = row_lo + half * 8;
        if (row < n_valid) {
          const size_t t = (size_t)(t0 + row);
          float x = o[n][2 * half], y = o[n][2 * half + 1];
          if (gate != nullptr) {
            const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(gate + t * ld_gate + (size_t)h * vdim + c);
            x *= 1.0f / (1.0f + __expf(-__bfloat162float(gv.x)));
            y *= 1.0f / (1.0f + __expf(-__bfloat162float(gv.y)));
          }
          *reinterpret_cast<__nv_bfloat162*>(out + (t * heads + h) * vdim + c) = __floats2bfloat162_rn(x, y);
        }
      }
    }
  }
}

// A block a token: where the token's tile of queries had its keys in several chunks, their sums are added in chunk order, then the
// output gate and the one rounding.
__global__ void sigmoid_mma_merge_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate,
                                         int64_t ld_gate, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_row,
                                         const int32_t* __restrict__ q_indptr, int heads, int vdim, int tiles_a_chunk, int max_chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  if (positions[t] < 0) return;
  const int r = token_row[t];
  const int t0 = q_indptr[r] + (t - q_indptr[r]) / kSmTile * kSmTile;
  const int n_valid = min(kSmTile, q_indptr[r + 1] - t0);
  const int all_tiles = (positions[t0] + n_valid - 1) / kSmTile + 1;
  const int n_chunks = min((all_tiles + tiles_a_chunk - 1) / tiles_a_chunk, max_chunks);
  if (n_chunks <= 1) return;                                   // the attention kernel wrote the token's output itself
  const int width = heads * vdim;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int h = i / vdim, c = i % vdim;
    const float* src = ws + (((size_t)t * heads + h) * max_chunks) * vdim + c;
    float a = 0.f;
    for (int z = 0; z < n_chunks; ++z) a += src[(size_t)z * vdim];
    if (gate != nullptr) a *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[(size_t)t * ld_gate + i])));
    out[(size_t)t * width + i] = __float2bfloat16_rn(a);
  }
}

}  // namespace roost

extern "C" int roost_sigmoid_attention_mma_supported(int dim, int vdim, int entry) {
  return dim % 16 == 0 && vdim % 16 == 0 && dim <= 128 && vdim <= 128 && entry % 8 == 0;
}

// q [tokens, heads, dim], out [tokens, heads * vdim], both bfloat16; rows: the step's rows (q_indptr has rows + 1 entries).
extern "C" int roost_sigmoid_attention_mma(const void* q, void* out, const void* k_base, const void* v_base, int entry, const void* gate, int64_t ld_gate,
                                           const float* slopes, const float* head_bias, const int32_t* positions, const int32_t* q_indptr,
                                           const int32_t* token_row, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens, int rows, int heads,
                                           int kv_heads, int dim, int vdim, int page_size, float scale, float* ws, int tiles_a_chunk, int max_chunks,
                                           roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && rows >= 0 && heads > 0 && kv_heads > 0 && page_size > 0 && heads % kv_heads == 0, "sigmoid_attention_mma: sizes must be positive");
  ROOST_REQUIRE(q && out && k_base && v_base && slopes && head_bias && positions && q_indptr && kv_indptr && kv_indices,
                "sigmoid_attention_mma: a pointer is null");
  if (!roost_sigmoid_attention_mma_supported(dim, vdim, entry)) return fail(ROOST_ERR_UNSUPPORTED, "sigmoid_attention_mma: sizes no tensor-core form serves");
  ROOST_REQUIRE((uintptr_t)q % 16 == 0 && (uintptr_t)k_base % 16 == 0 && (uintptr_t)v_base % 16 == 0 && (uintptr_t)out % 4 == 0 &&
                    (gate == nullptr || ((uintptr_t)gate % 4 == 0 && ld_gate % 2 == 0 && ld_gate >= (int64_t)heads * vdim)),
                "sigmoid_attention_mma: a pointer is not aligned");
  ROOST_REQUIRE(tiles_a_chunk >= 1 && max_chunks >= 1 && (max_chunks == 1 || (ws != nullptr && token_row != nullptr)),
                "sigmoid_attention_mma: chunks of keys need a workspace for their sums");
  if (tokens == 0 || rows == 0) return ROOST_OK;
  if (heads > 65535 || max_chunks > 65535) return fail(ROOST_ERR_UNSUPPORTED, "sigmoid_attention_mma: too many heads or chunks");
  const size_t smem = ((size_t)3 * kSmTile * (dim + 8) + (size_t)2 * kSmTile * (vdim + 8)) * sizeof(__nv_bfloat16);
  dim3 grid((tokens + kSmTile - 1) / kSmTile + rows, heads, max_chunks);
#define ROOST_SG_MMA(DMAX, VMAX)                                                                                                                  \
  do {                                                                                                                                            \
    auto kernel = sigmoid_attention_mma_kernel<DMAX, VMAX>;                                                                                       \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                   \
    launch_kernel(kernel, grid, dim3(128), smem, (cudaStream_t)stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_base, \
                  (const __nv_bfloat16*)v_base, entry, (const __nv_bfloat16*)gate, ld_gate, slopes, head_bias, positions, q_indptr, kv_indptr,    \
                  kv_indices, rows, heads, kv_heads, dim, vdim, page_size, scale, ws, tiles_a_chunk, max_chunks);                                 \
  } while (0)
  if (dim <= 64 && vdim <= 64) ROOST_SG_MMA(64, 64);
  else if (dim <= 64) ROOST_SG_MMA(64, 128);
  else if (vdim <= 64) ROOST_SG_MMA(128, 64);
  else ROOST_SG_MMA(128, 128);
#undef ROOST_SG_MMA
  if (max_chunks > 1)
    launch_kernel(sigmoid_mma_merge_kernel, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, (const float*)ws, (__nv_bfloat16*)out,
                  (const __nv_bfloat16*)gate, ld_gate, positions, token_row, q_indptr, heads, vdim, tiles_a_chunk, max_chunks);
  return check_launch("sigmoid_attention_mma");
}
