// Causal softmax attention of prompt portions over keys and values that were carried out of a latent cache for the step: the
// step's rows each own a stretch of `stride` entries of two dense tensors, keys [rows * stride, heads * dim] and values
// [rows * stride, heads * vdim] (made by two products from the rows' gathered latents), entry j of a row being its token at
// position j. bfloat16 on the tensor cores (mma.sync m16n8k16); scores, running maxima, weights and sums in 32-bit.
//
//   latent_gather:  a block an entry: the cached vector of (row, position j) copied to the dense [rows * stride, width] tensor,
//                   zeros beyond the row's length.
//   attention:      one block of four warps per (row, 64 of its query tokens, head), a warp 16 query tokens; key tiles of 64 and
//                   their values come by asynchronous copies a tile ahead; S = Q K^T; a running maximum and denominator a query;
//                   the weights exp(s - m) enter P V as two bfloat16 operands, their rounding and what it left over (16 bits of
//                   the 32-bit weights); the blocks of a row's last tiles start first. Sizes: dim and vdim multiples of 16 up to 128.
#include "common.cuh"

namespace roost {

constexpr int kCaTile = 64;

__device__ __forceinline__ void ca_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ca_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ca_mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ca_split_pair(float x, float y, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  const __nv_bfloat162 l = __floats2bfloat162_rn(x - __bfloat162float(h.x), y - __bfloat162float(h.y));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

__global__ void latent_gather_kernel(const __nv_bfloat16* __restrict__ pool, __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ kv_lens,
                                     const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_indices, int stride, int width,
                                     int page_size) {
  pdl_launch_dependents();
  const int r = blockIdx.y, j = blockIdx.x;
  pdl_wait();
  __nv_bfloat16* dst = out + ((size_t)r * stride + j) * width;
  const __nv_bfloat16* src = nullptr;
  if (j < kv_lens[r]) src = pool + ((size_t)kv_indices[kv_indptr[r] + j / page_size] * page_size + j % page_size) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src != nullptr ? src[i] : __float2bfloat16_rn(0.f);
}

__device__ __forceinline__ bool ca_tile_of_block(const int32_t* __restrict__ q_indptr, int rows, int b, int& r, int& k) {
  for (r = 0; r < rows; ++r) {
    const int tiles = (q_indptr[r + 1] - q_indptr[r] + kCaTile - 1) / kCaTile;
    if (b < tiles) {
      k = b;
      return true;
    }
    b -= tiles;
  }
  return false;
}

template <int DMAX, int VMAX>
__global__ void __launch_bounds__(128) carried_attention_kernel(const __nv_bfloat16* __restrict__ q, int64_t ld_q, __nv_bfloat16* __restrict__ out,
                                                               const __nv_bfloat16* __restrict__ keys, const __nv_bfloat16* __restrict__ values,
                                                               const int32_t* __restrict__ positions, const int32_t* __restrict__ q_indptr,
                                                               int rows, int heads, int dim, int vdim, int stride, float scale_log2e) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  const int ldq = dim + 8, ldv = vdim + 8;                    // padded rows: 16-byte aligned, ldmatrix without bank conflicts
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sm_raw);      // [64][dim + 8]
  __nv_bfloat16* Kb = Qs + kCaTile * ldq;                            // two buffers of [64][dim + 8]
  __nv_bfloat16* Vb = Kb + 2 * kCaTile * ldq;                        // two buffers of [64][vdim + 8]
  pdl_launch_dependents();
  int r, tile;
  if (!ca_tile_of_block(q_indptr, rows, (int)gridDim.x - 1 - (int)blockIdx.x, r, tile)) return;
  const int h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = q_indptr[r] + tile * kCaTile;
  const int n_valid = min(kCaTile, q_indptr[r + 1] - t0);
  const int p0 = positions[t0];
  if (p0 < 0) return;                                          // a padding row
  const int p_last = p0 + n_valid - 1;
  const __nv_bfloat16* krow = keys + ((size_t)r * stride) * heads * dim + (size_t)h * dim;
  const __nv_bfloat16* vrow = values + ((size_t)r * stride) * heads * vdim + (size_t)h * vdim;
  pdl_wait();
  const int qchunks = dim / 8, vchunks = vdim / 8;
  for (int idx = tid; idx < kCaTile * qchunks; idx += 128) {
    const int row = idx / qchunks, c = (idx % qchunks) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n_valid) v = *reinterpret_cast<const uint4*>(q + (size_t)(t0 + row) * ld_q + (size_t)h * dim + c);
    *reinterpret_cast<uint4*>(Qs + row * ldq + c) = v;
  }
  __syncthreads();
  uint32_t qa[DMAX / 16][4];
#pragma unroll
  for (int ks = 0; ks < DMAX / 16; ++ks)
    if (ks * 16 < dim) ca_ldmatrix_x4(qa[ks], Qs + (warp * 16 + (lane & 15)) * ldq + ks * 16 + (lane >> 4) * 8);
  float o[VMAX / 8][4];
#pragma unroll
  for (int n = 0; n < VMAX / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;   // running maxima (in units of log2) and denominators of the thread's two rows
  const int row_lo = warp * 16 + (lane >> 2);
  const int pos_lo = p0 + row_lo, pos_hi = pos_lo + 8;
  const int n_tiles = p_last / kCaTile + 1;
  auto fetch = [&](int kt) {
    const int k0 = kt * kCaTile;
    __nv_bfloat16* Kd = Kb + (kt & 1) * kCaTile * ldq;
    __nv_bfloat16* Vd = Vb + (kt & 1) * kCaTile * ldv;
    for (int idx = tid; idx < kCaTile * (qchunks + vchunks); idx += 128) {
      const bool is_k = idx < kCaTile * qchunks;
      const int i2 = is_k ? idx : idx - kCaTile * qchunks;
      const int per = is_k ? qchunks : vchunks;
      const int key = i2 / per, c = (i2 % per) * 8;
      const int kp = min(k0 + key, p_last);
      const __nv_bfloat16* src = is_k ? krow + (size_t)kp * heads * dim + c : vrow + (size_t)kp * heads * vdim + c;
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(is_k ? Kd + key * ldq + c : Vd + key * ldv + c);
      const int bytes = k0 + key <= p_last ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  fetch(0);
  for (int kt = 0; kt < n_tiles; ++kt) {
    const int k0 = kt * kCaTile;
    const __nv_bfloat16* Ks = Kb + (kt & 1) * kCaTile * ldq;
    const __nv_bfloat16* Vs = Vb + (kt & 1) * kCaTile * ldv;
    if (kt + 1 < n_tiles) {
      fetch(kt + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    if (k0 <= p0 + warp * 16 + 15) {                            // else every key of the tile lies after the warp's last query
      float s[kCaTile / 8][4];
#pragma unroll
      for (int n = 0; n < kCaTile / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DMAX / 16; ++ks) {
        if (ks * 16 < dim) {
#pragma unroll
          for (int np = 0; np < kCaTile / 16; ++np) {
            uint32_t b[4];
            ca_ldmatrix_x4(b, Ks + (np * 16 + (lane & 7) + (lane >> 4) * 8) * ldq + ks * 16 + ((lane >> 3) & 1) * 8);
            ca_mma_bf16(s[2 * np], qa[ks], b[0], b[1]);
            ca_mma_bf16(s[2 * np + 1], qa[ks], b[2], b[3]);
          }
        }
      }
      // scores in units of log2, keys after the query's position hidden; the tile's maxima a row
      const bool diagonal = k0 + kCaTile - 1 > p0 + warp * 16;
      float t_lo = -INFINITY, t_hi = -INFINITY;
#pragma unroll
      for (int n = 0; n < kCaTile / 8; ++n) {
        const int j = k0 + n * 8 + (lane & 3) * 2;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float z = s[n][e] * scale_log2e;
          if (diagonal && j + (e & 1) > (e < 2 ? pos_lo : pos_hi)) z = -INFINITY;
          s[n][e] = z;
        }
        t_lo = fmaxf(t_lo, fmaxf(s[n][0], s[n][1]));
        t_hi = fmaxf(t_hi, fmaxf(s[n][2], s[n][3]));
      }
      t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1));
      t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
      t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1));
      t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
      const float n_lo = fmaxf(m_lo, t_lo), n_hi = fmaxf(m_hi, t_hi);
      // a row that has seen no key yet keeps a maximum of -inf: exp2(-inf - (-inf)) must not be formed
      const float c_lo = n_lo == -INFINITY ? 1.f : exp2f(m_lo - n_lo), c_hi = n_hi == -INFINITY ? 1.f : exp2f(m_hi - n_hi);
      const float b_lo = n_lo == -INFINITY ? 0.f : n_lo, b_hi = n_hi == -INFINITY ? 0.f : n_hi;
      m_lo = n_lo;
      m_hi = n_hi;
      l_lo *= c_lo;
      l_hi *= c_hi;
#pragma unroll
      for (int n = 0; n < VMAX / 8; ++n) {
        o[n][0] *= c_lo;
        o[n][1] *= c_lo;
        o[n][2] *= c_hi;
        o[n][3] *= c_hi;
      }
#pragma unroll
      for (int kk = 0; kk < kCaTile / 16; ++kk) {
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int n = 2 * kk + half;
          const float w0 = exp2f(s[n][0] - b_lo), w1 = exp2f(s[n][1] - b_lo), w2 = exp2f(s[n][2] - b_hi), w3 = exp2f(s[n][3] - b_hi);
          l_lo += w0 + w1;
          l_hi += w2 + w3;
          ca_split_pair(w0, w1, hi[2 * half], lo[2 * half]);
          ca_split_pair(w2, w3, hi[2 * half + 1], lo[2 * half + 1]);
        }
        const uint32_t ah[4] = {hi[0], hi[1], hi[2], hi[3]}, al[4] = {lo[0], lo[1], lo[2], lo[3]};
#pragma unroll
        for (int np = 0; np < VMAX / 16; ++np) {
          if (np * 16 < vdim) {
            uint32_t b[4];
            ca_ldmatrix_x4_trans(b, Vs + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldv + np * 16 + (lane >> 4) * 8);
            ca_mma_bf16(o[2 * np], ah, b[0], b[1]);
            ca_mma_bf16(o[2 * np], al, b[0], b[1]);
            ca_mma_bf16(o[2 * np + 1], ah, b[2], b[3]);
            ca_mma_bf16(o[2 * np + 1], al, b[2], b[3]);
          }
        }
      }
    }
    __syncthreads();                                           // everybody is done with the buffer the next fetch fills
  }
  // the denominators: a row's four threads hold a quarter of its keys each
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float i_lo = l_lo > 0.f ? 1.0f / l_lo : 0.f, i_hi = l_hi > 0.f ? 1.0f / l_hi : 0.f;
#pragma unroll
  for (int n = 0; n < VMAX / 8; ++n) {
    if (n * 8 < vdim) {
      const int c = n * 8 + (lane & 3) * 2;
      if (row_lo < n_valid)
        *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(t0 + row_lo) * heads + h) * vdim + c) = __floats2bfloat162_rn(o[n][0] * i_lo, o[n][1] * i_lo);
      if (row_lo + 8 < n_valid)
        *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(t0 + row_lo + 8) * heads + h) * vdim + c) = __floats2bfloat162_rn(o[n][2] * i_hi, o[n][3] * i_hi);
    }
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_latent_gather(const void* pool, void* out, const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, int rows,
                                   int stride, int width, int page_size, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && stride > 0 && width > 0 && page_size > 0, "latent_gather: sizes must be positive");
  ROOST_REQUIRE(pool && out && kv_lens && kv_indptr && kv_indices, "latent_gather: a pointer is null");
  if (rows == 0) return ROOST_OK;
  if (rows > 65535) return fail(ROOST_ERR_UNSUPPORTED, "latent_gather: too many rows");
  launch_kernel(latent_gather_kernel, dim3(stride, rows), dim3(width >= 256 ? 128 : 64), 0, (cudaStream_t)stream, (const __nv_bfloat16*)pool,
                (__nv_bfloat16*)out, kv_lens, kv_indptr, kv_indices, stride, width, page_size);
  return check_launch("latent_gather");
}

extern "C" int roost_carried_attention_supported(int dim, int vdim) { return dim % 16 == 0 && vdim % 16 == 0 && dim <= 128 && vdim <= 128; }

// q: the heads' queries, rows ld_q apart (head h at column h * dim); out [tokens, heads * vdim]; keys [rows * stride, heads * dim] and
// values [rows * stride, heads * vdim]: entry r * stride + j is row r's token at position j. All bfloat16.
extern "C" int roost_carried_attention(const void* q, int64_t ld_q, void* out, const void* keys, const void* values, const int32_t* positions,
                                       const int32_t* q_indptr, int tokens, int rows, int heads, int dim, int vdim, int stride, float scale,
                                       roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && rows >= 0 && heads > 0 && stride > 0 && scale > 0.f, "carried_attention: sizes and the scale must be positive");
  ROOST_REQUIRE(q && out && keys && values && positions && q_indptr, "carried_attention: a pointer is null");
  if (!roost_carried_attention_supported(dim, vdim)) return fail(ROOST_ERR_UNSUPPORTED, "carried_attention: sizes no tensor-core form serves");
  ROOST_REQUIRE((uintptr_t)q % 16 == 0 && ld_q % 8 == 0 && ld_q >= (int64_t)heads * dim && (uintptr_t)keys % 16 == 0 && (uintptr_t)values % 16 == 0 &&
                    (uintptr_t)out % 4 == 0,
                "carried_attention: a pointer is not aligned");
  if (tokens == 0 || rows == 0) return ROOST_OK;
  if (heads > 65535) return fail(ROOST_ERR_UNSUPPORTED, "carried_attention: too many heads");
  const size_t smem = ((size_t)3 * kCaTile * (dim + 8) + (size_t)2 * kCaTile * (vdim + 8)) * sizeof(__nv_bfloat16);
  dim3 grid((tokens + kCaTile - 1) / kCaTile + rows, heads);
  const float scale_log2e = scale * 1.4426950408889634f;
#define ROOST_CA(DMAX, VMAX)                                                                                                                      \
  do {                                                                                                                                            \
    auto kernel = carried_attention_kernel<DMAX, VMAX>;                                                                                           \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                   \
    launch_kernel(kernel, grid, dim3(128), smem, (cudaStream_t)stream, (const __nv_bfloat16*)q, ld_q, (__nv_bfloat16*)out,                        \
                  (const __nv_bfloat16*)keys, (const __nv_bfloat16*)values, positions, q_indptr, rows, heads, dim, vdim, stride, scale_log2e);    \
  } while (0)
  if (dim <= 64 && vdim <= 64) ROOST_CA(64, 64);
  else if (dim <= 64) ROOST_CA(64, 128);
  else if (vdim <= 64) ROOST_CA(128, 64);
  else ROOST_CA(128, 128);
#undef ROOST_CA
  return check_launch("carried_attention");
}
