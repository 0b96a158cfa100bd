// Grouped-query causal attention without a softmax: the weight of a visible key is the sigmoid of its score, and the weights
// are not normalized over the keys. In 32-bit arithmetic over a paged cache of either dtype.
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
  const int first = z * tiles_per_split, last = min(n_tiles, first + tiles_per_split);
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
