// Grouped-query causal attention whose values have a size of their own and whose softmax may have a sink, in 32-bit
// arithmetic over a paged cache of either dtype.
//
//   prepare:   per token, on a row [q heads | k heads | v heads] of the fused projection: every query and key head has its
//              first rot_dims elements turned in interleaved pairs, (u, v) at (2i, 2i+1) -> (u cos a - v sin a, v cos a + u sin a)
//              with a = position * inv_freq[i] formed in double and reduced to [-pi, pi] (with `halves` the pair is
//              (i, i + rot_dims / 2) instead); then, with eps > 0, the head is
//              divided by sqrt(mean(x^2) + eps) (no weight). Queries are written back in place (or, with q_out, to a dense
//              [tokens, heads, dim] tensor of their own, which the tensor-core attention kernels read), keys and values go to the
//              token's cache slot (slot -1: nothing is written). The cache entry of (page, kv head, offset) starts at
//              ((page * kv_heads + head) * page_size + offset) * entry from k_base (keys) and v_base (values): two planes of one
//              size, or one plane whose entries are [key | value] (v_base = k_base + dim, entry = dim + vdim).
//   attention: one block per (token, key/value head, eight of its query heads, split); a warp a query head; key tiles of 32 at
//              absolute positions staged in shared memory as float32; a lane a key for the scores, a lane a value column for
//              the sums; running maximum and denominator a warp. The sink is a key of score 0 without a value: the running
//              maximum starts at 0 and the denominator at 1. A token's tiles may be dealt to several blocks in ranges
//              (split z of Z takes tiles [z n, (z + 1) n), n from the step's bound on lengths); the partial sums, maxima and
//              denominators are then combined in split order by a second kernel. A padding token (position -1) is skipped.
//              With a window a query at position p sees the keys p - window + 1 .. p: its tiles start at the tile of the first
//              such key, and no page before that tile's is looked up (the cache may have given it back). With a cap c a scaled
//              score s becomes c tanh(s / c).
#include "common.cuh"

namespace roost {

constexpr int kSaTile = 32;
constexpr int kSaWarps = 8;
constexpr int kSaMaxDim = 512;

template <typename T>
__global__ void __launch_bounds__(128) sink_prepare_kernel(T* qkv, int64_t ld, T* q_out, T* k_base, T* v_base, int entry, const double* __restrict__ inv_freq,
                                                          const int32_t* __restrict__ positions, const int32_t* __restrict__ slot_mapping,
                                                          int heads, int kv_heads, int dim, int vdim, int rot_dims, float eps, int page_size,
                                                          int halves) {
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
  const int slot = slot_mapping[t];
  pdl_wait();
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  T* row = qkv + (size_t)t * ld;
  const int pairs = (dim + 1) / 2;
  const size_t page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  for (int h = warp; h < heads + kv_heads; h += nwarps) {           // a warp a query or key head
    T* x = row + (size_t)h * dim;
    float a[kSaMaxDim / 64], b[kSaMaxDim / 64];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kSaMaxDim / 64; ++c) {
      const int j = c * 32 + lane;
      a[c] = b[c] = 0.f;
      if (j < pairs) {
        const int ia = halves && j < half ? j : 2 * j;                 // the pair's elements: (j, j + half) among the rotated ones
        const int ib = halves && j < half ? j + half : 2 * j + 1;      // with `halves`, neighbours otherwise and after them
        float u = to_float(x[ia]);
        float v = ib < dim ? to_float(x[ib]) : 0.f;
        if (j < half) {
          const float ru = u * cs[j] - v * sn[j], rv = v * cs[j] + u * sn[j];
          u = ru;
          v = rv;
        }
        a[c] = u;
        b[c] = v;
        ss = fmaf(u, u, fmaf(v, v, ss));
      }
    }
    ss = warp_sum(ss);
    const float inv = eps > 0.f ? 1.0f / sqrtf(ss / (float)dim + eps) : 1.0f;
    T* dst = q_out != nullptr ? q_out + ((size_t)t * heads + h) * dim : x;
    if (h >= heads) {
      if (slot < 0) continue;          // a padding token: no key is written
      dst = k_base + ((page * kv_heads + (h - heads)) * page_size + off) * entry;
    }
#pragma unroll
    for (int c = 0; c < kSaMaxDim / 64; ++c) {
      const int j = c * 32 + lane;
      if (j < pairs) {
        const int ia = halves && j < half ? j : 2 * j;
        const int ib = halves && j < half ? j + half : 2 * j + 1;
        dst[ia] = from_float<T>(a[c] * inv);
        if (ib < dim) dst[ib] = from_float<T>(b[c] * inv);
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
__global__ void __launch_bounds__(kSaWarps * 32) sink_attention_kernel(const T* __restrict__ qkv, int64_t ld, T* __restrict__ out, float* __restrict__ part,
                                                                     const T* __restrict__ k_base, const T* __restrict__ v_base, int entry,
                                                                     const int32_t* __restrict__ positions, const int32_t* __restrict__ token_row,
                                                                     const int32_t* __restrict__ kv_indptr, const int32_t* __restrict__ kv_indices,
                                                                     int heads, int kv_heads, int dim, int vdim, int page_size, float scale, int sink,
                                                                     int splits, int tiles_per_split, int window, float softcap) {
  extern __shared__ float sm[];
  float* ks = sm;                                          // [tile][dim + 1]
  float* vs = ks + (size_t)kSaTile * (dim + 1);            // [tile][vdim]
  float* qs = vs + (size_t)kSaTile * vdim;                 // [warps][dim]
  float* ps = qs + (size_t)kSaWarps * dim;                 // [warps][tile]
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int group = heads / kv_heads;
  const int blocks_a_group = (group + kSaWarps - 1) / kSaWarps;
  const int g = blockIdx.y / blocks_a_group, hb = blockIdx.y % blocks_a_group;
  const int z = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hg = hb * kSaWarps + warp;                     // the warp's head within the group
  const bool active = hg < group;
  const int h = g * group + hg;
  const int pos = positions[t];
  if (pos < 0) return;                                     // a padding token
  const int r = token_row[t];
  const int32_t* pages = kv_indices + kv_indptr[r];
  pdl_wait();
  if (active) {
    const T* q = qkv + (size_t)t * ld + (size_t)h * dim;
    for (int i = lane; i < dim; i += 32) qs[(size_t)warp * dim + i] = to_float(q[i]);
  }
  float m = -INFINITY, l = 0.f;
  if (sink && z == 0) {
    m = 0.f;
    l = 1.f;
  }
  float acc[kSaMaxDim / 32];
#pragma unroll
  for (int c = 0; c < kSaMaxDim / 32; ++c) acc[c] = 0.f;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;     // the first key the query sees
  const int n_tiles = pos / kSaTile + 1;
  const int first = lo / kSaTile + z * tiles_per_split, last = min(n_tiles, first + tiles_per_split);
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  for (int tile = first; tile < last; ++tile) {
    const int k0 = tile * kSaTile;
    __syncthreads();
    for (int kk = warp; kk < kSaTile; kk += kSaWarps) {      // a warp a key: its entry's address once, the lanes over its numbers
      const int kp = k0 + kk;
      float* kd = ks + (size_t)kk * (dim + 1);
      float* vd = vs + (size_t)kk * vdim;
      if (kp <= pos && kp >= lo) {
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
    s *= scale;
    if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
    if (k0 + lane > pos || k0 + lane < lo) s = -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    const float p = s > -INFINITY ? expf(s - m_new) : 0.f;
    const float keep = m > -INFINITY ? expf(m - m_new) : 0.f;
    l = l * keep + warp_sum(p);
    m = m_new;
    ps[warp * kSaTile + lane] = p;
    __syncwarp();
#pragma unroll
    for (int c = 0; c < kSaMaxDim / 32; ++c) {
      const int i = c * 32 + lane;
      if (i < vdim) {
        float a = acc[c] * keep;
        const float4* p4 = reinterpret_cast<const float4*>(ps + warp * kSaTile);
#pragma unroll
        for (int kk = 0; kk < kSaTile / 4; ++kk) {
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
    float* dst = part + (((size_t)t * heads + h) * splits + z) * (vdim + 2);
#pragma unroll
    for (int c = 0; c < kSaMaxDim / 32; ++c) {
      const int i = c * 32 + lane;
      if (i < vdim) dst[i] = acc[c];
    }
    if (lane == 0) {
      dst[vdim] = m;
      dst[vdim + 1] = l;
    }
    return;
  }
  T* o = out + ((size_t)t * heads + h) * vdim;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int c = 0; c < kSaMaxDim / 32; ++c) {
    const int i = c * 32 + lane;
    if (i < vdim) o[i] = from_float<T>(acc[c] * inv);
  }
}

// The partials of a token's head, combined in split order.
template <typename T>
__global__ void sink_merge_kernel(const float* __restrict__ part, T* __restrict__ out, const int32_t* __restrict__ positions, int heads, int vdim,
                                  int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  if (positions[t] < 0) return;
  const float* src = part + ((size_t)t * heads + h) * splits * (vdim + 2);
  float M = -INFINITY;
  for (int z = 0; z < splits; ++z) M = fmaxf(M, src[(size_t)z * (vdim + 2) + vdim]);
  float L = 0.f;
  for (int z = 0; z < splits; ++z) {
    const float mz = src[(size_t)z * (vdim + 2) + vdim];
    if (mz > -INFINITY) L += src[(size_t)z * (vdim + 2) + vdim + 1] * expf(mz - M);
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  T* o = out + ((size_t)t * heads + h) * vdim;
  for (int i = threadIdx.x; i < vdim; i += blockDim.x) {
    float a = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = src[(size_t)z * (vdim + 2) + vdim];
      if (mz > -INFINITY) a += src[(size_t)z * (vdim + 2) + i] * expf(mz - M);
    }
    o[i] = from_float<T>(a * inv);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_sink_attention_prepare(void* qkv, int64_t ld, void* q_out, void* k_base, void* v_base, int entry, const double* inv_freq,
                                            const int32_t* positions, const int32_t* slot_mapping, int tokens, int heads, int kv_heads, int dim,
                                            int vdim, int rot_dims, float eps, int page_size, int halves, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && page_size > 0, "sink_attention_prepare: sizes must be positive");
  ROOST_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dim, "sink_attention_prepare: the rotated width must be even and at most dim");
  ROOST_REQUIRE(qkv && k_base && v_base && positions && slot_mapping && (rot_dims == 0 || inv_freq), "sink_attention_prepare: a pointer is null");
  ROOST_REQUIRE(ld >= (int64_t)(heads + kv_heads) * dim + (int64_t)kv_heads * vdim && entry >= dim && entry >= vdim,
                "sink_attention_prepare: a row or a cache entry is too narrow");
  if (dim > kSaMaxDim) return fail(ROOST_ERR_UNSUPPORTED, "sink_attention_prepare: heads beyond 512 numbers");
  if (tokens == 0) return ROOST_OK;
  const size_t smem = ((size_t)rot_dims + 2) * sizeof(float);
  // four warps a token: measured faster than a warp a head (sixteen warps: 30.7 against 19.6 us at 2,048 tokens of 16 + 4 heads of 64)
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(sink_prepare_kernel<T>, dim3(tokens), dim3(128), smem, (cudaStream_t)stream, (T*)qkv, ld, (T*)q_out, (T*)k_base,
                                               (T*)v_base, entry, inv_freq, positions, slot_mapping, heads, kv_heads, dim, vdim, rot_dims, eps,
                                               page_size, halves));
  return check_launch("sink_attention_prepare");
}

extern "C" int roost_sink_attention(const void* qkv, int64_t ld, void* out, float* part, const void* k_base, const void* v_base, int entry,
                                    const int32_t* positions, const int32_t* token_row, const int32_t* kv_indptr, const int32_t* kv_indices,
                                    int tokens, int heads, int kv_heads, int dim, int vdim, int page_size, float scale, int sink, int splits,
                                    int tiles_per_split, int window, float softcap, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && page_size > 0, "sink_attention: sizes must be positive");
  ROOST_REQUIRE(heads % kv_heads == 0, "sink_attention: the query heads are no multiple of the key/value heads");
  ROOST_REQUIRE(window >= 0 && softcap >= 0.f, "sink_attention: the window and the scores' cap cannot be negative");
  ROOST_REQUIRE(splits >= 1 && tiles_per_split >= 1 && (splits == 1 || part != nullptr), "sink_attention: splits need a workspace for their partials");
  if (dim > kSaMaxDim || vdim > kSaMaxDim) return fail(ROOST_ERR_UNSUPPORTED, "sink_attention: heads or values beyond 512 numbers");
  const int group = heads / kv_heads;
  const int gy = kv_heads * ((group + kSaWarps - 1) / kSaWarps);
  if (splits > 65535 || gy > 65535) return fail(ROOST_ERR_UNSUPPORTED, "sink_attention: too many heads or splits");
  if (tokens == 0) return ROOST_OK;
  const size_t smem = ((size_t)kSaTile * (dim + 1 + vdim) + (size_t)kSaWarps * (dim + kSaTile)) * sizeof(float);
  dim3 grid(tokens, gy, splits);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = sink_attention_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, dim3(kSaWarps * 32), smem, (cudaStream_t)stream, (const T*)qkv, ld, (T*)out, splits > 1 ? part : (float*)nullptr,
                  (const T*)k_base, (const T*)v_base, entry, positions, token_row, kv_indptr, kv_indices, heads, kv_heads, dim, vdim, page_size,
                  scale, sink, splits, tiles_per_split, window, softcap);
    if (splits > 1)
      launch_kernel(sink_merge_kernel<T>, dim3(tokens, heads), dim3(128), 0, (cudaStream_t)stream, (const float*)part, (T*)out, positions, heads,
                    vdim, splits);
  });
  return check_launch("sink_attention");
}
