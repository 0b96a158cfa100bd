// Latent attention: a token's cache entry is one vector [c (rank) | shared rotated key part (rope)]; head h scores a key by
// (q_latent,h . c + q_rot,h . shared part) * scale, where q_latent,h is the head's plain query carried into the latent space,
// and sums p_j c_j over the visible keys j (max(0, pos - window + 1) .. pos; window <= 0: from 0). The heads' sums leave the
// latent space in a product of their own. Scores, softmax weights and sums are 32-bit whatever the cache's dtype is.
//
// latent_prepare: per token, the latent divided by its root mean square (eps inside the root) times a weight, the shared key
// part rotated, both written to the token's cache slot; every head's rotated query part rotated in place. The rotation pairs
// element i with i + dims/2 of the part's first `dims` elements; the angle position * inv_freq[i] is formed in 64-bit and
// reduced to [-pi, pi] before the 32-bit sincosf. rope 0: keys have no rotated part and the entry is the latent alone.
//
// latent_attention: one block per (query token, 8 heads, split); a warp a head. Keys are visited in tiles of 32 at absolute
// positions that are multiples of 32, a lane a key for the scores, a lane a latent dimension for the sums; the tile is read
// once for the block's heads. With splits > 1 the tiles of a token are dealt round-robin to `splits` blocks that leave
// (sum, maximum, denominator) partials, merged in split order by a second kernel: a decode step of few rows then fills the
// device. The order of every sum depends on the token's position, the window and the number of splits only.
#include "common.cuh"

namespace roost {

constexpr int kLaTile = 32;
constexpr int kLaWarps = 8;
constexpr int kLaMaxRank = 1024;

template <typename T>
__global__ void latent_prepare_kernel(T* q, const T* __restrict__ down, T* pool, const float* __restrict__ latent_w,
                                      const double* __restrict__ inv_freq, const int32_t* __restrict__ positions,
                                      const int32_t* __restrict__ slot_mapping, int heads, int nope, int rope, int rot_dims, int rank, float eps) {
  extern __shared__ float sm[];      // rot_dims/2 cosines, rot_dims/2 sines, 32 floats of scratch
  const int half = rot_dims / 2;
  float* cs = sm;
  float* sn = sm + half;
  float* scratch = sm + 2 * half;
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
  const int qh = nope + rope;
  T* qt = q + (size_t)t * heads * qh;
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    T* p = qt + (size_t)h * qh + nope;
    const float u = to_float(p[i]), v = to_float(p[i + half]);
    p[i] = from_float<T>(u * cs[i] - v * sn[i]);
    p[i + half] = from_float<T>(v * cs[i] + u * sn[i]);
  }
  if (down == nullptr) return;
  const int entry = rank + rope;
  const T* dt = down + (size_t)t * entry;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(dt[i]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const int slot = slot_mapping[t];
  if (slot < 0) return;             // a padding token: nothing is written
  const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
  T* e = pool + (size_t)slot * entry;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) e[i] = from_float<T>(to_float(dt[i]) * inv * latent_w[i]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = to_float(dt[rank + i]), v = to_float(dt[rank + i + half]);
    e[rank + i] = from_float<T>(u * cs[i] - v * sn[i]);
    e[rank + i + half] = from_float<T>(v * cs[i] + u * sn[i]);
  }
  for (int i = rot_dims + threadIdx.x; i < rope; i += blockDim.x) e[rank + i] = dt[rank + i];
}

template <typename T>
__global__ void latent_attention_kernel(const T* __restrict__ q_latent, const T* __restrict__ q, T* __restrict__ out, float* __restrict__ part,
                                        const T* __restrict__ pool, const int32_t* __restrict__ positions,
                                        const int32_t* __restrict__ token_row, const int32_t* __restrict__ kv_indptr,
                                        const int32_t* __restrict__ kv_indices, int tokens, int heads, int nope, int rope, int rank,
                                        int page_size, float scale, int window, int splits) {
  extern __shared__ float smem[];
  const int E = rank + rope;
  const int ek = E + 1;                        // padded rows: a lane per key reads without bank conflicts
  float* ks = smem;                            // [kLaTile][E + 1]
  float* qs = ks + kLaTile * ek;               // [kLaWarps][E]
  float* ps = qs + kLaWarps * E;               // [kLaWarps][kLaTile]
  pdl_launch_dependents();
  const int t = blockIdx.x, z = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * kLaWarps + warp;
  const bool active = h < heads;
  const int pos = positions[t];
  const int b = token_row[t];
  const int32_t* pages = kv_indices + kv_indptr[b];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  pdl_wait();
  if (active) {
    const T* ql = q_latent + ((size_t)h * tokens + t) * rank;
    for (int i = lane; i < rank; i += 32) qs[warp * E + i] = to_float(ql[i]);
    const T* qr = q + ((size_t)t * heads + h) * (nope + rope) + nope;
    for (int i = lane; i < rope; i += 32) qs[warp * E + rank + i] = to_float(qr[i]);
  }
  float m = -INFINITY, l = 0.f;
  float o[kLaMaxRank / 32];
#pragma unroll
  for (int i = 0; i < kLaMaxRank / 32; ++i) o[i] = 0.f;

  const int first = lo / kLaTile;
  for (int ti = first + ((z - first % splits) + splits) % splits; ti * kLaTile <= pos; ti += splits) {
    const int j0 = ti * kLaTile;
    __syncthreads();  // the previous tile has been consumed (and qs is written, the first time)
    for (int r = warp; r < kLaTile; r += kLaWarps) {
      const int j = j0 + r;
      if (j >= lo && j <= pos) {
        const int page = pages[j / page_size];
        const T* e = pool + ((size_t)page * page_size + (j % page_size)) * E;
        for (int i = lane; i < E; i += 32) ks[r * ek + i] = to_float(e[i]);
      } else {
        for (int i = lane; i < E; i += 32) ks[r * ek + i] = 0.f;
      }
    }
    __syncthreads();
    if (active) {
      const int j = j0 + lane;
      const bool vis = j >= lo && j <= pos;
      float s = 0.f;
      const float* kr = ks + lane * ek;
      const float* qr = qs + warp * E;
      for (int i = 0; i < E; ++i) s = fmaf(qr[i], kr[i], s);
      s = vis ? s * scale : -INFINITY;
      const float m_new = fmaxf(m, warp_max(s));   // the tile holds at least one visible key
      const float p = vis ? expf(s - m_new) : 0.f;
      const float corr = expf(m - m_new);           // 0 on the first tile (m = -inf)
      l = l * corr + warp_sum(p);
      m = m_new;
      ps[warp * kLaTile + lane] = p;
      __syncwarp();
      const float* pr = ps + warp * kLaTile;
#pragma unroll
      for (int c = 0; c < kLaMaxRank / 32; ++c) {
        const int i = c * 32 + lane;
        if (i < rank) {
          float acc = o[c] * corr;
          for (int r = 0; r < kLaTile; ++r) acc = fmaf(pr[r], ks[r * ek + i], acc);
          o[c] = acc;
        }
      }
      __syncwarp();
    }
  }
  if (!active) return;
  if (part != nullptr) {
    float* dst = part + (((size_t)t * heads + h) * splits + z) * (rank + 2);
#pragma unroll
    for (int c = 0; c < kLaMaxRank / 32; ++c) {
      const int i = c * 32 + lane;
      if (i < rank) dst[i] = o[c];
    }
    if (lane == 0) {
      dst[rank] = m;
      dst[rank + 1] = l;
    }
    return;
  }
  T* ov = out + ((size_t)h * tokens + t) * rank;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int c = 0; c < kLaMaxRank / 32; ++c) {
    const int i = c * 32 + lane;
    if (i < rank) ov[i] = from_float<T>(o[c] * inv);
  }
}

// The partials of a token's head, combined in split order.
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ part, T* __restrict__ out, int tokens, int heads, int rank, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const float* src = part + ((size_t)t * heads + h) * splits * (rank + 2);
  float M = -INFINITY;
  for (int z = 0; z < splits; ++z) M = fmaxf(M, src[(size_t)z * (rank + 2) + rank]);
  float L = 0.f;
  for (int z = 0; z < splits; ++z) {
    const float mz = src[(size_t)z * (rank + 2) + rank];
    if (mz > -INFINITY) L += src[(size_t)z * (rank + 2) + rank + 1] * expf(mz - M);
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  T* ov = out + ((size_t)h * tokens + t) * rank;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = src[(size_t)z * (rank + 2) + rank];
      if (mz > -INFINITY) acc += src[(size_t)z * (rank + 2) + i] * expf(mz - M);
    }
    ov[i] = from_float<T>(acc * inv);
  }
}

}  // namespace roost

using namespace roost;

extern "C" int roost_latent_prepare(void* q, const void* down, void* pool, const float* latent_w, const double* inv_freq,
                                    const int32_t* positions, const int32_t* slot_mapping, int tokens, int heads, int nope, int rope,
                                    int rot_dims, int rank, float eps, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && nope > 0 && rope >= 0 && rank > 0, "latent_prepare: sizes must be positive");
  ROOST_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rope, "latent_prepare: the rotated width must be even and at most rope");
  ROOST_REQUIRE(q && (inv_freq || rot_dims == 0) && positions, "latent_prepare: a pointer is null");
  ROOST_REQUIRE(down == nullptr || (pool && latent_w && slot_mapping && eps > 0.f), "latent_prepare: a latent needs its pool, weight, slots and eps");
  if (tokens == 0) return ROOST_OK;
  const size_t smem = ((size_t)rot_dims + 32) * sizeof(float);
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(latent_prepare_kernel<T>, dim3(tokens), dim3(128), smem, (cudaStream_t)stream, (T*)q, (const T*)down,
                                               (T*)pool, latent_w, inv_freq, positions, slot_mapping, heads, nope, rope, rot_dims, rank, eps));
  return check_launch("latent_prepare");
}

extern "C" int roost_latent_attention(const void* q_latent, const void* q, void* out, float* part, const void* pool, const int32_t* positions,
                                      const int32_t* token_row, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens, int heads,
                                      int nope, int rope, int rank, int page_size, float scale, int window, int splits, int dtype,
                                      roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && heads > 0 && nope > 0 && rope >= 0 && rank > 0 && page_size > 0, "latent_attention: sizes must be positive");
  ROOST_REQUIRE(splits >= 1 && (splits == 1 || part != nullptr), "latent_attention: splits need a workspace for their partials");
  if (rank > kLaMaxRank) return fail(ROOST_ERR_UNSUPPORTED, "latent_attention: a latent of more than 1024 numbers");
  if (splits > 65535 || (heads + kLaWarps - 1) / kLaWarps > 65535) return fail(ROOST_ERR_UNSUPPORTED, "latent_attention: too many heads or splits");
  if (tokens == 0) return ROOST_OK;
  const int E = rank + rope;
  const size_t smem = ((size_t)kLaTile * (E + 1) + (size_t)kLaWarps * E + kLaWarps * kLaTile) * sizeof(float);
  if (smem > 220 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "latent_attention: a cache entry too wide for shared memory");
  dim3 grid(tokens, (heads + kLaWarps - 1) / kLaWarps, splits);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = latent_attention_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, dim3(kLaWarps * 32), smem, (cudaStream_t)stream, (const T*)q_latent, (const T*)q, (T*)out,
                  splits > 1 ? part : (float*)nullptr, (const T*)pool, positions, token_row, kv_indptr, kv_indices, tokens, heads, nope, rope,
                  rank, page_size, scale, window, splits);
    if (splits > 1)
      launch_kernel(latent_merge_kernel<T>, dim3(tokens, heads), dim3(128), 0, (cudaStream_t)stream, (const float*)part, (T*)out, tokens, heads,
                    rank, splits);
  });
  return check_launch("latent_attention");
}
