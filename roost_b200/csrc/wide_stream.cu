// The ends and the norm of a model whose residual stream is kept in 32-bit whatever the activation dtype is: an embedding
// gather that scales (the product formed and stored in 32-bit), a layer norm with weight and bias that first adds a branch
// output to the stream in 32-bit, and the tanh cap of 32-bit logits.
//
// layer norm: y = (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations; mean and var are two
// passes over the row, which a block keeps in shared memory, so that var is a sum of squares of small numbers.
#include "common.cuh"

namespace roost {

template <typename T>
__global__ void embedding_scaled_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids, float* __restrict__ out,
                                        int hidden, int vocab, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const T* src = table + (size_t)(ok ? id : 0) * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_float(src[i]) * scale : 0.f;
}

// One block per output row. addend (may be null): s = stream + addend in 32-bit, written back to the stream unless the rows
// are gathered.
template <typename T>
__global__ void layer_norm_kernel(float* stream, const T* __restrict__ addend, const float* __restrict__ w, const float* __restrict__ b,
                                  T* __restrict__ out, const int32_t* __restrict__ rows, int hidden, float eps) {
  extern __shared__ float row[];  // hidden floats, then 32 floats of reduction scratch
  float* scratch = row + hidden;
  pdl_launch_dependents();
  pdl_wait();
  const int i_out = blockIdx.x;
  const size_t r = rows ? (size_t)rows[i_out] : (size_t)i_out;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = stream[r * hidden + i];
    if (addend) {
      v += to_float(addend[r * hidden + i]);
      if (!rows) stream[r * hidden + i] = v;
    }
    row[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, scratch) / (float)hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row[i] - mean;
    ss += d * d;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)i_out * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>((row[i] - mean) * inv * w[i] + b[i]);
}

// Root-mean-square norm over a 32-bit stream. One block per output row. s = stream + addend (activation dtype, may be null)
// + extra (32-bit, may be null), each sum in 32-bit; s is written back to the stream unless the rows are gathered; the output is
// s / sqrt(mean(s^2) + eps) * w, or s itself where w is null, rounded once.
// With gate (32-bit, [rows, hidden]) the addend is first multiplied element by element by sigmoid(gate + gate_bias): a sublayer's
// output scaled by a gate that was computed from the sublayer's own input.
template <typename T>
__global__ void wide_rms_norm_kernel(float* stream, const T* __restrict__ addend, const float* __restrict__ extra, const float* __restrict__ w,
                                     T* __restrict__ out, const int32_t* __restrict__ rows, int hidden, float eps,
                                     const float* __restrict__ gate, const float* __restrict__ gate_bias) {
  extern __shared__ float row[];  // hidden floats, then 32 floats of reduction scratch
  float* scratch = row + hidden;
  pdl_launch_dependents();
  pdl_wait();
  const int i_out = blockIdx.x;
  const size_t r = rows ? (size_t)rows[i_out] : (size_t)i_out;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = stream[r * hidden + i];
    if (addend) {
      float a = to_float(addend[r * hidden + i]);
      if (gate) a *= 1.0f / (1.0f + expf(-(gate[r * hidden + i] + gate_bias[i])));
      v += a;
    }
    if (extra) v += extra[r * hidden + i];
    if ((addend || extra) && !rows) stream[r * hidden + i] = v;
    row[i] = v;
    ss = fmaf(v, v, ss);
  }
  T* o = out + (size_t)i_out * hidden;
  if (w == nullptr) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>(row[i]);
    return;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>(row[i] * inv * w[i]);
}

// The mean of up to four branch outputs, each divided by its root mean square over the row and multiplied by its weight.
struct NormedMeanArgs {
  const void* x[4];
  const float* w[4];
};

template <typename T>
__global__ void normed_mean_kernel(NormedMeanArgs a, int n, T* __restrict__ out, int hidden, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  float inv[4];
  if constexpr (sizeof(T) == 2) {
    // rows of 16-bit numbers that the block covers with eight a thread: every branch's row is read once, 16 bytes a thread, and kept
    bool aligned = reinterpret_cast<uintptr_t>(out) % 16 == 0;
    for (int b = 0; b < n; ++b) aligned = aligned && reinterpret_cast<uintptr_t>(a.x[b]) % 16 == 0;
    if (aligned && hidden % 8 == 0 && hidden <= (int)blockDim.x * 8) {
      const int i8 = threadIdx.x * 8;
      const bool live = i8 < hidden;
      float v[4][8];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        if (b < n) {
          union { uint4 u; T e[8]; } raw;
          raw.u = live ? *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(a.x[b]) + t * hidden + i8) : make_uint4(0, 0, 0, 0);
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[b][j] = to_float(raw.e[j]);
            ss = fmaf(v[b][j], v[b][j], ss);
          }
          ss = block_sum(ss, scratch);
          inv[b] = 1.0f / sqrtf(ss / (float)hidden + eps);
        }
      }
      if (live) {
        const float share = 1.0f / (float)n;
        union { uint4 u; T e[8]; } res;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float s = 0.f;
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if (b < n) s = fmaf(v[b][j] * inv[b], a.w[b][i8 + j], s);
          res.e[j] = from_float<T>(s * share);
        }
        *reinterpret_cast<uint4*>(out + t * hidden + i8) = res.u;
      }
      return;
    }
  }
  for (int b = 0; b < n; ++b) {
    const T* x = reinterpret_cast<const T*>(a.x[b]) + t * hidden;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = to_float(x[i]);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    inv[b] = 1.0f / sqrtf(ss / (float)hidden + eps);
  }
  const float share = 1.0f / (float)n;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float s = 0.f;
    for (int b = 0; b < n; ++b) s = fmaf(to_float(reinterpret_cast<const T*>(a.x[b])[t * hidden + i]) * inv[b], a.w[b][i], s);
    out[t * hidden + i] = from_float<T>(s * share);
  }
}

// table[id] + pairs[row] as a 32-bit stream; row = (previous id * mul_prev + id * mul_cur) mod buckets, or `buckets` for a
// request's first token (and for padding tokens, position -1). The token before a row's first token of this step is state[slot].
template <typename T>
__global__ void pair_embedding_kernel(const T* __restrict__ table, const T* __restrict__ pairs, const int32_t* __restrict__ ids,
                                      const int32_t* __restrict__ positions, const int32_t* __restrict__ token_row,
                                      const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots, const int32_t* __restrict__ state,
                                      float* __restrict__ out, int hidden, int vocab, int buckets, int mul_prev, int mul_cur) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  int row = buckets;
  if (positions[t] > 0) {
    const int r = token_row[t];
    const int prev = t > q_indptr[r] ? ids[t - 1] : state[slots[r]];
    row = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % buckets);
    if (row < 0) row += buckets;
  }
  const T* a = table + (size_t)(ok ? id : 0) * hidden;
  const T* b = pairs + (size_t)row * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_float(a[i]) + to_float(b[i]) : 0.f;
}

__global__ void last_token_store_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ q_indptr, const int32_t* __restrict__ slots,
                                        int32_t* state, int rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int lo = q_indptr[r], hi = q_indptr[r + 1];
  if (hi > lo) state[slots[r]] = ids[hi - 1];
}

// y[t, :] += bias over 32-bit sums.
__global__ void add_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, size_t n, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] += bias[i % width];
}

// out[t, :] = gelu_tanh(gate[t, :]) * table[ids[t], :], the function on the 32-bit values, rounded once.
template <typename T>
__global__ void gelu_mul_rows_kernel(const T* __restrict__ gate, const T* __restrict__ table, const int32_t* __restrict__ ids, T* __restrict__ out,
                                     int width, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  const T* e = table + (size_t)(ok ? id : 0) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    out[t * width + i] = from_float<T>(ok ? gelu_tanh_f(to_float(gate[t * width + i])) * to_float(e[i]) : 0.f);
}

__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] * inv_cap);
}

__global__ void scale_kernel(float* __restrict__ x, size_t n, float factor) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= factor;
}

}  // namespace roost

using namespace roost;

extern "C" int roost_embedding_scaled(const void* table, const int32_t* ids, float* out, int tokens, int hidden, int vocab, float scale,
                                      int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding_scaled: tokens, hidden and vocab must be positive");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(embedding_scaled_kernel<T>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, (const T*)table, ids,
                                               out, hidden, vocab, scale));
  return check_launch("embedding_scaled");
}

extern "C" int roost_layer_norm(float* stream, const void* addend, const float* w, const float* b, void* out, const int32_t* rows, int n_out,
                                int hidden, float eps, int dtype, roost_stream_t stream_handle) {
  ROOST_REQUIRE(n_out >= 0 && hidden > 0, "layer_norm: rows and hidden must be positive");
  ROOST_REQUIRE(eps > 0.f, "layer_norm: eps must be positive");
  ROOST_REQUIRE(stream && w && b && out, "layer_norm: a pointer is null");
  if (n_out == 0) return ROOST_OK;
  const size_t smem = ((size_t)hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "layer_norm: a row of more than 51168 elements does not fit in shared memory");
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = layer_norm_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream_handle, stream, (const T*)addend, w, b, (T*)out, rows, hidden, eps);
  });
  return check_launch("layer_norm");
}

extern "C" int roost_softcap(float* logits, int64_t n, float cap, roost_stream_t stream) {
  ROOST_REQUIRE(n >= 0 && cap > 0.f, "softcap: the count must not be negative and the cap must be positive");
  if (n == 0) return ROOST_OK;
  const int64_t blocks = (n + 255) / 256;
  if (blocks > 2147483647LL) return fail(ROOST_ERR_UNSUPPORTED, "softcap: too many logits for one launch");
  launch_kernel(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, logits, (size_t)n, cap, 1.0f / cap);
  return check_launch("softcap");
}

extern "C" int roost_wide_rms_norm(float* stream, const void* addend, const float* extra, const float* w, void* out, const int32_t* rows, int n_out,
                                   int hidden, float eps, int dtype, roost_stream_t stream_handle) {
  ROOST_REQUIRE(n_out >= 0 && hidden > 0, "wide_rms_norm: rows and hidden must be positive");
  ROOST_REQUIRE(eps > 0.f, "wide_rms_norm: eps must be positive");
  ROOST_REQUIRE(stream && out, "wide_rms_norm: a pointer is null");
  if (n_out == 0) return ROOST_OK;
  const size_t smem = ((size_t)hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "wide_rms_norm: a row of more than 51168 elements does not fit in shared memory");
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = wide_rms_norm_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream_handle, stream, (const T*)addend, extra, w, (T*)out, rows, hidden, eps,
                  (const float*)nullptr, (const float*)nullptr);
  });
  return check_launch("wide_rms_norm");
}

extern "C" int roost_wide_rms_norm_gated(float* stream, const void* addend, const float* gate, const float* gate_bias, const float* w, void* out,
                                         const int32_t* rows, int n_out, int hidden, float eps, int dtype, roost_stream_t stream_handle) {
  ROOST_REQUIRE(n_out >= 0 && hidden > 0, "wide_rms_norm_gated: rows and hidden must be positive");
  ROOST_REQUIRE(eps > 0.f, "wide_rms_norm_gated: eps must be positive");
  ROOST_REQUIRE(stream && addend && gate && gate_bias && out, "wide_rms_norm_gated: a pointer is null");
  if (n_out == 0) return ROOST_OK;
  const size_t smem = ((size_t)hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return fail(ROOST_ERR_UNSUPPORTED, "wide_rms_norm_gated: a row of more than 51168 elements does not fit in shared memory");
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  ROOST_DISPATCH_DTYPE(dtype, T, {
    auto kernel = wide_rms_norm_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, dim3(n_out), dim3(threads), smem, (cudaStream_t)stream_handle, stream, (const T*)addend, (const float*)nullptr, w, (T*)out,
                  rows, hidden, eps, gate, gate_bias);
  });
  return check_launch("wide_rms_norm_gated");
}

extern "C" int roost_scale(float* x, int64_t n, float factor, roost_stream_t stream) {
  ROOST_REQUIRE(n >= 0 && (n == 0 || x), "scale: a pointer is null");
  if (n == 0) return ROOST_OK;
  const int64_t blocks = (n + 255) / 256;
  if (blocks > 2147483647LL) return fail(ROOST_ERR_UNSUPPORTED, "scale: too many numbers for one launch");
  launch_kernel(scale_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, x, (size_t)n, factor);
  return check_launch("scale");
}

extern "C" int roost_normed_mean(const void* const* xs, const float* const* ws, int n, void* out, int tokens, int hidden, float eps, int dtype,
                                 roost_stream_t stream) {
  ROOST_REQUIRE(n >= 1 && n <= 4, "normed_mean: one to four branches");
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && eps > 0.f && out, "normed_mean: sizes and eps must be positive");
  if (tokens == 0) return ROOST_OK;
  NormedMeanArgs a = {};
  for (int b = 0; b < n; ++b) {
    ROOST_REQUIRE(xs[b] && ws[b], "normed_mean: a pointer is null");
    a.x[b] = xs[b];
    a.w[b] = ws[b];
  }
  const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(normed_mean_kernel<T>, dim3(tokens), dim3(threads), 0, (cudaStream_t)stream, a, n, (T*)out, hidden, eps));
  return check_launch("normed_mean");
}

extern "C" int roost_pair_embedding(const void* table, const void* pairs, const int32_t* ids, const int32_t* positions, const int32_t* token_row,
                                    const int32_t* q_indptr, const int32_t* slots, const int32_t* state, float* out, int tokens, int hidden,
                                    int vocab, int buckets, int mul_prev, int mul_cur, int dtype, roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0 && buckets > 0 && mul_prev >= 0 && mul_cur >= 0, "pair_embedding: sizes must be positive");
  ROOST_REQUIRE(table && pairs && ids && positions && token_row && q_indptr && slots && state && out, "pair_embedding: a pointer is null");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(pair_embedding_kernel<T>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream, (const T*)table,
                                               (const T*)pairs, ids, positions, token_row, q_indptr, slots, state, out, hidden, vocab, buckets,
                                               mul_prev, mul_cur));
  return check_launch("pair_embedding");
}

extern "C" int roost_last_token_store(const int32_t* ids, const int32_t* q_indptr, const int32_t* slots, int32_t* state, int rows,
                                      roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && ids && q_indptr && slots && state, "last_token_store: a pointer is null");
  if (rows == 0) return ROOST_OK;
  launch_kernel(last_token_store_kernel, dim3((rows + 127) / 128), dim3(128), 0, (cudaStream_t)stream, ids, q_indptr, slots, state, rows);
  return check_launch("last_token_store");
}

extern "C" int roost_add_bias(float* y, const float* bias, int rows, int width, roost_stream_t stream) {
  ROOST_REQUIRE(rows >= 0 && width > 0 && y && bias, "add_bias: sizes must be positive");
  const size_t n = (size_t)rows * width;
  if (n == 0) return ROOST_OK;
  launch_kernel(add_bias_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, y, bias, n, width);
  return check_launch("add_bias");
}

extern "C" int roost_gelu_mul_rows(const void* gate, const void* table, const int32_t* ids, void* out, int tokens, int width, int vocab, int dtype,
                                   roost_stream_t stream) {
  ROOST_REQUIRE(tokens >= 0 && width > 0 && vocab > 0 && gate && table && ids && out, "gelu_mul_rows: sizes must be positive");
  if (tokens == 0) return ROOST_OK;
  ROOST_DISPATCH_DTYPE(dtype, T, launch_kernel(gelu_mul_rows_kernel<T>, dim3(tokens), dim3(width >= 256 ? 256 : 64), 0, (cudaStream_t)stream,
                                               (const T*)gate, (const T*)table, ids, (T*)out, width, vocab));
  return check_launch("gelu_mul_rows");
}
