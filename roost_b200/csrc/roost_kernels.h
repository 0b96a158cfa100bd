/* roost_b200 kernel library: the C ABI.
 *
 * Every entry point is a plain C function that takes device pointers, sizes and a CUDA stream, launches on
 * that stream and returns a status; nothing here allocates device memory or synchronises. The reference puts
 * its kernels behind a versioned C ABI with status codes and per-op entry points
 * (kernels/include/roost_kernels.h:55-72,107-164,244-262); this is the same boundary with this engine's own
 * op set. A caller checks roost_abi_version() first.
 *
 * dtype codes: 0 = float32, 1 = bfloat16. All index tables are int32. Matrices are row-major.
 */
#ifndef ROOST_B200_KERNELS_H
#define ROOST_B200_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ROOST_ABI_VERSION 15

#define ROOST_OK 0
#define ROOST_ERR_INVALID 1      /* an argument is out of range or inconsistent; nothing was launched */
#define ROOST_ERR_UNSUPPORTED 2  /* the sizes are valid but no kernel serves them; nothing was launched */
#define ROOST_ERR_CUDA 3         /* the CUDA runtime reported an error at launch */

#define ROOST_F32 0
#define ROOST_BF16 1

/* gate functions of gated feed-forwards, applied to the 32-bit gate g and up u: silu(g) u; gelu_tanh(g) u; with g = min(g,
 * limit) and u = clamp(u, -limit, limit): g sigmoid(1.702 g) (u + 1) */
#define ROOST_ACT_SILU 0
#define ROOST_ACT_GELU_TANH 1
#define ROOST_ACT_CLAMPED_SWISH 2

/* Added to the `window` argument of the tensor-core attention entry points (roost_attention_prefill, _decode, _decode_cluster,
 * _decode_static): the softmax's denominator gets one more term, exp(0 - maximum), a key of score 0 that has no value. */
#define ROOST_ATTENTION_SINK (1 << 30)
/* Also added to `window`: the softmax weights enter the second product as two bfloat16 operands, their rounding and what it left
 * over, so that 16 bits of the 32-bit weights count (the denominator is summed from the 32-bit weights anyway). The mma.sync
 * kernels serve it; plan the prefill's work items with roost_attention_prefill_tile_rows_mma. */
#define ROOST_ATTENTION_WIDE_WEIGHTS (1 << 29)
int roost_attention_prefill_tile_rows_mma(int head_dim, int kv_heads, long long packed_rows);

typedef void* roost_stream_t;

int roost_abi_version(void);
/* Programmatic dependent launch for the library's kernels (off by default): a kernel may start its preamble, and the
 * weight-streaming product its first loads of weights, while the kernel before it on the stream is finishing.
 * With it on, a kernel reads before it waits for the kernel in front: weights (norm weights, the products' weight
 * matrices), index tables (the `rows` of the norms, the work lists of the attention kernels, q_indptr, kv_lens,
 * kv_indptr, kv_indices) and pages of the cache that hold only tokens of earlier steps. A caller must therefore not
 * have those written by the kernel launched directly before the call that reads them (a copy in between is enough);
 * activations and the pages of the step's own tokens are read after the wait. */
void roost_set_pdl(int on);
/* Message of the last non-OK status on this thread. */
const char* roost_last_error(void);

/* Writes, in stream order and without synchronising, the error words of the kernels that wait with a limit into
 * out[0..2] (the tcgen05 products, the decode attention, the tcgen05 prefill attention; 0: no wait was given up since
 * the words were last cleared by roost_gemm_tcgen05_status() / roost_attention_status()) and 1 into out[3]. out is
 * device memory, or with out_is_host page-locked host memory (refused when the device cannot write it): a caller that
 * copies a step's results to the host anyway learns of a given-up wait with them, at no extra synchronisation. */
int roost_status_snapshot(int32_t* out, int out_is_host, roost_stream_t stream);

/* out[t,:] = table[ids[t],:]; an id outside [0, vocab) gives a zero row. */
int roost_embedding(const void* table, const int32_t* ids, void* out, int tokens, int hidden, int vocab, int dtype,
                    roost_stream_t stream);

/* out[i,:] = x[r,:] / sqrt(mean(x[r,:]^2) + eps) * w, r = rows ? rows[i] : i. w has dtype wdtype. */
int roost_rms_norm(const void* x, const void* w, void* out, const int32_t* rows, int n_out, int hidden, float eps,
                   int dtype, int wdtype, roost_stream_t stream);

/* s = residual[r,:] + x[r,:] rounded to dtype; out[i,:] = rms_norm(s). Without rows, residual[r,:] = s is
 * written back (the running residual stream); with rows the residual is left as it is. */
int roost_add_rms_norm(const void* x, void* residual, const void* w, void* out, const int32_t* rows, int n_out,
                       int hidden, float eps, int dtype, int wdtype, roost_stream_t stream);

/* out[t,i] = silu(gate_i) * up_i, x: [tokens, 2*inter]. block 0: a row of x is [gate | up]; block b > 0: blocks of b gate
 * values followed by their b up values (the layout the fused product below wants its weight rows in). */
int roost_silu_mul(const void* x, void* out, int tokens, int inter, int block, int dtype, roost_stream_t stream);

/* Per token and head: optional RMS norm over head_dim (q heads with q_w, k heads with k_w), NeoX rotation of
 * the first rotary_dim elements by angle position * inv_freq[i] (inv_freq: double[rotary_dim/2]; rotary_dim 0
 * = no rotation), then q to q_out[t, h, :], k and v into their page slot:
 * pool[(page * kv_heads + h) * page_size + offset][:] with slot = page * page_size + offset from slot_mapping
 * (a negative slot is skipped). qkv rows hold [q heads | k heads | v heads] with row stride qkv_stride
 * elements; with write_kv 0 only the q part is read. cos_sin: null, or the table roost_rope_table made for these
 * positions and this inv_freq (tokens x rotary_dim/2 pairs). */
int roost_qk_norm_rope_cache(const void* qkv, int64_t qkv_stride, void* q_out, void* k_pool, void* v_pool,
                             const void* q_w, const void* k_w, const double* inv_freq, const int32_t* positions,
                             const int32_t* slot_mapping, const float* cos_sin, int tokens, int q_heads, int kv_heads,
                             int head_dim, int rotary_dim, float eps, int page_size, int64_t pool_pages, int write_kv,
                             int dtype, int wdtype, roost_stream_t stream);

/* The cosines and sines of a step's rotations: cos_sin[(t * half + i) * 2 + {0, 1}] = (cos, sin)(positions[t] * inv_freq[i])
 * for i < half, the angle formed in 64-bit and reduced to [-pi, pi] before the 32-bit sincosf. They depend on the
 * positions only, so a step computes them once and hands them to roost_qk_norm_rope_cache of every layer (its cos_sin
 * argument; null there computes the same values in place). */
int roost_rope_table(const int32_t* positions, const double* inv_freq, int tokens, int half, float* cos_sin, roost_stream_t stream);

/* Causal grouped-query attention over a paged cache, one query token per block and key/value head; 32-bit
 * arithmetic throughout. Token t belongs to batch row token_row[t] and sits at absolute position
 * positions[t]; it sees keys max(0, pos - window + 1) .. pos (window <= 0: from 0). Row b's pages are
 * kv_indices[kv_indptr[b] ..]; key j lies in page j / page_size. */
int roost_paged_attention_generic(const void* q, void* out, const void* k_pool, const void* v_pool,
                                  const int32_t* positions, const int32_t* token_row, const int32_t* kv_indptr,
                                  const int32_t* kv_indices, int tokens, int q_heads, int kv_heads, int head_dim,
                                  int page_size, float scale, int window, int dtype, roost_stream_t stream);

/* Tensor-core attention for bfloat16 (attention_mma.cu). head_dim must be one roost_attention_mma_supported accepts.
 * q_indptr[b] .. q_indptr[b+1] are row b's tokens, kv_lens[b] its keys after this step.
 * prefill work: int32 pairs (batch row, first packed row of a tile of tile_rows rows; roost_attention_prefill_tile_rows picks 64 or 128),
 * packed row = token * group + head. With 128-row tiles, head size 64 or 128, a power-of-two number of query heads per
 * key/value head, pages of 16, 32, 64, ... rows and K and V in one allocation, prompt portions run the tcgen05 kernel
 * (attention_tc.cu) unless roost_attention_set_prefill_tc(0) was called; q then has `tokens` rows.
 * decode work: int32 quadruples (batch row, first key, one past the last key, partial slot or -1); rows with at most
 * 16 packed rows only; the first key of an item is a multiple of 64. merge_work: quadruples (batch row, first slot,
 * chunks | packed rows << 24, the row's first token) for rows split into several chunks; merge_rows: the most packed
 * rows any of them has.
 * part_o: float[slots * kv_heads * 16 * head_dim], part_ml: float[slots * kv_heads * 16 * 2].
 * pool_pages: pages of k_pool and v_pool; with head size 64 or 128, pages of 8, 16 or a multiple of 32 rows and pools
 * on 128-byte boundaries, decode streams keys and values through the copy engine (TMA) unless
 * roost_attention_set_decode_tma(0) was called; 0 when not known (the cp.async kernel runs). It copies whole pages:
 * every slot of a page a block table names must be readable, whatever it holds.
 * roost_attention_status(): 0, or the code of a wait the copy-engine kernel gave up, or 9 when a work item named a
 * partial slot beyond the workspace of roost_attention_decode_static (read and cleared). */
int roost_attention_mma_supported(int head_dim);
int roost_attention_prefill_tile_rows(int head_dim, int q_heads, int kv_heads, int page_size, long long pool_pages, const void* k_pool,
                                      const void* v_pool, long long packed_rows);
void roost_attention_set_prefill_tc(int on);
int roost_attention_prefill(const void* q, long long tokens, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                            const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                            int items, int tile_rows, int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages,
                            float scale, int window, roost_stream_t stream);
/* The same with a cap c on the scores: a scaled score s becomes c tanh(s / c) before the mask and the softmax. Served by the mma.sync
 * kernels: items of 64 or 128 packed rows (roost_attention_prefill_tile_rows_mma). */
int roost_attention_prefill_capped(const void* q, long long tokens, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                            const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                            int items, int tile_rows, int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages,
                            float scale, int window, float softcap, roost_stream_t stream);
int roost_attention_decode(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                           const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                           int items, const int32_t* merge_work, int merge_items, int merge_rows, float* part_o, float* part_ml,
                           int q_heads, int kv_heads, int head_dim, int page_size, long long pool_pages, float scale, int window,
                           roost_stream_t stream);
void roost_attention_set_decode_tma(int on);
int roost_attention_status(void);
/* The split decode attention without partial results in memory and without a merge kernel: the grid is thread-block
 * clusters of cluster_chunks (1, 2, 4 or 8) CTAs, one cluster a (row, key/value head). The work list holds exactly
 * cluster_chunks items (batch row, first key, end key, unused) a row, in key order, the row's chunks first and empty
 * items (end key 0) after them; padding rows are cluster_chunks items of batch row -1. CTA r of a cluster takes the
 * row's r-th item and CTA 0 combines the results in that order through distributed shared memory, with the merge
 * kernel's arithmetic: the same bits as roost_attention_decode gives for the same chunks. Served where the copy-engine
 * decode kernel is (roost_attention_decode_cluster_supported). */
int roost_attention_decode_cluster_supported(int head_dim, int page_size, long long pool_pages, int kv_heads, const void* k_pool,
                                             const void* v_pool);
int roost_attention_decode_cluster(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                   const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* work,
                                   int items, int cluster_chunks, int q_heads, int kv_heads, int head_dim, int page_size,
                                   long long pool_pages, float scale, int window, roost_stream_t stream);

/* The split decode attention without a workspace argument. It has no counterpart in the reference: it exists for
 * callers that must not allocate device memory while they run (a host that gave the whole GPU to its own arena at
 * start-up, a loop that may never synchronise the device as cudaMalloc and cudaFree do, a plug-in that may not grow
 * its process's footprint). Same arguments and result as roost_attention_decode, except that the partial results of
 * rows split into several chunks (`slots` of them, as the work lists number them) live in a fixed device array of
 * roost_attention_decode_static_capacity_floats() floats (16 MiB) inside the library, which every process that
 * loads the library holds on each GPU it uses until it exits. It calls no cudaMalloc, cudaFree or other allocating
 * routine. A call whose slots need more than the array holds returns ROOST_ERR_UNSUPPORTED and launches nothing.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device current);
 * make that first call outside any stream capture. All calls share the one array and it keeps what the last call
 * wrote; nothing in it needs clearing, because a call writes every element it later reads. Two calls that overlap
 * on the GPU (different streams, or one stream's call still running when another is launched elsewhere) race on the
 * array: order them on one stream or with events. `slots` must exceed every slot id the work lists name: an item that
 * names a slot at or beyond it is skipped, its output rows stay unwritten and roost_attention_status() returns 9, so that
 * a wrong work list cannot write past the library's array. */
int roost_attention_decode_static_capacity_floats(void);
int roost_attention_decode_static(const void* q, void* out, const void* k_pool, const void* v_pool, const int32_t* q_indptr,
                                  const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices,
                                  const int32_t* work, int items, const int32_t* merge_work, int merge_items, int slots,
                                  int q_heads, int kv_heads, int head_dim, int page_size, float scale, int window,
                                  roost_stream_t stream);

/* out[m,n] = sum_k a[m,k] * w[n,k], plain FFMA in 32-bit (no tensor cores, no reduced-precision mode), the
 * sum over k in increasing order for every output, whatever m is. in_dtype/out_dtype: 0 or 1. */
int roost_gemm_simt(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw,
                    int64_t ldo, int in_dtype, int out_dtype, roost_stream_t stream);


/* out[m,n] = sum_k a[m,k] * w[n,k], bfloat16 operands, 32-bit accumulation in tensor memory (tcgen05.mma fed by TMA;
 * gemm_tcgen05.cu). k and the row strides must be multiples of 8. out_dtype: 1 bfloat16, 0 float32. Every wait inside
 * the kernel is bounded; roost_gemm_tcgen05_status() returns the code of a wait that was given up since the last call
 * (0: none) and synchronises the device. */
int roost_gemm_tcgen05_supported(int m, int n, int k, int64_t lda, int64_t ldw);
int roost_gemm_tcgen05(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw, int64_t ldo,
                       int out_dtype, roost_stream_t stream);
int roost_gemm_tcgen05_status(void);
/* 1 (default): tiles of 256 x 256 on pairs of CTAs (tcgen05 cta_group::2); 0: tiles of 128 x 256 on single CTAs. */
void roost_gemm_tcgen05_set_pairs(int on);
/* The gate/up product with SiLU(gate) * up applied to the accumulator: w [n = 2 * inter, k] with rows in blocks of 128
 * gate rows followed by their 128 up rows; out [m, n / 2] bfloat16. n must be a multiple of 256. */
int roost_gemm_tcgen05_swiglu(const void* a, const void* w, void* out, int m, int n, int k, int64_t lda, int64_t ldw,
                              int64_t ldo, roost_stream_t stream);

/* out[m,n] = sum_k x[m,k] * w[n,k] for 1 <= m <= 64 rows of bfloat16 x: w streamed once by TMA through a persistent
 * CTA per SM, the products on tcgen05 with w's rows as the 128-row operand, the work split into equal contiguous ranges
 * of (128 rows x 64 k) units with a fixed-order fix-up of tiles shared by neighbouring CTAs (gemm_tcgen05.cu).
 * ws: roost_gemm_stream_workspace_floats() floats, flags: roost_gemm_stream_workspace_flags() int32, zero before the first
 * call and left zero by every call. */
int roost_gemm_stream_workspace_floats(void);
int roost_gemm_stream_workspace_flags(void);
int roost_gemm_stream_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_stream(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                      int out_dtype, float* ws, int32_t* flags, roost_stream_t stream);
/* The same product for weights of few 128-row tiles and a long k (an output projection, a down projection): k split
 * over thread-block clusters of up to 8 CTAs, one cluster a tile, the partial sums added up in CTA order through
 * distributed shared memory; no workspace. Supported where roost_gemm_stream is and the tiles are few enough for every
 * cluster to run at once with two CTAs an SM (n up to about 18,900 rows on 148 SMs). */
int roost_gemm_split_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_split_preferred(int m, int n, int k, int64_t ldx, int64_t ldw);  /* measured faster than the other products */
int roost_gemm_split(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                     int out_dtype, roost_stream_t stream);
/* The k-split product with the SwiGLU of the fused product: w's rows in blocks of 256 (128 gate rows, then the 128 up
 * rows of the same outputs), out[m, j] = silu(gate_j) * up_j with n / 2 columns; at most 32 rows of x. */
int roost_gemm_split_swiglu_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_split_swiglu(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                            int out_dtype, roost_stream_t stream);
/* The same with the SwiGLU of the fused product: w's rows in blocks of 256 (128 gate rows, then the 128 up rows of the
 * same outputs), out[m, j] = silu(gate_j) * up_j with n / 2 columns; at most 32 rows of x, n a multiple of 256. */
int roost_gemm_stream_swiglu_supported(int m, int n, int k, int64_t ldx, int64_t ldw);
int roost_gemm_stream_swiglu(const void* x, const void* w, void* out, int m, int n, int k, int64_t ldx, int64_t ldw, int64_t ldo,
                             int out_dtype, float* ws, int32_t* flags, roost_stream_t stream);

/* ids[r] = index of the largest logit of row r, ties to the lowest index, NaN never chosen (-1 if none). */
int roost_argmax(const float* logits, int64_t stride, int rows, int vocab, int32_t* ids, roost_stream_t stream);
/* The same result with a row split over `splits` (1 to 32) blocks, for vocabularies that one SM reads too slowly.
 * part_v, part_i: rows * splits entries of scratch; counters: rows words that are zero before the first call (the
 * kernel leaves them zero). */
int roost_argmax_split(const float* logits, int64_t stride, int rows, int vocab, int32_t* ids, int splits, float* part_v,
                       int32_t* part_i, uint32_t* counters, roost_stream_t stream);

/* Temperature / top-k / top-p / min-p sampling with a Philox4x32-10 draw per row; see sampling.cu.
 * workspace: rows * vocab floats. temperature <= 0 is greedy. */
int roost_sample(const float* logits, int64_t stride, int rows, int vocab, const float* temperature,
                 const int32_t* top_k, const float* top_p, const float* min_p, const uint64_t* seeds,
                 const uint64_t* offsets, float* workspace, int32_t* ids, roost_stream_t stream);

/* What the reference's sampler does beside the draw (src/Starlings.Roost.Ops/CpuOps.Sampling.cs:10-46), in its float32 form.
 * roost_sample_penalise: out[r, v] (rows * vocab floats) = logits[r, v] with the repetition, frequency and presence
 * penalties of row r applied for the tokens counted in counts[row_slot[r], :] (int32 [slots, vocab]: the request's output
 * so far) or named by prompt_bits[row_slot[r], :] (bit v % 32 of word v / 32 of (vocab + 31) / 32 words a slot), and
 * then -inf where the token's bit in mask_bits[row_slot[r], :] is 0 (mask_bits may be null: no token is removed); a row
 * with row_slot < 0 is copied. roost_sample_count_tokens: counts[row_slot[r], ids[r]] += 1. roost_sample_prompt_bits: sets
 * the bits of n token ids in one slot's words. roost_sample_logprobs: logprob[r] = log-softmax of the raw logits of row r
 * at ids[r] (-inf for id -1; logprob may be null), and the `top` highest raw logits of the row, ties to the lower index,
 * with their log-softmax (id -1 and -inf where the row has fewer non-NaN logits). */
int roost_sample_penalise(const float* logits, int64_t stride, int rows, int vocab, float* out, const int32_t* counts,
                          const uint32_t* prompt_bits, const uint32_t* mask_bits, const int32_t* row_slot, const float* repetition,
                          const float* presence, const float* frequency, roost_stream_t stream);
int roost_sample_count_tokens(int32_t* counts, int vocab, const int32_t* row_slot, const int32_t* ids, int rows, roost_stream_t stream);
int roost_sample_prompt_bits(uint32_t* bits, const int32_t* ids, int n, int vocab, roost_stream_t stream);
int roost_sample_logprobs(const float* logits, int64_t stride, int rows, int vocab, const int32_t* ids, float* logprob, int top,
                          int32_t* top_ids, float* top_vals, roost_stream_t stream);

/* ---- a model whose residual stream is kept in 32-bit (wide_stream.cu) ---- */
/* out[t,:] = table[ids[t],:] * scale as float32; an id outside [0, vocab) gives a zero row. */
int roost_embedding_scaled(const void* table, const int32_t* ids, float* out, int tokens, int hidden, int vocab, float scale,
                           int dtype, roost_stream_t stream);
/* s = stream[r,:] (+ addend[r,:], of the activation dtype, when not null) in 32-bit, r = rows ? rows[i] : i; without rows the
 * sum is written back to the stream. out[i,:] = (s - mean) / sqrt(var + eps) * w + b in the activation dtype `dtype`. */
int roost_layer_norm(float* stream, const void* addend, const float* w, const float* b, void* out, const int32_t* rows, int n_out,
                     int hidden, float eps, int dtype, roost_stream_t stream_handle);
/* x <- cap * tanh(x / cap) over n floats. */
int roost_softcap(float* logits, int64_t n, float cap, roost_stream_t stream);
/* `batch` products out[b] = a[b] w[b]^T on FFMA; the batch strides are in elements (see roost_gemm_simt). */
int roost_gemm_simt_batched(const void* a, const void* w, void* out, int batch, int m, int n, int k, int64_t lda, int64_t ldw,
                            int64_t ldo, int64_t batch_a, int64_t batch_w, int64_t batch_o, int in_dtype, int out_dtype,
                            roost_stream_t stream);

/* ---- latent attention (latent_attention.cu) ---- */
/* q: [tokens, heads * (nope + rope)], every head's last `rope` elements rotated in place (their first rot_dims elements,
 * pairs (i, i + rot_dims/2), angle positions[t] * inv_freq[i]). down (may be null): [tokens, rank + rope]; its first `rank`
 * elements divided by their root mean square (eps inside the root) times latent_w, its last `rope` rotated the same way, go
 * to pool[slot_mapping[t] * (rank + rope) ..] (a negative slot is skipped). */
int roost_latent_prepare(void* q, const void* down, void* pool, const float* latent_w, const double* inv_freq,
                         const int32_t* positions, const int32_t* slot_mapping, int tokens, int heads, int nope, int rope,
                         int rot_dims, int rank, float eps, int dtype, roost_stream_t stream);
/* q_latent: [heads, tokens, rank]; q as above (rotated); pool: [pages, page_size, rank + rope]; out: [heads, tokens, rank] =
 * sum_j p_j c_j with p the softmax over the visible keys of (q_latent . c_j + q_rot . r_j) * scale. splits > 1 deals a
 * token's key tiles to that many blocks; part: float[tokens * heads * splits * (rank + 2)]. Tables as in
 * roost_paged_attention_generic. */
int roost_latent_attention(const void* q_latent, const void* q, void* out, float* part, const void* pool, const int32_t* positions,
                           const int32_t* token_row, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens, int heads,
                           int nope, int rope, int rank, int page_size, float scale, int window, int splits, int dtype,
                           roost_stream_t stream);

/* The same on the tensor cores for bfloat16 steps of many tokens (latent_attention_tc.cu): q_indptr[b] .. q_indptr[b+1] are
 * the tokens of batch row b (batch_rows rows). Serves nope and rope that are multiples of 8 and a rank that is a multiple of
 * 16 up to 512. */
int roost_latent_attention_tc_supported(int nope, int rope, int rank);
int roost_latent_attention_tc(const void* q_latent, const void* q, void* out, const void* pool, const int32_t* positions,
                              const int32_t* q_indptr, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens,
                              int batch_rows, int heads, int nope, int rope, int rank, int page_size, float scale, int window,
                              roost_stream_t stream);

/* ---- the Mamba-2 recurrence (mamba2.cu; the layout of a state slot and the formulas are at the top of that file) ---- */
int roost_mamba2_conv(const void* u, int64_t ld, int col, void* out, const float* w, const float* bias, const float* state,
                      int64_t state_stride, int conv_off, const int32_t* token_row, const int32_t* q_indptr, const int32_t* slots,
                      int tokens, int channels, int taps, int act, int dtype, roost_stream_t stream);   /* act != 0: SiLU of the sum */
int roost_mamba2_conv_state(const void* u, int64_t ld, int col, float* state, int64_t state_stride, int conv_off,
                            const int32_t* q_indptr, const int32_t* slots, int rows, int channels, int taps, int dtype,
                            roost_stream_t stream);
int roost_mamba2_scan(const void* xbc, const void* u, int64_t ld_u, int dt_col, float* y, const float* dt_bias, const float* a_log,
                      const float* d_skip, float* state, int64_t state_stride, const int32_t* q_indptr, const int32_t* slots,
                      int rows, int tokens, int heads, int head_dim, int state_rows, int groups, float* ws_state, float* ws_decay,
                      int dtype, roost_stream_t stream);
/* With ws_state (float[chunks * heads * head_dim * state_rows]) and ws_decay (float[chunks * heads]), chunks =
 * roost_mamba2_scan_chunks(tokens, rows), roost_mamba2_scan cuts long rows into chunks that run side by side; with null
 * pointers it walks every row in one pass. */
int roost_mamba2_scan_chunks(int tokens, int rows);
int roost_gated_group_norm(const float* y, const void* u, int64_t ld_u, const float* w, void* out, int tokens, int inner, int groups,
                           float eps, int dtype, roost_stream_t stream);

/* ---- a feed-forward routed over experts (routed_experts.cu) ---- */
int roost_moe_tile_rows(void);   /* rows of a tile of sorted rows */
/* out[t, e] = x[t, :] . w[e, :] in 32-bit. */
int roost_moe_router_logits(const void* x, const void* w, float* out, int tokens, int hidden, int experts, int dtype, roost_stream_t stream);
/* scratch: int32[3 * tokens * top]; tiles: int32[3 * max_tiles], max_tiles >= ceil(tokens * top / tile rows) + experts;
 * counts: int32[experts], zero on entry and left at zero. mode 0: sigmoid scores, compared by logit. mode 1: softmax scores
 * over the `experts` routed columns of a row of `columns` logits, compared with correction[e] (may be null) added; a pair's
 * weight is score * scale. Experts from `real` on (identity experts) get sorted rows but no tiles. */
/* wide_tiles (may be null): the same rows cut into tiles of roost_moe_wide_tile_rows() rows, int32[3 * max_wide_tiles], for
 * roost_gemm_tcgen05_grouped. */
int roost_moe_wide_tile_rows(void);
int roost_moe_route(const float* logits, int tokens, int columns, int experts, int real, int top, int mode, const float* correction,
                    float scale, int32_t* token_of, float* weight_of, int32_t* expert_of, int32_t* inverse, int32_t* offsets, int32_t* tiles,
                    int max_tiles, int32_t* wide_tiles, int max_wide_tiles, int32_t* scratch, int32_t* counts, roost_stream_t stream);
/* Sorted rows against the experts' matrices w [experts, n, k] on tcgen05 (gemm_tcgen05.cu): out[row, :] = a[row, :] w[e]^T, or
 * with gated != 0 (n = 2 * inter, an expert's rows in blocks of 128 gate rows then their 128 up rows) the gate function `act`
 * of gate and up, n / 2 columns. tile_list: the route's wide tiles. k a multiple of 8; gated: n a multiple of 256. */
int roost_gemm_tcgen05_grouped(const void* a, const void* w, void* out, const int32_t* tile_list, int m_tiles, int rows, int experts,
                               int n, int k, int gated, int act, float limit, roost_stream_t stream);
/* xs[row, :] = x[token_of[row], :], times weight_of[row] (rounded once) when scaled != 0. */
int roost_moe_gather_scale(const void* x, void* xs, const int32_t* token_of, const float* weight_of, int rows, int hidden, int scaled,
                           int dtype, roost_stream_t stream);
/* out[row, :] = a[row, :] w1[e]^T (w2 null) or act(a w1[e]^T, a w2[e]^T), e the row's expert; w: [experts, n, k]. With
 * block > 0 the gated form's weights are one tensor, w1 = [experts, 2 n, k], an expert's rows interleaved in blocks of
 * `block` gate rows then their `block` up rows (w2: any non-null value). Rows of experts from `real` on are skipped (form 1;
 * form 0 has no tiles for them). */
int roost_moe_expert_gemm(const void* a, const void* w1, const void* w2, void* out, const int32_t* tiles, int max_tiles,
                          const int32_t* expert_of, int rows, int n, int k, int form, int block, int act, float limit, int real, int dtype,
                          roost_stream_t stream);
int roost_moe_combine(const void* ys, const int32_t* inverse, const void* shared, void* out, int tokens, int hidden, int top, int dtype,
                      roost_stream_t stream);
/* out[t, :] = sum_k weight_of[r] * (expert_of[r] < real ? ys[r, :] : x[t, :]), r = inverse[t * top + k], plus, with shared,
 * sigmoid(gate[t * gate_stride]) * shared[t, :] (gate null: plus shared). */
int roost_moe_combine_weighted(const void* ys, const int32_t* inverse, const float* weight_of, const int32_t* expert_of, const void* x,
                               const void* shared, const float* gate, int gate_stride, void* out, int tokens, int hidden, int top, int real,
                               int dtype, roost_stream_t stream);

/* ---- several 32-bit residual streams a token; gate functions (residual_streams.cu) ---- */
/* streams: float[tokens, n_streams, width]. Per output row i (token t = rows ? rows[i] : i): with init_from every stream
 * becomes a copy of init_from[t, :]; with y (and mix [from, to], write) x'_r = sum_s mix[s, r] x_s + write[r] y[t, :], stored unless
 * rows is given; then u = sum_s read[s] x'_s (read null: the plain sum) and out[i, :] = u / sqrt(mean(u^2) + eps) * norm_w. */
int roost_stream_step(float* streams, const void* y, const void* init_from, const float* mix, const float* write, const float* read,
                      const float* norm_w, const int32_t* rows, void* out, int n_out, int n_streams, int width, float eps, int dtype,
                      roost_stream_t stream);
/* out[t, i] = act(gate[t, i], up[t, i]) over rows [gate | up] (block 0) or blocks of `block` gate then `block` up values. */
int roost_gated_act_mul(const void* x, void* out, int tokens, int inter, int block, int act, float limit, int dtype, roost_stream_t stream);

/* ---- attention with a sink, unit-norm heads and values of their own size (sink_attention.cu) ---- */
/* qkv rows [q heads | k heads | v heads] with row stride ld: rotation of interleaved pairs and unit root mean square (eps <= 0:
 * none) on q (in place, or to the dense [tokens, heads, dim] q_out when it is given) and k; k and v to the cache entry of the token's slot: ((page * kv_heads + head) * page_size + offset) *
 * entry from k_base and v_base. */
int roost_sink_attention_prepare(void* qkv, int64_t ld, void* q_out, void* k_base, void* v_base, int entry, const double* inv_freq,
                                 const int32_t* positions, const int32_t* slot_mapping, int tokens, int heads, int kv_heads, int dim, int vdim,
                                 int rot_dims, float eps, int page_size, int halves, int dtype, roost_stream_t stream);
/* out [tokens, heads * vdim]. sink != 0: one is added to the softmax's denominator. splits > 1: a token's key tiles of 32 are
 * dealt in ranges of tiles_per_split to `splits` blocks whose partials (part: float[tokens * heads * splits * (vdim + 2)]) a
 * second kernel combines. */
int roost_sink_attention(const void* qkv, int64_t ld, void* out, float* part, const void* k_base, const void* v_base, int entry,
                         const int32_t* positions, const int32_t* token_row, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens,
                         int heads, int kv_heads, int dim, int vdim, int page_size, float scale, int sink, int splits, int tiles_per_split,
                         int window, float softcap, int dtype, roost_stream_t stream);   /* window 0: every earlier key; softcap 0: none */

/* ---- the Mamba selective scan (mamba1.cu) ---- */
/* Per (row, channel): dt = softplus(dt_raw + dt_bias); S <- exp(dt a_neg) S + dt x B; y = S . C + d_skip x; out = y silu(z). xc
 * [tokens, inner]; dt_raw float[tokens, inner]; dbc rows [dt | B | C]; xz rows [x | z]; state slots [inner * n_state | ...].
 * With ws_state (float[chunks * inner * n_state]) and ws_dt (float[chunks * inner]), chunks = roost_mamba1_scan_chunks(tokens,
 * rows), rows are cut into chunks of 64 tokens that run side by side (three launches); with null pointers every row is walked
 * in one pass. */
int roost_mamba1_scan_chunks(int tokens, int rows);
int roost_mamba1_scan(const void* xc, const float* dt_raw, const void* dbc, int64_t ld_dbc, const void* xz, int64_t ld_xz, void* out,
                      const float* dt_bias, const float* a_neg, const float* d_skip, float* state, int64_t state_stride,
                      const int32_t* q_indptr, const int32_t* slots, int rows, int tokens, int inner, int n_state, int dt_rank,
                      float* ws_state, float* ws_dt, int dtype, roost_stream_t stream);

/* ---- a 32-bit stream with root-mean-square norms, a hashed pair embedding, token inputs (wide_stream.cu) ---- */
/* s = stream + addend (activation dtype, may be null) + extra (float, may be null), written back unless `rows` gathers; out = s /
 * sqrt(mean(s^2) + eps) * w, or s where w is null. */
int roost_wide_rms_norm(float* stream, const void* addend, const float* extra, const float* w, void* out, const int32_t* rows, int n_out,
                        int hidden, float eps, int dtype, roost_stream_t stream_handle);
/* The same with the addend multiplied element by element by sigmoid(gate + gate_bias) first (gate: float32 [rows, hidden]). */
int roost_wide_rms_norm_gated(float* stream, const void* addend, const float* gate, const float* gate_bias, const float* w, void* out,
                              const int32_t* rows, int n_out, int hidden, float eps, int dtype, roost_stream_t stream_handle);
int roost_scale(float* x, int64_t n, float factor, roost_stream_t stream);   /* x *= factor */
/* out = mean over the n (1 to 4) branches of xs[b] / sqrt(mean(xs[b]^2) + eps) * ws[b]. */
int roost_normed_mean(const void* const* xs, const float* const* ws, int n, void* out, int tokens, int hidden, float eps, int dtype,
                      roost_stream_t stream);
/* out[t] = table[ids[t]] + pairs[row]: row = (previous id * mul_prev + id * mul_cur) mod buckets, `buckets` at position <= 0; the id
 * before a row's first token of the step is state[slots[row]]. */
int roost_pair_embedding(const void* table, const void* pairs, const int32_t* ids, const int32_t* positions, const int32_t* token_row,
                         const int32_t* q_indptr, const int32_t* slots, const int32_t* state, float* out, int tokens, int hidden, int vocab,
                         int buckets, int mul_prev, int mul_cur, int dtype, roost_stream_t stream);
/* state[slots[r]] = the last id of row r (rows without tokens keep theirs). */
int roost_last_token_store(const int32_t* ids, const int32_t* q_indptr, const int32_t* slots, int32_t* state, int rows, roost_stream_t stream);
int roost_add_bias(float* y, const float* bias, int rows, int width, roost_stream_t stream);
/* out[t] = gelu_tanh(gate[t]) * table[ids[t]]. */
int roost_gelu_mul_rows(const void* gate, const void* table, const int32_t* ids, void* out, int tokens, int width, int vocab, int dtype,
                        roost_stream_t stream);

/* ---- the gated linear recurrence (gated_recurrence.cu) ---- */
/* u [tokens, width]; gates float[blocks][tokens][2 * width / blocks]; yx rows [y | ...]; state slots [S: width | ...].
 * ws_state, ws_decay: float[roost_gated_recurrence_scan_chunks(tokens, rows) * width] each, or both null. With them the rows are
 * cut into chunks of 16 tokens that run side by side (three launches); without, every row is walked in one pass. */
int roost_gated_recurrence_scan_chunks(int tokens, int rows);
int roost_gated_recurrence_scan(const void* u, const float* gates, const void* yx, int64_t ld_yx, void* out, const float* gate_bias,
                                const float* decay, float* state, int64_t state_stride, const int32_t* q_indptr, const int32_t* slots,
                                int rows, int tokens, int width, int blocks, float* ws_state, float* ws_decay, int dtype, roost_stream_t stream);

/* ---- the matrix memory (matrix_memory.cu) ---- */
/* qkv rows [q: heads x dim | k: heads x dim | v: heads x vdim | ...]; gates float[tokens][i a head | f a head]; out float[tokens,
 * heads * vdim]; state slots, head after head, [S: dim x vdim | n: dim | m]. */
/* ws: float[roost_matrix_memory_scan_chunks(tokens, rows) * heads * (dim * vdim + dim + 3)], or null. With it the rows are cut into
 * chunks of 64 tokens that run side by side (three launches); without, every row is walked in one pass. */
int roost_matrix_memory_scan_chunks(int tokens, int rows);
int roost_matrix_memory_scan(const void* qkv, int64_t ld, const float* gates, float* out, float* state, int64_t state_stride,
                             const int32_t* q_indptr, const int32_t* slots, int rows, int tokens, int heads, int dim, int vdim, float cap,
                             float floor_, float* ws, int dtype, roost_stream_t stream);
/* out = o / sqrt(mean over a head of o^2 + eps) * w * sigmoid(u[:, col:]); w may be null (no weight); gate_silu: the gate is
 * g sigmoid(g) instead. */
int roost_head_norm_gate(const float* o, const void* u, int64_t ld_u, int col, const float* w, void* out, int tokens, int heads, int vdim,
                         float eps, int gate_silu, int dtype, roost_stream_t stream);

/* ---- retention (retention.cu): S <- decay_h S + k v^T, o = S^T q a head; the slot holds S [heads, dim, vdim] ---- */
/* qk (float32 [tokens, 2 * heads * dim]) = the rotated query heads and the rotated, scaled key heads of rows [q heads | k heads | ...]. */
int roost_retention_prepare(const void* u, int64_t ld, float* qk, const double* inv_freq, const int32_t* positions, int tokens, int heads,
                            int dim, int rot_dims, float k_scale, int dtype, roost_stream_t stream);
/* ws: float[roost_retention_scan_chunks(tokens, rows) * heads * dim * vdim], or null. With it the rows are cut into chunks of 64 tokens
 * that run side by side. v: the values' first column in rows ldv apart; out float32 [tokens, heads * vdim]. */
int roost_retention_scan_chunks(int tokens, int rows);
int roost_retention_scan(const float* qk, const void* v, int64_t ldv, float* out, float* state, int64_t state_stride, const float* decay,
                         const int32_t* q_indptr, const int32_t* slots, int rows, int tokens, int heads, int dim, int vdim, float* ws, int dtype,
                         roost_stream_t stream);

/* ---- attention with sigmoid weights (sigmoid_attention.cu) ---- */
/* Queries and keys divided by their root mean square times q_w / k_w (dim numbers each); queries times
 * 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1) into q_out [tokens, heads, dim]; keys and values into the cache. */
int roost_sigmoid_attention_prepare(const void* qkv, int64_t ld, void* q_out, void* k_base, void* v_base, int entry, const float* q_w,
                                    const float* k_w, const int32_t* positions, const int32_t* slot_mapping, int tokens, int heads, int kv_heads,
                                    int dim, int vdim, float eps, float temp_coef, int temp_every, int page_size, int dtype, roost_stream_t stream);
/* out[t, h] = sum over j <= p of sigmoid((q . k_j) scale - slopes[h] (p - j) + head_bias[h]) v_j, times sigmoid(gate[t, h, :]) where gate is
 * not null (rows ld_gate apart). part: float[tokens * heads * splits * vdim] when splits > 1. */
int roost_sigmoid_attention(const void* q, void* out, float* part, const void* k_base, const void* v_base, int entry, const void* gate,
                            int64_t ld_gate, const float* slopes, const float* head_bias, const int32_t* positions, const int32_t* token_row,
                            const int32_t* kv_indptr, const int32_t* kv_indices, int tokens, int heads, int kv_heads, int dim, int vdim,
                            int page_size, float scale, int splits, int tiles_per_split, int dtype, roost_stream_t stream);

/* The same on the tensor cores (bfloat16; dim and vdim multiples of 16 up to 128, entry a multiple of 8), a block per (row, 64 query
 * tokens, query head): for steps that bring prompt portions. q_indptr: the rows' token ranges (rows + 1 entries). */
int roost_sigmoid_attention_mma_supported(int dim, int vdim, int entry);
int roost_sigmoid_attention_mma(const void* q, void* out, const void* k_base, const void* v_base, int entry, const void* gate, int64_t ld_gate,
                                const float* slopes, const float* head_bias, const int32_t* positions, const int32_t* q_indptr,
                                const int32_t* token_row, const int32_t* kv_indptr, const int32_t* kv_indices, int tokens, int rows, int heads,
                                int kv_heads, int dim, int vdim, int page_size, float scale, float* ws, int tiles_a_chunk, int max_chunks,
                                roost_stream_t stream);   /* max_chunks > 1: a tile's keys in chunks of tiles_a_chunk tiles of 64 keys, their sums
                                                             in ws: float[tokens * heads * max_chunks * vdim]; the last chunk takes what a longer row has left */

/* ---- carried_attention.cu: prompt portions over keys and values carried out of a latent cache for the step (bfloat16) ---- */
/* out [rows * stride, width]: entry r * stride + j is the cached vector of row r's token at position j, zeros from kv_lens[r] on. */
int roost_latent_gather(const void* pool, void* out, const int32_t* kv_lens, const int32_t* kv_indptr, const int32_t* kv_indices, int rows,
                        int stride, int width, int page_size, roost_stream_t stream);
int roost_carried_attention_supported(int dim, int vdim);   /* multiples of 16 up to 128 */
/* Causal softmax attention of the step's queries (rows ld_q apart, head h at column h * dim) over keys [rows * stride, heads * dim] and
 * values [rows * stride, heads * vdim] laid out like the gather's output: out [tokens, heads * vdim]. */
int roost_carried_attention(const void* q, int64_t ld_q, void* out, const void* keys, const void* values, const int32_t* positions,
                            const int32_t* q_indptr, int tokens, int rows, int heads, int dim, int vdim, int stride, float scale,
                            roost_stream_t stream);

/* ---- activations.cu ---- */
/* y = a_pos z^2 + z / 2 (z > 0), a_neg (exp(z) - 1 - z) + z / 2 (z <= 0). */
int roost_xielu(const void* x, void* out, int64_t n, float a_pos, float a_neg, int dtype, roost_stream_t stream);
/* x[t, h, :] *= sigmoid(g[t, col + h]) in place; g's rows are ld_g apart. */
int roost_head_gate_mul(void* x, const void* g, int64_t ld_g, int col, int tokens, int heads, int vdim, int dtype, roost_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
