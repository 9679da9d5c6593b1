/*
 * relation_lm_b200 — C ABI of the B200 (sm_100a) implementation of Relation
 * LM's routed selection-and-reduction path.
 *
 * Every entry point mirrors one operator of the reference project (path and
 * line of the Python/Triton operator it replaces are cited per function; paths
 * are relative to the reference project root).  A binding passes raw device
 * pointers, sizes and a CUDA stream; nothing here depends on PyTorch.
 *
 * Conventions
 *   - All pointers are DEVICE pointers unless stated otherwise.  Tensors are
 *     row-major contiguous unless a stride argument says otherwise.
 *   - Float tensors carry an rlm_dtype code and are up-cast to fp32 on load;
 *     all arithmetic is fp32.  Tensors read by bulk (TMA) copies — key caches,
 *     block statistics, the partner-anchor cache — must be 16-byte aligned.
 *   - `position` is a device int64 scalar shared by the whole batch (the
 *     reference reads it on the device so that a captured CUDA graph sees new
 *     positions).  The *_rows variants take per-row int32 sequence and
 *     position arrays instead (`position` may then be NULL).
 *   - Calls validate their arguments on the host and return a negative
 *     rlm_status WITHOUT launching when something is wrong.  They never
 *     allocate, never synchronise and never throw.  Work is enqueued on
 *     `stream` (a cudaStream_t passed as void*).
 *   - `status` (optional, may be NULL) is a device int32 word.  A kernel that
 *     detects a device-side problem (bounded wait expired, position outside
 *     the cache) ORs an RLM_DEV_* bit into it and returns early; it never
 *     traps.  The caller zeroes and reads it.
 */
#ifndef RELATION_LM_B200_H
#define RELATION_LM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RLM_ABI_VERSION 2

typedef enum { RLM_F32 = 0, RLM_BF16 = 1, RLM_F16 = 2 } rlm_dtype;

typedef enum {
    RLM_OK = 0,
    RLM_ERR_NULL = -1,        /* a required pointer is NULL */
    RLM_ERR_SHAPE = -2,       /* unsupported or inconsistent sizes */
    RLM_ERR_DTYPE = -3,       /* unknown dtype code */
    RLM_ERR_ALIGN = -4,       /* a bulk-copied tensor is not 16-byte aligned */
    RLM_ERR_SMEM = -5,        /* the per-row working set exceeds shared memory */
    RLM_ERR_LAUNCH = -6,      /* the CUDA runtime refused the launch */
    RLM_ERR_UNSUPPORTED = -7  /* valid request this build does not implement */
} rlm_status;

#define RLM_DEV_TIMEOUT 1      /* a bounded wait on a bulk copy expired */
#define RLM_DEV_POSITION 2     /* position / row index outside the caches */

/*
 * Programmatic dependent launch (extension; off by default).  When enabled, every kernel of this
 * library is launched with programmatic stream serialisation: its CTAs may start while the kernel
 * before it on the stream is still running, set up their barriers / tensor memory, request their
 * weight tiles and affine parameters and, for the decode form of the selectors, request the key-cache windows and block
 * statistics, and only then wait for the earlier kernels to complete.  Results are unchanged
 * provided the caller keeps one rule: the key caches, block statistics and the `position` scalar
 * passed to a selector must not be written by the kernel launched immediately before it on the
 * same stream (in a decode step they are written by the cache append, several launches earlier).
 * Returns the previous setting.  The setting belongs to the calling host thread (another thread's
 * launches are not affected) and is read at launch (capture) time.
 */
int rlm_set_programmatic_launch(int enabled);

/* Library identity.  rlm_last_error() returns a host string describing the
 * last non-zero status returned on the calling thread. */
int rlm_abi_version(void);
const char* rlm_last_error(void);
/* Number of kernels this library has launched since it was loaded (host counter). */
int64_t rlm_launch_count(void);

/*
 * Fused anchor + partner selection for the current position.
 * Replaces relation_lm::relation_select_packed
 * (src/relation_lm/kernels/relation_select.py:311-382, kernel :9-308).
 *
 *   anchor_query [N,64], anchor_router_query [N,64], partner_base [N,128]   query_dtype
 *     (unit inner stride; row strides in ELEMENTS are passed, so the three may be column
 *     slices of one query-side projection)
 *   anchor_keys, partner_keys [B,T,64]; partner_anchor_cache [B,T,128]      key_dtype
 *   *_mean, *_std [B,NB,4,16]                                               stats_dtype
 *   *_gamma [4], *_bias [4,buckets]                                         param_dtype
 *   out_anchor [N] i32, out_anchor_score [N] f32,
 *   out_partner [N,k_out] i32, out_partner_score [N,k_out] f32
 * Decode form: row_batch = row_position = NULL, N == B, row i uses sequence i
 * at *position.  Rows form: row i uses sequence row_batch[i] at row_position[i].
 * block_size is T / NB.  strict_valid selects the strict remote-block rule
 * (blocks must end before the local window); 0 is the compatibility rule.
 * Empty partner slots carry score -inf and index t - local_window + 1.
 */
int rlm_relation_select_packed(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma,
    const void* anchor_bias, const void* partner_base, const void* partner_anchor_cache,
    const void* partner_keys, const void* partner_mean, const void* partner_std,
    const void* partner_gamma, const void* partner_bias, const int64_t* position,
    const int32_t* row_batch, const int32_t* row_position,
    int32_t* out_anchor, float* out_anchor_score, int32_t* out_partner, float* out_partner_score,
    int64_t anchor_query_stride, int64_t anchor_router_query_stride, int64_t partner_base_stride,
    int n_rows, int n_seq, int max_t, int n_blocks, int buckets,
    int local_window, int top_blocks, int k_out, int strict_valid,
    int query_dtype, int key_dtype, int stats_dtype, int param_dtype,
    int32_t* status, void* stream);

/*
 * Anchor half alone.  Replaces relationlex::anchor_select
 * (src/relation_lm/kernels/triton_select.py:255-295, kernel :9-120).
 * exclude_index (optional, [N, exclude_count] i32, at most 8 per row, entries < 0 unused) bars
 * positions from the candidates: the distinct-anchor rule of multi-anchor selection
 * (src/relation_lm/models/multi_relation_blocks.py:86-95).  A row whose candidates are all
 * barred returns index 0 with score -inf.
 */
int rlm_anchor_select(
    const void* anchor_query, const void* anchor_keys, const void* router_query,
    const void* block_mean, const void* block_std, const void* gamma, const void* bias,
    const int64_t* position, const int32_t* row_batch, const int32_t* row_position,
    const int32_t* exclude_index, int exclude_count,
    int32_t* out_index, float* out_score,
    int n_rows, int n_seq, int max_t, int n_blocks, int buckets,
    int local_window, int top_blocks, int strict_valid,
    int query_dtype, int key_dtype, int stats_dtype, int param_dtype,
    int32_t* status, void* stream);

/*
 * Partner half alone, exact and router queries precomputed by the caller.
 * Replaces relationlex::partner_topk
 * (src/relation_lm/kernels/triton_select.py:298-346, kernel :123-252).
 * anchor_index [N] i32 is excluded from the candidates, and so are the positions of
 * exclude_index (as for rlm_anchor_select): the "no anchor of any slot is a partner" rule of
 * multi-anchor selection (src/relation_lm/models/multi_relation_blocks.py:133-139).
 */
int rlm_partner_topk(
    const void* partner_query, const void* partner_keys, const void* router_query,
    const void* block_mean, const void* block_std, const void* gamma, const void* bias,
    const int64_t* position, const int32_t* row_batch, const int32_t* row_position,
    const int32_t* anchor_index, const int32_t* exclude_index, int exclude_count,
    int32_t* out_index, float* out_score,
    int n_rows, int n_seq, int max_t, int n_blocks, int buckets,
    int local_window, int top_blocks, int k_out, int strict_valid,
    int query_dtype, int key_dtype, int stats_dtype, int param_dtype,
    int32_t* status, void* stream);

/*
 * Router state update for the current position.  Replaces
 * relation_lm::router_cache_update
 * (src/relation_lm/kernels/router_cache.py:175-241, kernel :9-172).
 *   anchor_raw, partner_raw [B,64] with row strides in ELEMENTS (views of the
 *   packed projection)                                   raw_dtype
 *   four caches [B,T,64]                                 cache_dtype (mutated at row t)
 *   four stats  [B,NB,4,16]                              stats_dtype (mutated at block t/block_size)
 *   conv weights [64,3]                                  weight_dtype
 *   out [B,2,64] f32: the convolved anchor and partner router keys.
 */
int rlm_router_cache_update(
    const void* anchor_raw, int64_t anchor_raw_stride, const void* partner_raw,
    int64_t partner_raw_stride, void* anchor_raw_cache, void* partner_raw_cache,
    void* anchor_conv_cache, void* partner_conv_cache, void* anchor_mean, void* anchor_std,
    void* partner_mean, void* partner_std, const void* anchor_conv_weight,
    const void* partner_conv_weight, const int64_t* position, float* out,
    int batch, int max_t, int n_blocks, int block_size,
    int raw_dtype, int cache_dtype, int stats_dtype, int weight_dtype,
    int32_t* status, void* stream);

/*
 * Factorised first relation-MLP layer over gathered rows.  Replaces
 * relation_lm::relation_hidden_cached
 * (src/relation_lm/kernels/relation_reduce.py:149-183, kernel :72-146).
 *   expanded_cache [B,T,2H], operand_cache [B,T,R]       cache_dtype
 *   anchor_index [N] i32, partner_index [N,K] i32
 *   product_weight [H,R]                                 weight_dtype
 *   out [N,K,H] out_dtype (the reference operator returns fp32; a 16-bit output feeds the
 *   second MLP layer's GEMM without a cast kernel)
 * row_batch == NULL: row i gathers from sequence i.  Indices outside [0,T)
 * (empty partner slots) are clamped; their output is masked by the reduce op.
 */
int rlm_relation_hidden_cached(
    const void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const void* product_weight, const int32_t* row_batch,
    void* out, int n_rows, int n_seq, int max_t, int relation_dim, int hidden_dim, int k_out,
    int cache_dtype, int weight_dtype, int out_dtype, int32_t* status, void* stream);

/*
 * Same, and first computes the current position's expanded row from
 * operand_cache[b, t], stores it into expanded_cache[b, t] and uses the fresh
 * values wherever an index equals t.  Replaces
 * relation_lm::relation_hidden_cache_update
 * (src/relation_lm/kernels/relation_reduce.py:312-357, kernel :186-309).
 *   anchor_weight, partner_weight, product_weight [H,R]; first_bias [H]   weight_dtype
 */
int rlm_relation_hidden_cache_update(
    void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const void* anchor_weight, const void* partner_weight,
    const void* product_weight, const void* first_bias, const int64_t* position, void* out,
    int batch, int max_t, int relation_dim, int hidden_dim, int k_out,
    int cache_dtype, int weight_dtype, int out_dtype, int32_t* status, void* stream);

/*
 * Per-partner LayerNorm, active-K softmax and weighted sum.  Replaces
 * relation_lm::relation_norm_reduce
 * (src/relation_lm/kernels/relation_reduce.py:420-450, kernel :360-417).
 *   raw [N,K,D] raw_dtype; partner_scores [N,K] f32; norm_weight, norm_bias [D] param_dtype
 *   out [N,D] f32 (may be NULL when residual is given).  row_position == NULL: all rows use
 *   *position.  residual (optional, [N,D] f32, updated in place): residual += (*mix) * context,
 *   the `hidden + sigmoid(mix_logit) * context` of the reference's relation layer
 *   (src/relation_lm/models/stacked_relation.py:124) with mix a device fp32 scalar.
 *   next_normalized (optional, with residual; [N,D] bfloat16 / float16 = next_dtype): LayerNorm of the
 *   updated residual row with next_norm_weight / next_norm_bias [D] f32 and next_norm_eps, i.e. the
 *   normalised input of the next layer's query projection (or of the output heads).
 *   raw_splits > 1: raw is the sum of raw_splits slices raw_split_stride ELEMENTS apart (the output of
 *   rlm_packed_projection with split K); raw_bias (optional, [D] param_dtype) is added to every
 *   partner row (the bias of the second relation-MLP layer).  Both need D a multiple of 8.
 */
int rlm_relation_norm_reduce(
    const void* raw, const float* partner_scores, const void* norm_weight, const void* norm_bias,
    const int64_t* position, const int32_t* row_position, float norm_eps, float* out,
    float* residual, const float* mix, const float* next_norm_weight, const float* next_norm_bias,
    float next_norm_eps, void* next_normalized, int next_dtype, int raw_splits,
    int64_t raw_split_stride, const void* raw_bias,
    int n_rows, int k_out, int dim, int raw_dtype, int param_dtype,
    int32_t* status, void* stream);

/*
 * rlm_relation_norm_reduce in its residual + next-LayerNorm form, followed by the next layer's
 * query projection in the same launch (extension, for decode batches of a few rows):
 *   proj_out[N, proj_out_dim] = next_normalized[N, D] . proj_weight[proj_out_dim, D]^T,
 * the F.linear of the reference's relation layer on its LayerNorm-ed input
 * (src/relation_lm/models/stacked_relation.py:96-104), with fp32 accumulation over the 16-bit
 * normalised row.  A cluster of proj_out_dim / 32 CTAs serves a row.
 *   proj_weight, proj_out, next_normalized: bfloat16 / float16 (next_dtype); D a multiple of 64;
 *   proj_out_dim = 32, 64, ... 256; every row uses *position; other arguments as above.
 */
int rlm_relation_norm_reduce_project(
    const void* raw, const float* partner_scores, const void* norm_weight, const void* norm_bias,
    const int64_t* position, float norm_eps, float* residual, const float* mix,
    const float* next_norm_weight, const float* next_norm_bias, float next_norm_eps, void* next_normalized,
    const void* proj_weight, void* proj_out, int proj_out_dim, int next_dtype, const void* raw_bias,
    int n_rows, int k_out, int dim, int raw_dtype, int param_dtype, int32_t* status, void* stream);

/*
 * Prefill of the router state (extension): raw and convolved router keys and the block
 * statistics of positions [0, length) of ZERO-INITIALISED caches in one launch, leaving the
 * state that `length` successive rlm_router_cache_update calls would leave (including the
 * zero-padded statistics of a trailing partial block; the full-sequence form is
 * DistilledBlockRouter.block_statistics(_causal_conv(keys)), src/relation_lm/routing/block_router.py:51-68).
 *   anchor_raw, partner_raw: [B, length, 64] views with row and batch strides in ELEMENTS.
 */
int rlm_router_cache_prefill(
    const void* anchor_raw, int64_t anchor_row_stride, int64_t anchor_batch_stride,
    const void* partner_raw, int64_t partner_row_stride, int64_t partner_batch_stride,
    void* anchor_raw_cache, void* partner_raw_cache, void* anchor_conv_cache,
    void* partner_conv_cache, void* anchor_mean, void* anchor_std, void* partner_mean,
    void* partner_std, const void* anchor_conv_weight, const void* partner_conv_weight, int length,
    int batch, int max_t, int n_blocks, int block_size, int raw_dtype, int cache_dtype,
    int stats_dtype, int weight_dtype, void* stream);

/*
 * Packed sparse-cache projection on the tensor cores (tcgen05, TMEM accumulator, TMA loads):
 * out[rows, n_out] = x[rows, d_in] . weight[n_out, d_in]^T.  Replaces the F.linear inside
 * PackedSparseCacheProjection.project (src/relation_lm/inference/packed_cache.py:52-57); the
 * caller splits the packed columns.  Also used for the query-side router projections.
 *   x [rows, d_in] with a row stride in ELEMENTS (multiple of 8), weight [n_out, d_in]:
 *   bfloat16 or float16 (in_dtype); out [rows, n_out] contiguous, any rlm_dtype (out_dtype).
 *   d_in a multiple of 8, n_out a multiple of 32; fp32 operands return RLM_ERR_UNSUPPORTED.
 *   bias (optional, [n_out] f32) is added to every row before the output is rounded, as F.linear
 *   with a bias does (the boundary head of the output projection).
 *   k_splits > 1 (split K, for few rows and a long d_in): k_splits CTAs share an output tile and out
 *   becomes k_splits fp32 slices [k_splits, rows, n_out] whose sum is the product (out_dtype
 *   RLM_F32, no bias, k_splits a divisor of d_in / 64); rlm_relation_norm_reduce sums them.
 */
int rlm_packed_projection(const void* x, int64_t x_row_stride, const void* weight,
                          const float* bias, void* out, int rows, int d_in, int n_out, int in_dtype,
                          int out_dtype, int k_splits, int32_t* status, void* stream);

/*
 * LayerNorm fused into the projection, for decode batches (extension):
 * out[rows, n_out] = LayerNorm(x; gamma, beta, eps) . weight[n_out, d_in]^T with the normalised
 * rows rounded to the weight dtype, as the reference's `layer_norm(...)` followed by `F.linear`
 * on a low-precision model does.  gamma = beta = NULL skips the normalisation (plain cast).
 *   x [rows, d_in] fp32, row stride in ELEMENTS (row tiles of 128); d_in a multiple of 64 up to 1024;
 *   weight bfloat16 / float16 [n_out, d_in]; n_out a multiple of 32; out contiguous, any dtype.
 */
int rlm_norm_projection(const float* x, int64_t x_row_stride, const float* gamma,
                        const float* beta, float eps, const void* weight, void* out, int rows,
                        int d_in, int n_out, int weight_dtype, int out_dtype, int32_t* status,
                        void* stream);

/*
 * LayerNorm of fp32 rows into a 16-bit matrix (extension): the first half of
 * rlm_norm_projection for batches beyond one row tile, where normalising once and streaming
 * the result through rlm_packed_projection beats normalising per output-column tile.  Same
 * arithmetic as rlm_norm_projection; gamma = beta = NULL gives a plain cast.  No reference
 * counterpart beyond `layer_norm(...).to(dtype)` in the model code.
 *   x [rows, d_in] fp32, row stride in ELEMENTS; d_in a multiple of 8 up to 1024;
 *   out [rows, d_in] contiguous bfloat16 / float16.
 */
int rlm_layer_norm_cast(const float* x, int64_t x_row_stride, const float* gamma, const float* beta,
                        float eps, void* out, int rows, int d_in, int out_dtype, void* stream);

/*
 * Expanded-cache rows of the current position for every layer of a stack in one launch
 * (extension, tensor cores): expanded[l, b, t, :H] = anchor_weight[l] . operand[l, b, t] + first_bias[l],
 * expanded[l, b, t, H:] = partner_weight[l] . operand[l, b, t].  It is the cache half of
 * rlm_relation_hidden_cache_update (src/relation_lm/kernels/relation_reduce.py:215-251) taken out
 * of the per-layer loop, the "separate_update" mode the reference recommends for batched decode
 * (src/relation_lm/kernels/relation_reduce.py:60-70): the operand rows of position t are all
 * known once the packed projection has been appended, so the per-layer kernels can then use
 * rlm_relation_hidden_cached.
 *   expanded_cache [layers, B, T, 2H], operand_cache [layers, B, T, R], weights [layers, H, R],
 *   first_bias [layers, H]: bfloat16 or float16 (one dtype); R a multiple of 64, H of 128.
 */
int rlm_expanded_cache_append(void* expanded_cache, const void* operand_cache,
                              const void* anchor_weight, const void* partner_weight,
                              const void* first_bias, const int64_t* position, int layers, int batch,
                              int max_t, int relation_dim, int hidden_dim, int dtype,
                              int32_t* status, void* stream);

/*
 * The same with the operand rows of position t taken from the packed projection rows of that
 * position instead of the operand cache: packed [B, row stride] in the caches' dtype, layer l's
 * operand at columns [l * packed_layer_stride + operand_offset, + R) (384 + R and 128 for the layout
 * of rlm_sparse_cache_append).  Same results, but independent of the state append: under
 * programmatic dependent launch the kernel works while the launch right before it (the append) is
 * still running and waits for it only at its end.  Rule for callers: `packed` must come from an
 * earlier launch than the immediate predecessor on the stream.
 */
int rlm_expanded_cache_append_packed(void* expanded_cache, const void* packed, int64_t packed_row_stride,
                                     int packed_layer_stride, int operand_offset,
                                     const void* anchor_weight, const void* partner_weight,
                                     const void* first_bias, const int64_t* position, int layers,
                                     int batch, int max_t, int relation_dim, int hidden_dim,
                                     int dtype, int32_t* status, void* stream);

/*
 * Decode-state append for every layer of a stack in one launch (extension).  Does what a
 * reference decode step does per layer after PackedSparseCacheProjection.project
 * (src/relation_lm/inference/packed_cache.py:52-57): writes the four token features into
 * row t of their caches and runs router_cache_update
 * (src/relation_lm/kernels/router_cache.py:175-241) on the two router slices.
 *   packed [B, layers*(384+R)] packed_dtype, row stride in elements; per layer the columns are
 *     anchor_key 64 | partner_key 64 | operand R | partner_anchor 128 | anchor_router 64 | partner_router 64
 *   anchor_keys, partner_keys [layers,B,T,64]; operand_cache [layers,B,T,R];
 *   partner_anchor_cache [layers,B,T,128]; router caches [layers,B,T,64]      cache_dtype
 *   stats [layers,B,NB,4,16] stats_dtype; conv weights [layers,64,3] weight_dtype
 *   out [layers,B,2,64] f32 or NULL.
 */
int rlm_sparse_cache_append(
    const void* packed, int64_t packed_row_stride, int relation_dim, void* anchor_keys,
    void* partner_keys, void* operand_cache, void* partner_anchor_cache, void* anchor_raw_cache,
    void* partner_raw_cache, void* anchor_conv_cache, void* partner_conv_cache, void* anchor_mean,
    void* anchor_std, void* partner_mean, void* partner_std, const void* anchor_conv_weight,
    const void* partner_conv_weight, const int64_t* position, float* out, int layers, int batch,
    int max_t, int n_blocks, int block_size, int packed_dtype, int cache_dtype, int stats_dtype,
    int weight_dtype, int32_t* status, void* stream);

/*
 * Fused relation tail (extension): second relation-MLP layer + relation_norm_reduce + residual.
 * Does in one launch what a reference decode step does with F.linear(hidden, W2, b2)
 * (benchmarks/benchmark_relation_reduce.py:63) followed by relation_lm::relation_norm_reduce
 * (src/relation_lm/kernels/relation_reduce.py:420-450) and `hidden + sigmoid(mix) * context`
 * (src/relation_lm/models/stacked_relation.py:124).
 *   relation_hidden [B, K, H] and second_weight [d, H], second_bias [d]: bfloat16 or float16 (dtype)
 *   partner_scores [B, K] f32; norm_weight, norm_bias [d] f32; position device int64
 *   residual [B, d] f32 (optional, += (*mix) * context), context [B, d] f32 (optional output)
 *   scratch: caller-owned device memory of at least rlm_relation_tail_scratch_bytes() bytes,
 *   ZERO before the first call; the kernel leaves it zero again, so one buffer serves every
 *   call that is ordered on a stream.  Calls that overlap on the GPU need separate buffers.
 *   A launch that reported RLM_DEV_TIMEOUT through `status` leaves partial sums behind: zero the
 *   buffer again before the next call.
 *   K must divide 128; d a multiple of 64 up to 1024; H a multiple of 8.
 */
int64_t rlm_relation_tail_scratch_bytes(int batch, int k_out, int d_model);
int rlm_relation_tail(const void* relation_hidden, const void* second_weight,
                      const void* second_bias, const float* partner_scores,
                      const float* norm_weight, const float* norm_bias, const int64_t* position,
                      float norm_eps, float* residual, const float* mix, float* context,
                      void* scratch, int64_t scratch_bytes, int batch, int k_out, int d_model,
                      int hidden_dim, int dtype, int32_t* status, void* stream);

/*
 * The whole relation tail of a layer in one launch, for decode batches of a few sequences
 * (extension): relation hidden states (relation_lm::relation_hidden_cached,
 * src/relation_lm/kernels/relation_reduce.py:149-183), the second relation-MLP layer the reference
 * leaves to F.linear (benchmarks/benchmark_relation_reduce.py:55-64), relation_lm::relation_norm_reduce
 * (relation_reduce.py:420-450), `hidden + sigmoid(mix) * context` (models/stacked_relation.py:124),
 * the LayerNorm of the updated row and, with `query_weight`, the next layer's query-side projection.
 * A thread-block cluster of H / 128 CTAs serves up to 64 (sequence, partner) pairs; the hidden
 * states stay on chip (tcgen05 GEMMs chained through shared memory, split-K sums exchanged
 * through distributed shared memory in a fixed order: results are deterministic).
 *   expanded_cache [B,T,2H], operand_cache [B,T,R], product_weight [H,R], second_weight [d,H],
 *   second_bias [d], query_weight [NQ,d] (optional), normalized [B,d] and query [B,NQ] outputs:
 *   all bfloat16 or all float16 (dtype); anchor_index [B], partner_index [B,K] int32 (gathered
 *   indices are clamped to the cache); partner_scores [B,K], norm / next-norm parameters [d],
 *   residual [B,d] (in/out) and mix (one element): float32.
 * Supported: H = 4 d with d in {128, 256, 512}, R a multiple of 64 up to 256, K <= 64, NQ a
 * multiple of 16 * (H / 128) with at most 64 outputs per CTA; anything else returns
 * RLM_ERR_UNSUPPORTED.  rlm_relation_layer_tail_supported() also checks that the device can
 * host one cluster (1 = supported).  No scratch memory is used.
 */
int rlm_relation_layer_tail_supported(int n_seq, int k_out, int relation_dim, int hidden_dim,
                                      int d_model, int n_query, int dtype);
int rlm_relation_layer_tail(
    const void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const float* partner_scores, const void* product_weight,
    const void* second_weight, const void* second_bias, const float* norm_weight, const float* norm_bias,
    const int64_t* position, float norm_eps, float* residual, const float* mix,
    const float* next_norm_weight, const float* next_norm_bias, float next_norm_eps, void* normalized,
    const void* query_weight, void* query, int n_seq, int k_out, int max_t, int relation_dim,
    int hidden_dim, int d_model, int n_query, int dtype, int32_t* status, void* stream);

/*
 * A whole relation layer of a decode step in one launch (extension): rlm_relation_select_packed in
 * its decode form (one query row per sequence, all at *position) followed by
 * rlm_relation_layer_tail, in the tail's cluster.  The first CTAs of a cluster each select for one
 * of the cluster's sequences, in the shared memory the tail's tiles occupy from the gathers on,
 * while the weight slices stream in; the indices and scores are written to the out_* arrays
 * (results identical to the two separate calls, bit for bit) and handed to the tail through a
 * cluster barrier.
 * Arguments: the selector's (see rlm_relation_select_packed; queries, caches and block statistics
 * in `dtype`, router parameters in `param_dtype`), then the tail's.  Supported when the tail is,
 * the selector's working set (block statistics, local window, remote blocks) fits the tile memory
 * (about 45 KB at relation width 64, 53 KB at 128); rlm_relation_layer_supported() answers 1 then, and rlm_relation_layer returns
 * RLM_ERR_UNSUPPORTED otherwise (use the two launches).
 */
int rlm_relation_layer_supported(int n_seq, int k_out, int relation_dim, int hidden_dim, int d_model,
                                 int n_query, int dtype, int max_t, int n_blocks, int buckets,
                                 int local_window, int top_blocks);
int rlm_relation_layer(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    const int64_t* position, int32_t* out_anchor, float* out_anchor_score, int32_t* out_partner,
    float* out_partner_score, int64_t anchor_query_stride, int64_t anchor_router_query_stride,
    int64_t partner_base_stride, int n_blocks, int buckets, int local_window, int top_blocks, int strict_valid,
    int param_dtype,
    const void* expanded_cache, const void* operand_cache, const void* product_weight, const void* second_weight,
    const void* second_bias, const float* norm_weight, const float* norm_bias, float norm_eps, float* residual,
    const float* mix, const float* next_norm_weight, const float* next_norm_bias, float next_norm_eps,
    void* normalized, const void* query_weight, void* query, int n_seq, int k_out, int max_t, int relation_dim,
    int hidden_dim, int d_model, int n_query, int dtype, int32_t* status, void* stream);

/*
 * rlm_relation_tail for callers that cannot hand over scratch memory.  This entry point has no
 * counterpart in the reference project.
 *
 * Who needs it: hosts that are not allowed to allocate device memory once they are running —
 * a serving process that gave all device memory to its own pool at start-up, a plug-in loaded
 * into an engine that owns the allocator, or a latency-critical thread for which the implicit
 * device-wide synchronisation of cudaMalloc / cudaFree is unacceptable.  Such a caller has
 * nowhere to get the split-K accumulator that rlm_relation_tail asks for, so the library keeps
 * one inside its own image: a fixed device array of 512 KB + 256 bytes that every GPU holds
 * from the moment the library is loaded on it until the process ends.
 *
 * Same arguments and results as rlm_relation_tail without `scratch` / `scratch_bytes`.
 *   - Limit: batch * k_out <= 128 and d_model <= 1024; anything larger is rejected with
 *     RLM_ERR_SHAPE before any work is enqueued.
 *   - The function allocates nothing and frees nothing (no cudaMalloc, no cudaFree, no library
 *     routine that allocates).  The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress), remembers it and opts the kernel into its shared-memory size; the
 *     CUDA runtime may also load the kernel and the array onto the device at that moment, which
 *     is the one time device memory is touched on the caller's behalf.  So make one warm-up call
 *     per device at start-up, with the device current and before any stream capture begins;
 *     every later call leaves free device memory unchanged.
 *   - Sizes, dtypes and alignment are checked before anything is put on the stream: a rejected
 *     call has enqueued nothing.
 *   - All calls on one device share the one array, and it still holds what the previous call
 *     left; each call clears the part it uses on `stream` before launching.  Two calls that can
 *     run at the same time on one GPU (different streams without an ordering between them)
 *     would corrupt each other's sums: order them.
 */
int rlm_relation_tail_static(const void* relation_hidden, const void* second_weight,
                             const void* second_bias, const float* partner_scores,
                             const float* norm_weight, const float* norm_bias,
                             const int64_t* position, float norm_eps, float* residual,
                             const float* mix, float* context, int batch, int k_out,
                             int d_model, int hidden_dim, int dtype, int32_t* status,
                             void* stream);

/*
 * Input embedding of one decode position (extension; the reference computes it for whole
 * sequences, src/relation_lm/models/relation_lm.py:130-131):
 * out[b] = (token_table[tokens[b]] + boundary_table[boundaries[b]]) * scale + position_table[*position]
 *   tokens, boundaries [B] int64; tables [V, d] / [Vb, d] table_dtype; position_table [T, d] f32;
 *   out [B, d] f32.  Ids outside the tables set RLM_DEV_POSITION and leave the row unwritten.
 *   norm1_out / norm2_out (optional, [B, d] bfloat16 / float16 = norm_out_dtype): LayerNorm of the
 *   embedded row with norm{1,2}_weight / norm{1,2}_bias [d] f32 and norm_eps — the normalised inputs of
 *   the packed projection (memory norm) and of the first layer's query projection (input norm).
 */
int rlm_decode_embed(const int64_t* tokens, const int64_t* boundaries, const void* token_table,
                     const void* boundary_table, const float* position_table,
                     const int64_t* position, float scale, float* out, int batch, int d_model,
                     int vocab, int boundary_vocab, int max_t, int table_dtype,
                     const float* norm1_weight, const float* norm1_bias, void* norm1_out,
                     const float* norm2_weight, const float* norm2_bias, void* norm2_out,
                     float norm_eps, int norm_out_dtype, int32_t* status, void* stream);

/*
 * Greedy next token (extension): next_token[b] = index of the largest of logits[b, 0:vocab]
 * (ties to the lowest index), the `logits.argmax(-1)` that closes a greedy decode step; with
 * `position` given the device position scalar is advanced by one in the same launch.
 *   logits [rows, >= vocab] any rlm_dtype, row stride in ELEMENTS; next_token [rows] int64.
 */
int rlm_greedy_token(const void* logits, int64_t row_stride, int64_t* next_token, int64_t* position,
                     int rows, int vocab, int dtype, void* stream);

/*
 * Projection of at most 16 rows on the CUDA cores (extension; the F.linear of one decode position,
 * src/relation_lm/inference/packed_cache.py:52-57, and the output heads of
 * src/relation_lm/models/relation_lm.py:121-124, 204-207):
 *   out[m, n] = sum_k x[m, k] * weight[n, k] (+ bias[n])
 *   x [rows, d] (row stride in ELEMENTS), weight [n, d], out [rows, n]: bfloat16 or float16 (dtype),
 *   bias [n] f32 optional; d = 256 or 512 (RLM_ERR_UNSUPPORTED otherwise: use rlm_packed_projection).
 * Greedy head (vocab > 0): also next_token[m] = arg-max of the rounded out[m, 0:vocab] (lowest index
 * on ties) as int64 and, with `position`, the device position scalar advanced by one — what
 * rlm_greedy_token does in a launch of its own.  `argmax_scratch` is caller-owned device memory of
 * rlm_skinny_argmax_scratch_bytes() bytes, ZERO before the first call; every launch leaves it
 * zero.  Launches that share it must be ordered on a stream.
 */
int64_t rlm_skinny_argmax_scratch_bytes(void);

/*
 * L2 prefetch of up to 16 address ranges (extension; no counterpart in the reference project): one
 * launch issues `prefetch.global.L2` for every whole 128-byte line of the ranges, in the order
 * given.  It moves nothing into the SMs and nothing depends on it: run it on a side stream at the
 * head of a decode step (a sibling branch of the step's CUDA graph) with the weights and caches the
 * step's later kernels will read, so that a step that starts with a cold L2 does not fetch them
 * from DRAM one dependent round trip at a time.  `ranges` and `bytes` are HOST arrays.
 */
int rlm_l2_prefetch(const void* const* ranges, const int64_t* bytes, int n_ranges, void* stream);

/*
 * Sliding decode state (extension; "persistent ring-buffer state and contexts beyond 512" is an
 * open item of the reference's roadmap, docs/roadmap.md:8 — the reference has no code for it).
 * Every tensor k is a contiguous [n_outer[k], rows[k], row_bytes[k]] array of position-indexed rows
 * (the caches of src/relation_lm/inference/packed_cache.py:10-17 and of
 * src/relation_lm/kernels/router_cache.py:256-291, or the router's block statistics with one row
 * per block); the launch moves rows [shift, rows) to [0, rows - shift) in place and leaves the last
 * `shift` rows as they were.  A decoder whose position has reached its context slides every cache
 * by a whole number of router blocks (and the block statistics by that many blocks), lowers its
 * position by the same number of rows and goes on: the candidates of later steps are the ones a
 * ring buffer of the same capacity would still hold, with positions counted from the oldest row
 * kept.  Up to 16 tensors per call; row_bytes a multiple of 16, bases 16-byte aligned
 * (RLM_ERR_ALIGN); 0 <= shift < rows (RLM_ERR_SHAPE).  The four arrays are HOST arrays.
 */
int rlm_state_slide(void* const* tensors, const int64_t* n_outer, const int64_t* rows,
                    const int64_t* row_bytes, const int64_t* shift_rows, int n_tensors, void* stream);

/*
 * The front of a decode step in one launch (extension): the embedding of one position
 * (src/relation_lm/models/relation_lm.py:130-131: (token + boundary embedding) * scale + position
 * embedding), two LayerNorms of the embedded rows and one projection of each,
 *   out_first [B, n_first]  = LayerNorm(x; norm1) @ weight[:n_first].T
 *   out_second [B, n_second] = LayerNorm(x; norm2) @ weight[n_first:].T
 * (in the decode step: the packed projection of the memory-normed rows,
 * src/relation_lm/inference/packed_cache.py:52-57, and layer 0's query projection of its input-normed
 * rows).  weight [n_first + n_second, d]: the two matrices stacked.  hidden [B, d] fp32 receives x;
 * norm1_out / norm2_out [B, d] (optional) the normalised rows.  Tables, weight and outputs share
 * bfloat16 or float16; position table and LayerNorm parameters fp32.  B <= 16, d in {256, 512},
 * n_first a multiple of 8.  Token / boundary ids out of range set RLM_DEV_POSITION in `status`.
 */
int rlm_decode_front(
    const int64_t* tokens, const int64_t* boundaries, const void* token_table, const void* boundary_table,
    const float* position_table, const int64_t* position, float scale, const float* norm1_weight,
    const float* norm1_bias, const float* norm2_weight, const float* norm2_bias, float norm_eps, const void* weight,
    float* hidden, void* norm1_out, void* norm2_out, void* out_first, void* out_second, int batch, int d_model,
    int n_first, int n_second, int vocab, int boundary_vocab, int max_t, int dtype, int32_t* status, void* stream);
int rlm_skinny_projection(const void* x, int64_t x_row_stride, const void* weight, const float* bias,
                          void* out, int rows, int d_in, int n_out, int dtype, int vocab,
                          void* argmax_scratch, int64_t* next_token, int64_t* position, void* stream);

/*
 * Packed sparse-cache projection of one decode position for every layer, with the state update in
 * its epilogue (extension): what a reference decode step does with
 * PackedSparseCacheProjection.project (src/relation_lm/inference/packed_cache.py:52-57), the four
 * token-cache row writes and relation_lm::router_cache_update (src/relation_lm/kernels/router_cache.py:175-241)
 * per layer, in ONE launch.  Column c of layer l's 384 + R packed columns goes where the state keeps
 * it: anchor key | partner key | operand | partner-anchor -> row *position of the token caches;
 * router keys -> raw cache, three-tap causal convolution, conv cache, and the current block's mean /
 * biased std (ascending rows, the fresh un-rounded value at the current row) — each channel by
 * the thread that holds its output.  Results equal rlm_skinny_projection followed by
 * rlm_sparse_cache_append bit for bit.
 *   x [B <= 16, d] (row stride in ELEMENTS), weight [layers * (384 + R), d], packed_out [B, layers * (384 + R)]
 *   (optional), caches [layers, B, T, w] and statistics [layers, B, NB, 4, 16]: all bfloat16 or all
 *   float16 (dtype); conv weights [layers, 64, 3] f32; d = 256 or 512.
 */
int rlm_packed_projection_append(
    const void* x, int64_t x_row_stride, const void* weight, void* packed_out, int relation_dim,
    void* anchor_keys, void* partner_keys, void* operand_cache, void* partner_anchor_cache,
    void* anchor_raw_cache, void* partner_raw_cache, void* anchor_conv_cache, void* partner_conv_cache,
    void* anchor_mean, void* anchor_std, void* partner_mean, void* partner_std,
    const float* anchor_conv_weight, const float* partner_conv_weight, const int64_t* position,
    int layers, int batch, int d_in, int max_t, int n_blocks, int block_size, int dtype, int32_t* status,
    void* stream);

/*
 * Whole-sequence (prefill) form of rlm_relation_select_packed (extension): query rows
 * b * query_length + t for every position t < query_length of every sequence b; row (b, t) equals
 * the decode operator at position t of sequence b (src/relation_lm/kernels/relation_select.py:50-308),
 * given final block statistics, bit for bit.  One CTA serves a tile of 32 consecutive positions:
 * the block statistics they share and the union of their local windows are staged once; every
 * warp then walks one query's chain at a time (remote blocks are read where they lie).  Same
 * tensors as the decode form without `position`; at most 512 candidates per query.
 */
int rlm_relation_select_packed_prefill(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    int32_t* out_anchor, float* out_anchor_score, int32_t* out_partner, float* out_partner_score,
    int64_t anchor_query_stride, int64_t anchor_router_query_stride, int64_t partner_base_stride,
    int n_seq, int query_length, int max_t, int n_blocks, int buckets, int local_window, int top_blocks, int k_out,
    int strict_valid, int query_dtype, int key_dtype, int stats_dtype, int param_dtype, int32_t* status,
    void* stream);

/*
 * Routed multi-anchor selection, all slots of a query row in one launch (extension).  The
 * reference's multi-anchor layer is dense (src/relation_lm/models/multi_relation_blocks.py:69-148);
 * this applies its rules inside each slot's routed candidate set (local window + that slot's
 * best remote blocks): slot s is active at position t iff s <= t (:82-84); slots choose anchors
 * one after another, positions taken by earlier slots barred (:86-93); an inactive slot reports
 * anchor 0 (:94); every slot's partner selection bars the anchors of all active slots (:133-139);
 * inactive slots have no partners (:140-142); a partner slot is active iff its score is finite
 * (:144-147: inactive partner slots report index 0 and score -inf).
 *   anchor_query, anchor_router_query [N,S,64], partner_base [N,S,128] (query-side half of the
 *   factorised partner query; the anchor-side half comes from partner_anchor_cache)   query_dtype
 *     (slots contiguous inside a row; the row strides in ELEMENTS are passed, so the three may be
 *     column slices of one query-side projection)
 *   anchor_keys, partner_keys [S,B,T,64], partner_anchor_cache [S,B,T,128]              key_dtype
 *   *_mean, *_std [S,B,NB,4,16] stats_dtype; *_gamma [S,4], *_bias [S,4,buckets] param_dtype
 *   row_batch, row_position [N] int32
 *   out_anchor [N,S] i32, out_anchor_score [N,S] f32, out_anchor_active [N,S] u8,
 *   out_partner [N,S,K] i32, out_partner_score [N,S,K] f32.  1 <= S <= 8.
 */
int rlm_relation_select_multi_rows(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    const int32_t* row_batch, const int32_t* row_position, int32_t* out_anchor, float* out_anchor_score,
    uint8_t* out_anchor_active, int32_t* out_partner, float* out_partner_score,
    int64_t anchor_query_stride, int64_t anchor_router_query_stride, int64_t partner_base_stride,
    int n_rows, int n_seq, int slots,
    int max_t, int n_blocks, int buckets, int local_window, int top_blocks, int k_out, int strict_valid,
    int query_dtype, int key_dtype, int stats_dtype, int param_dtype, int32_t* status, void* stream);

/*
 * rlm_relation_select_multi_rows for whole sequences (extension): the query rows are
 * b * query_length + t for every position t < query_length of every sequence b, all tensors bfloat16
 * (router parameters any dtype).  A CTA serves a tile of consecutive positions; the block statistics
 * and the window union of one slot and stream are staged once per tile and phase, and every warp
 * walks its queries through the 2 S phases (anchors of slot 0 .. S - 1, then partners).  Results are
 * those of rlm_relation_select_multi_rows on the same rows, bit for bit.  At most 512 candidates
 * per query (window + remote blocks); other dtypes return RLM_ERR_UNSUPPORTED.
 */
int rlm_relation_select_multi_prefill(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    int32_t* out_anchor, float* out_anchor_score, uint8_t* out_anchor_active, int32_t* out_partner,
    float* out_partner_score, int64_t anchor_query_stride, int64_t anchor_router_query_stride,
    int64_t partner_base_stride, int query_length, int n_seq, int slots, int max_t, int n_blocks, int buckets,
    int local_window, int top_blocks, int k_out, int strict_valid, int query_dtype, int key_dtype, int stats_dtype,
    int param_dtype, int32_t* status, void* stream);

/*
 * Slot mixing of a multi-anchor relation layer (extension; the last lines of
 * MultiAnchorRelationBlock.forward, src/relation_lm/models/multi_relation_blocks.py:170-178):
 *   w[n,s] = slot_weight[s] * active[n,s] / max(sum_s' slot_weight[s'] * active[n,s'], 1e-9)
 *   hidden[n] += (*gate) * sum_s w[n,s] * slot_context[n,s]
 *   slot_context [N,S,d] f32, anchor_active [N,S] u8, slot_weight [S] f32 (softmax of the learned
 *   logits), gate one f32 (sigmoid of the residual gate), hidden [N,d] f32 in/out; S <= 8, d % 4 == 0.
 */
int rlm_slot_mix_residual(const float* slot_context, const uint8_t* anchor_active, const float* slot_weight,
                          const float* gate, float* hidden, int n_rows, int slots, int d_model, void* stream);

/*
 * Self-test of the bounded device-side wait (extension, test support; no counterpart in the
 * reference project).  Launches one CTA that waits, for at most `cycle_limit` SM cycles
 * (1 .. 2^24), on an mbarrier nothing will ever complete, then ORs RLM_DEV_TIMEOUT into *status
 * and returns — the path every kernel of the library takes when one of its bulk copies does not
 * arrive.  `waited_cycles` (optional device int64) receives the cycles spent waiting.
 */
int rlm_selftest_bounded_wait(int32_t* status, int64_t cycle_limit, int64_t* waited_cycles,
                              void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RELATION_LM_B200_H */
