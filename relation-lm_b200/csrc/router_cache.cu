// Router state update for the current position (sm_100a), for one layer
// (the reference operator) or for every layer of a stack in one launch together
// with the token-cache row writes that precede it in a decode step.
//
// One CTA per (sequence, layer), one thread per (stream, channel).  The
// conv-cache tile of the current block is staged in shared memory by two bulk
// copies issued at entry; the three-tap causal convolution, the cache writes
// and the output are done while they fly; block mean and biased standard
// deviation are then accumulated from shared memory in ascending row order
// with the fresh (un-rounded) row substituted at the current position.
//
// Semantics follow src/relation_lm/kernels/router_cache.py:33-172 of the
// reference project; the packed column order is that of
// src/relation_lm/inference/packed_cache.py:10-17.

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kD = 64;
constexpr int kThreads = 2 * kD;

struct RouterArgs {
    const void* raw[2];
    int64_t raw_stride[2];          // row stride of the raw inputs, elements
    int64_t raw_layer_stride;       // distance between layers inside a raw row, elements
    void* raw_cache[2];
    void* conv_cache[2];
    void* mean[2];
    void* stdv[2];
    const void* weight[2];
    const int64_t* position;
    float* out;                     // may be NULL for the stacked form
    int32_t* status;
    int batch, max_t, n_blocks, block_size, layers;
    int raw_dtype, cache_dtype, stats_dtype, weight_dtype;
    // stacked form only: token features copied from the packed row into their caches
    const void* packed;             // [B, layers * packed_width]
    int64_t packed_stride;
    int packed_width;               // 64 + 64 + R + 128 (+ 64 + 64 router columns)
    void* token_cache[4];           // anchor_keys, partner_keys, operand, partner_anchor  [layers,B,T,w]
    int token_width[4];
};

// kBf16: raw keys, caches and statistics are all bfloat16 (the decode step), so their dtype
// branches fold away; the three conv weights of a channel keep their run-time dtype.
template <bool kBf16>
__device__ __forceinline__ void router_update(const RouterArgs& a, int b, int layer,
                                              unsigned char* smem, uint32_t bar, int t) {
    const int tid = threadIdx.x;
    const int raw_dtype = kBf16 ? RLM_BF16 : a.raw_dtype, cache_dtype = kBf16 ? RLM_BF16 : a.cache_dtype,
              stats_dtype = kBf16 ? RLM_BF16 : a.stats_dtype, weight_dtype = a.weight_dtype;
    const int s = tid / kD, c = tid % kD;
    const int bs = a.block_size;
    const int blk = t / bs, start = blk * bs;
    const int cs = cache_dtype == RLM_F32 ? 4 : 2;
    const uint32_t tile_bytes = static_cast<uint32_t>(bs) * kD * cs;
    const int64_t seq = static_cast<int64_t>(layer) * a.batch + b;   // row of the [layers*B, ...] tensors
    if (tid == 0) {
        mbar_expect_tx(bar, 2 * tile_bytes);
        for (int i = 0; i < 2; ++i)
            bulk_g2s(smem_u32(smem) + i * tile_bytes,
                     static_cast<const char*>(a.conv_cache[i]) + (seq * a.max_t + start) * kD * cs,
                     tile_bytes, bar);
    }
    const int64_t row_t = (seq * a.max_t + t) * kD + c;
    const int64_t row_1 = (seq * a.max_t + max(t - 1, 0)) * kD + c;
    const int64_t row_2 = (seq * a.max_t + max(t - 2, 0)) * kD + c;
    const float raw = load_scalar(a.raw[s], b * a.raw_stride[s] + layer * a.raw_layer_stride + c, raw_dtype);
    const float prev1 = load_scalar(a.raw_cache[s], row_1, cache_dtype);
    const float prev2 = load_scalar(a.raw_cache[s], row_2, cache_dtype);
    const int64_t wrow = (static_cast<int64_t>(layer) * kD + c) * 3;
    const float w0 = load_scalar(a.weight[s], wrow + 0, weight_dtype);
    const float w1 = load_scalar(a.weight[s], wrow + 1, weight_dtype);
    const float w2 = load_scalar(a.weight[s], wrow + 2, weight_dtype);
    const float v1 = t >= 1 ? 1.0f : 0.0f, v2 = t >= 2 ? 1.0f : 0.0f;
    float conv = __fmul_rn(raw, w2);
    conv = __fadd_rn(conv, __fmul_rn(__fmul_rn(prev1, w1), v1));
    conv = __fadd_rn(conv, __fmul_rn(__fmul_rn(prev2, w0), v2));
    store_scalar(a.raw_cache[s], row_t, cache_dtype, raw);
    store_scalar(a.conv_cache[s], row_t, cache_dtype, conv);
    if (a.out) a.out[(seq * 2 + s) * kD + c] = conv;

    bool ok = mbar_wait(bar, 0);
    if (__syncthreads_or(!ok)) {
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
        return;
    }
    const unsigned char* tile = smem + s * tile_bytes;
    const int cur = t - start;
    float sum = 0.0f;
    for (int r = 0; r < bs; ++r) {
        float x = r == cur ? conv : load_scalar(tile, r * kD + c, cache_dtype);
        sum = __fadd_rn(sum, x);
    }
    const float mean = __fdiv_rn(sum, static_cast<float>(bs));
    float acc = 0.0f;
    for (int r = 0; r < bs; ++r) {
        float x = r == cur ? conv : load_scalar(tile, r * kD + c, cache_dtype);
        float d = __fsub_rn(x, mean);
        acc = __fmaf_rn(d, d, acc);
    }
    const float sd = __fsqrt_rn(__fdiv_rn(acc, static_cast<float>(bs)));
    const int64_t stat = (seq * a.n_blocks + blk) * kD + c;
    store_scalar(a.mean[s], stat, stats_dtype, mean);
    store_scalar(a.stdv[s], stat, stats_dtype, sd);
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads) router_cache_update_kernel(const RouterArgs a) {
    const int raw_dtype = kBf16 ? RLM_BF16 : a.raw_dtype, cache_dtype = kBf16 ? RLM_BF16 : a.cache_dtype;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar_storage;
    griddep_sync();
    const int b = blockIdx.x, layer = blockIdx.y, tid = threadIdx.x;
    const int t = static_cast<int>(*a.position);
    const int blk = t / a.block_size;
    if (t < 0 || t >= a.max_t || blk >= a.n_blocks || (blk + 1) * a.block_size > a.max_t) {
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
        return;
    }
    const uint32_t bar = smem_u32(&bar_storage);
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (a.packed) {
        // token features of this layer: packed columns -> row t of the four token caches
        const int64_t seq = static_cast<int64_t>(layer) * a.batch + b;
        const int64_t src = b * a.packed_stride + static_cast<int64_t>(layer) * a.packed_width;
        int first = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int w = a.token_width[i];
            for (int c = tid; c < w; c += kThreads)
                store_scalar(a.token_cache[i], (seq * a.max_t + t) * w + c, cache_dtype,
                             load_scalar(a.packed, src + first + c, raw_dtype));
            first += w;
        }
    }
    router_update<kBf16>(a, b, layer, smem, bar, t);
}

// Prefill: conv + statistics of positions [0, length) of zero-initialised caches in one launch,
// leaving exactly the state that `length` successive single-position updates would leave.
// One CTA per (sequence, block); a thread owns one (stream, channel) and walks the block's rows
// in ascending order.  A single-position update reads earlier rows of the block back from the
// cache (rounded to the cache dtype) and uses the un-rounded value only for its own row, so
// the statistics of a block are those computed at its last filled position: rounded values
// for the rows before it, the fp32 value for that row, zeros (the fresh cache) after it.
struct PrefillArgs {
    const void* raw[2];
    int64_t raw_row_stride[2], raw_batch_stride[2];   // elements
    void* raw_cache[2];
    void* conv_cache[2];
    void* mean[2];
    void* stdv[2];
    const void* weight[2];
    int batch, max_t, n_blocks, block_size, length;
    int raw_dtype, cache_dtype, stats_dtype, weight_dtype;
};

__device__ __forceinline__ float round_to(float v, int dtype) {
    if (dtype == RLM_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    if (dtype == RLM_F16) return __half2float(__float2half_rn(v));
    return v;
}

__global__ void __launch_bounds__(kThreads) router_cache_prefill_kernel(const PrefillArgs a) {
    griddep_sync();
    const int b = blockIdx.x, blk = blockIdx.y, tid = threadIdx.x;
    const int s = tid / kD, c = tid % kD;
    const int bs = a.block_size, start = blk * bs;
    const int last = min(start + bs, a.length) - 1;        // last filled position of the block
    if (last < start) return;
    const float w0 = load_scalar(a.weight[s], c * 3 + 0, a.weight_dtype);
    const float w1 = load_scalar(a.weight[s], c * 3 + 1, a.weight_dtype);
    const float w2 = load_scalar(a.weight[s], c * 3 + 2, a.weight_dtype);
    const int64_t src = b * a.raw_batch_stride[s] + c;
    auto raw_at = [&](int p) {      // as the raw cache holds it: rounded to the cache dtype
        return round_to(load_scalar(a.raw[s], src + p * a.raw_row_stride[s], a.raw_dtype), a.cache_dtype);
    };
    auto conv_at = [&](int p, float cur, float prev1, float prev2) {
        float v = __fmul_rn(cur, w2);
        v = __fadd_rn(v, __fmul_rn(__fmul_rn(prev1, w1), p >= 1 ? 1.0f : 0.0f));
        v = __fadd_rn(v, __fmul_rn(__fmul_rn(prev2, w0), p >= 2 ? 1.0f : 0.0f));
        return v;
    };
    const int64_t cache_row0 = (static_cast<int64_t>(b) * a.max_t + start) * kD + c;
    float sum = 0.0f;
    float prev1 = start >= 1 ? raw_at(start - 1) : 0.0f, prev2 = start >= 2 ? raw_at(start - 2) : 0.0f;
    for (int p = start; p <= last; ++p) {
        // the update convolves the un-rounded incoming key with the cached (rounded) history
        const float cur = load_scalar(a.raw[s], src + p * a.raw_row_stride[s], a.raw_dtype);
        const float conv = conv_at(p, cur, prev1, prev2);
        store_scalar(a.raw_cache[s], cache_row0 + static_cast<int64_t>(p - start) * kD, a.cache_dtype, cur);
        store_scalar(a.conv_cache[s], cache_row0 + static_cast<int64_t>(p - start) * kD, a.cache_dtype, conv);
        sum = __fadd_rn(sum, p == last ? conv : round_to(conv, a.cache_dtype));
        prev2 = prev1;
        prev1 = round_to(cur, a.cache_dtype);
    }
    for (int p = last + 1; p < start + bs; ++p) sum = __fadd_rn(sum, 0.0f);
    const float mean = __fdiv_rn(sum, static_cast<float>(bs));
    float acc = 0.0f;
    prev1 = start >= 1 ? raw_at(start - 1) : 0.0f;
    prev2 = start >= 2 ? raw_at(start - 2) : 0.0f;
    for (int p = start; p < start + bs; ++p) {
        float x = 0.0f;
        if (p <= last) {
            const float cur = load_scalar(a.raw[s], src + p * a.raw_row_stride[s], a.raw_dtype);
            const float conv = conv_at(p, cur, prev1, prev2);
            x = p == last ? conv : round_to(conv, a.cache_dtype);
            prev2 = prev1;
            prev1 = round_to(cur, a.cache_dtype);
        }
        const float d = __fsub_rn(x, mean);
        acc = __fmaf_rn(d, d, acc);
    }
    const float sd = __fsqrt_rn(__fdiv_rn(acc, static_cast<float>(bs)));
    const int64_t stat = (static_cast<int64_t>(b) * a.n_blocks + blk) * kD + c;
    store_scalar(a.mean[s], stat, a.stats_dtype, mean);
    store_scalar(a.stdv[s], stat, a.stats_dtype, sd);
}

int validate_and_launch(RouterArgs& a, void* stream, const char* who) {
    if (a.batch == 0 || a.layers == 0) return RLM_OK;
    if (a.batch < 0 || a.layers < 0 || a.max_t < 1 || a.n_blocks < 1 || a.block_size < 1 ||
        static_cast<int64_t>(a.n_blocks) * a.block_size > a.max_t) {
        set_error("router update: need n_blocks * block_size <= T and positive sizes");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(a.raw_dtype) || !valid_dtype(a.cache_dtype) || !valid_dtype(a.stats_dtype) ||
        !valid_dtype(a.weight_dtype)) {
        set_error("router update: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    if (!aligned16(a.conv_cache[0]) || !aligned16(a.conv_cache[1])) {
        set_error("router update: conv caches must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    const int smem_bytes = 2 * a.block_size * kD * dtype_size(a.cache_dtype);
    if (smem_bytes > kSmemDynamicLimit) {
        set_error("router update: block tile exceeds 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    const bool bf16 = a.raw_dtype == RLM_BF16 && a.cache_dtype == RLM_BF16 && a.stats_dtype == RLM_BF16;
    auto kernel = bf16 ? router_cache_update_kernel<true> : router_cache_update_kernel<false>;
    if (smem_bytes > 48 * 1024) {
        int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
        if (rc != RLM_OK) return rc;
    }
    dim3 grid(a.batch, a.layers);
    launch_kernel(kernel, dim3(grid), dim3(kThreads), smem_bytes, stream, a);
    count_launch();
    return check_launch(who);
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_router_cache_update(
    const void* anchor_raw, int64_t anchor_raw_stride, const void* partner_raw,
    int64_t partner_raw_stride, void* anchor_raw_cache, void* partner_raw_cache,
    void* anchor_conv_cache, void* partner_conv_cache, void* anchor_mean, void* anchor_std,
    void* partner_mean, void* partner_std, const void* anchor_conv_weight,
    const void* partner_conv_weight, const int64_t* position, float* out, int batch, int max_t,
    int n_blocks, int block_size, int raw_dtype, int cache_dtype, int stats_dtype,
    int weight_dtype, int32_t* status, void* stream) {
    using namespace rlm;
    const void* need[] = {anchor_raw, partner_raw, anchor_raw_cache, partner_raw_cache,
                          anchor_conv_cache, partner_conv_cache, anchor_mean, anchor_std,
                          partner_mean, partner_std, anchor_conv_weight, partner_conv_weight,
                          position, out};
    for (const void* q : need)
        if (!q) { set_error("router_cache_update: NULL pointer"); return RLM_ERR_NULL; }
    RouterArgs a{};
    a.raw[0] = anchor_raw; a.raw[1] = partner_raw;
    a.raw_stride[0] = anchor_raw_stride; a.raw_stride[1] = partner_raw_stride;
    a.raw_cache[0] = anchor_raw_cache; a.raw_cache[1] = partner_raw_cache;
    a.conv_cache[0] = anchor_conv_cache; a.conv_cache[1] = partner_conv_cache;
    a.mean[0] = anchor_mean; a.mean[1] = partner_mean;
    a.stdv[0] = anchor_std; a.stdv[1] = partner_std;
    a.weight[0] = anchor_conv_weight; a.weight[1] = partner_conv_weight;
    a.position = position; a.out = out; a.status = status;
    a.batch = batch; a.max_t = max_t; a.n_blocks = n_blocks; a.block_size = block_size; a.layers = 1;
    a.raw_dtype = raw_dtype; a.cache_dtype = cache_dtype; a.stats_dtype = stats_dtype;
    a.weight_dtype = weight_dtype;
    return validate_and_launch(a, stream, "router_cache_update_kernel");
}

extern "C" int rlm_sparse_cache_append(
    const void* packed, int64_t packed_row_stride, int relation_dim, void* anchor_keys,
    void* partner_keys, void* operand_cache, void* partner_anchor_cache, void* anchor_raw_cache,
    void* partner_raw_cache, void* anchor_conv_cache, void* partner_conv_cache, void* anchor_mean,
    void* anchor_std, void* partner_mean, void* partner_std, const void* anchor_conv_weight,
    const void* partner_conv_weight, const int64_t* position, float* out, int layers, int batch,
    int max_t, int n_blocks, int block_size, int packed_dtype, int cache_dtype, int stats_dtype,
    int weight_dtype, int32_t* status, void* stream) {
    using namespace rlm;
    const void* need[] = {packed, anchor_keys, partner_keys, operand_cache, partner_anchor_cache,
                          anchor_raw_cache, partner_raw_cache, anchor_conv_cache, partner_conv_cache,
                          anchor_mean, anchor_std, partner_mean, partner_std, anchor_conv_weight,
                          partner_conv_weight, position};
    for (const void* q : need)
        if (!q) { set_error("sparse_cache_append: NULL pointer"); return RLM_ERR_NULL; }
    if (relation_dim < 1) { set_error("sparse_cache_append: relation_dim must be positive"); return RLM_ERR_SHAPE; }
    RouterArgs a{};
    const int width = 64 + 64 + relation_dim + 128 + 64 + 64;
    const size_t es = dtype_size(valid_dtype(packed_dtype) ? packed_dtype : 0);
    a.packed = packed; a.packed_stride = packed_row_stride; a.packed_width = width;
    a.token_cache[0] = anchor_keys; a.token_cache[1] = partner_keys;
    a.token_cache[2] = operand_cache; a.token_cache[3] = partner_anchor_cache;
    a.token_width[0] = 64; a.token_width[1] = 64; a.token_width[2] = relation_dim; a.token_width[3] = 128;
    a.raw[0] = static_cast<const char*>(packed) + (256 + relation_dim) * es;
    a.raw[1] = static_cast<const char*>(packed) + (320 + relation_dim) * es;
    a.raw_stride[0] = a.raw_stride[1] = packed_row_stride;
    a.raw_layer_stride = width;
    a.raw_cache[0] = anchor_raw_cache; a.raw_cache[1] = partner_raw_cache;
    a.conv_cache[0] = anchor_conv_cache; a.conv_cache[1] = partner_conv_cache;
    a.mean[0] = anchor_mean; a.mean[1] = partner_mean;
    a.stdv[0] = anchor_std; a.stdv[1] = partner_std;
    a.weight[0] = anchor_conv_weight; a.weight[1] = partner_conv_weight;
    a.position = position; a.out = out; a.status = status;
    a.batch = batch; a.max_t = max_t; a.n_blocks = n_blocks; a.block_size = block_size; a.layers = layers;
    a.raw_dtype = packed_dtype; a.cache_dtype = cache_dtype; a.stats_dtype = stats_dtype;
    a.weight_dtype = weight_dtype;
    return validate_and_launch(a, stream, "sparse_cache_append");
}

extern "C" int rlm_router_cache_prefill(
    const void* anchor_raw, int64_t anchor_row_stride, int64_t anchor_batch_stride,
    const void* partner_raw, int64_t partner_row_stride, int64_t partner_batch_stride,
    void* anchor_raw_cache, void* partner_raw_cache, void* anchor_conv_cache,
    void* partner_conv_cache, void* anchor_mean, void* anchor_std, void* partner_mean,
    void* partner_std, const void* anchor_conv_weight, const void* partner_conv_weight, int length,
    int batch, int max_t, int n_blocks, int block_size, int raw_dtype, int cache_dtype,
    int stats_dtype, int weight_dtype, void* stream) {
    using namespace rlm;
    if (batch == 0 || length == 0) return RLM_OK;
    const void* need[] = {anchor_raw, partner_raw, anchor_raw_cache, partner_raw_cache,
                          anchor_conv_cache, partner_conv_cache, anchor_mean, anchor_std,
                          partner_mean, partner_std, anchor_conv_weight, partner_conv_weight};
    for (const void* q : need)
        if (!q) { set_error("router_cache_prefill: NULL pointer"); return RLM_ERR_NULL; }
    if (batch < 0 || length < 0 || length > max_t || n_blocks < 1 || block_size < 1 ||
        static_cast<int64_t>(n_blocks) * block_size > max_t ||
        (length + block_size - 1) / block_size > n_blocks) {
        set_error("router_cache_prefill: need length <= T and n_blocks * block_size <= T covering it");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(raw_dtype) || !valid_dtype(cache_dtype) || !valid_dtype(stats_dtype) ||
        !valid_dtype(weight_dtype)) {
        set_error("router_cache_prefill: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    PrefillArgs a{};
    a.raw[0] = anchor_raw; a.raw[1] = partner_raw;
    a.raw_row_stride[0] = anchor_row_stride; a.raw_row_stride[1] = partner_row_stride;
    a.raw_batch_stride[0] = anchor_batch_stride; a.raw_batch_stride[1] = partner_batch_stride;
    a.raw_cache[0] = anchor_raw_cache; a.raw_cache[1] = partner_raw_cache;
    a.conv_cache[0] = anchor_conv_cache; a.conv_cache[1] = partner_conv_cache;
    a.mean[0] = anchor_mean; a.mean[1] = partner_mean;
    a.stdv[0] = anchor_std; a.stdv[1] = partner_std;
    a.weight[0] = anchor_conv_weight; a.weight[1] = partner_conv_weight;
    a.batch = batch; a.max_t = max_t; a.n_blocks = n_blocks; a.block_size = block_size; a.length = length;
    a.raw_dtype = raw_dtype; a.cache_dtype = cache_dtype; a.stats_dtype = stats_dtype; a.weight_dtype = weight_dtype;
    dim3 grid(batch, (length + block_size - 1) / block_size);
    launch_kernel(router_cache_prefill_kernel, dim3(grid), dim3(kThreads), 0, stream, a);
    count_launch();
    return check_launch("router_cache_prefill_kernel");
}
