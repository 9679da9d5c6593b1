// Router state update for the current position (sm_100a).
//
// One CTA per sequence, one thread per (stream, channel).  The conv-cache tile
// of the current block is staged in shared memory by two bulk copies issued at
// entry; the three-tap causal convolution, the cache writes and the output are
// done while they fly; block mean and biased standard deviation are then
// accumulated from shared memory in ascending row order with the fresh
// (un-rounded) row substituted at the current position.
//
// Semantics follow src/relation_lm/kernels/router_cache.py:33-172 of the
// reference project.

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kD = 64;
constexpr int kThreads = 2 * kD;

struct RouterArgs {
    const void* raw[2];
    int64_t raw_stride[2];
    void* raw_cache[2];
    void* conv_cache[2];
    void* mean[2];
    void* stdv[2];
    const void* weight[2];
    const int64_t* position;
    float* out;
    int32_t* status;
    int batch, max_t, n_blocks, block_size;
    int raw_dtype, cache_dtype, stats_dtype, weight_dtype;
};

__global__ void __launch_bounds__(kThreads) router_cache_update_kernel(const RouterArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bar_storage;
    const int b = blockIdx.x, tid = threadIdx.x;
    const int s = tid / kD, c = tid % kD;
    const int t = static_cast<int>(*a.position);
    const int bs = a.block_size;
    const int blk = t / bs, start = blk * bs;
    if (t < 0 || t >= a.max_t || blk >= a.n_blocks || start + bs > a.max_t) {
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
        return;
    }
    const int cs = a.cache_dtype == RLM_F32 ? 4 : 2;
    const uint32_t tile_bytes = static_cast<uint32_t>(bs) * kD * cs;
    const uint32_t bar = smem_u32(&bar_storage);
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(bar, 2 * tile_bytes);
        for (int i = 0; i < 2; ++i)
            bulk_g2s(smem_u32(smem) + i * tile_bytes,
                     static_cast<const char*>(a.conv_cache[i]) + (static_cast<size_t>(b) * a.max_t + start) * kD * cs,
                     tile_bytes, bar);
    }
    const int64_t row_t = (static_cast<int64_t>(b) * a.max_t + t) * kD + c;
    const int64_t row_1 = (static_cast<int64_t>(b) * a.max_t + max(t - 1, 0)) * kD + c;
    const int64_t row_2 = (static_cast<int64_t>(b) * a.max_t + max(t - 2, 0)) * kD + c;
    const float raw = load_scalar(a.raw[s], b * a.raw_stride[s] + c, a.raw_dtype);
    const float prev1 = load_scalar(a.raw_cache[s], row_1, a.cache_dtype);
    const float prev2 = load_scalar(a.raw_cache[s], row_2, a.cache_dtype);
    const float w0 = load_scalar(a.weight[s], c * 3 + 0, a.weight_dtype);
    const float w1 = load_scalar(a.weight[s], c * 3 + 1, a.weight_dtype);
    const float w2 = load_scalar(a.weight[s], c * 3 + 2, a.weight_dtype);
    const float v1 = t >= 1 ? 1.0f : 0.0f, v2 = t >= 2 ? 1.0f : 0.0f;
    float conv = __fmul_rn(raw, w2);
    conv = __fadd_rn(conv, __fmul_rn(__fmul_rn(prev1, w1), v1));
    conv = __fadd_rn(conv, __fmul_rn(__fmul_rn(prev2, w0), v2));
    store_scalar(a.raw_cache[s], row_t, a.cache_dtype, raw);
    store_scalar(a.conv_cache[s], row_t, a.cache_dtype, conv);
    a.out[(static_cast<int64_t>(b) * 2 + s) * kD + c] = conv;

    bool ok = mbar_wait(bar, 0);
    if (__syncthreads_or(!ok)) {
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
        return;
    }
    const unsigned char* tile = smem + s * tile_bytes;
    const int cur = t - start;
    float sum = 0.0f;
    for (int r = 0; r < bs; ++r) {
        float x = r == cur ? conv : load_scalar(tile, r * kD + c, a.cache_dtype);
        sum = __fadd_rn(sum, x);
    }
    const float mean = __fdiv_rn(sum, static_cast<float>(bs));
    float acc = 0.0f;
    for (int r = 0; r < bs; ++r) {
        float x = r == cur ? conv : load_scalar(tile, r * kD + c, a.cache_dtype);
        float d = __fsub_rn(x, mean);
        acc = __fmaf_rn(d, d, acc);
    }
    const float sd = __fsqrt_rn(__fdiv_rn(acc, static_cast<float>(bs)));
    const int64_t stat = (static_cast<int64_t>(b) * a.n_blocks + blk) * kD + c;
    store_scalar(a.mean[s], stat, a.stats_dtype, mean);
    store_scalar(a.stdv[s], stat, a.stats_dtype, sd);
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
    if (batch == 0) return RLM_OK;
    const void* need[] = {anchor_raw, partner_raw, anchor_raw_cache, partner_raw_cache,
                          anchor_conv_cache, partner_conv_cache, anchor_mean, anchor_std,
                          partner_mean, partner_std, anchor_conv_weight, partner_conv_weight,
                          position, out};
    for (const void* q : need)
        if (!q) { set_error("router_cache_update: NULL pointer"); return RLM_ERR_NULL; }
    if (batch < 0 || max_t < 1 || n_blocks < 1 || block_size < 1 ||
        static_cast<int64_t>(n_blocks) * block_size > max_t) {
        set_error("router_cache_update: need n_blocks * block_size <= T and positive sizes");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(raw_dtype) || !valid_dtype(cache_dtype) || !valid_dtype(stats_dtype) ||
        !valid_dtype(weight_dtype)) {
        set_error("router_cache_update: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    if (!aligned16(anchor_conv_cache) || !aligned16(partner_conv_cache)) {
        set_error("router_cache_update: conv caches must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    const int smem_bytes = 2 * block_size * kD * dtype_size(cache_dtype);
    if (smem_bytes > kSmemDynamicLimit) {
        set_error("router_cache_update: block tile exceeds 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    if (smem_bytes > 48 * 1024) {
        int rc = allow_large_smem(reinterpret_cast<const void*>(router_cache_update_kernel), kSmemPerCta);
        if (rc != RLM_OK) return rc;
    }
    RouterArgs a{};
    a.raw[0] = anchor_raw; a.raw[1] = partner_raw;
    a.raw_stride[0] = anchor_raw_stride; a.raw_stride[1] = partner_raw_stride;
    a.raw_cache[0] = anchor_raw_cache; a.raw_cache[1] = partner_raw_cache;
    a.conv_cache[0] = anchor_conv_cache; a.conv_cache[1] = partner_conv_cache;
    a.mean[0] = anchor_mean; a.mean[1] = partner_mean;
    a.stdv[0] = anchor_std; a.stdv[1] = partner_std;
    a.weight[0] = anchor_conv_weight; a.weight[1] = partner_conv_weight;
    a.position = position; a.out = out; a.status = status;
    a.batch = batch; a.max_t = max_t; a.n_blocks = n_blocks; a.block_size = block_size;
    a.raw_dtype = raw_dtype; a.cache_dtype = cache_dtype; a.stats_dtype = stats_dtype;
    a.weight_dtype = weight_dtype;
    router_cache_update_kernel<<<batch, kThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(a);
    count_launch();
    return check_launch("router_cache_update_kernel");
}
