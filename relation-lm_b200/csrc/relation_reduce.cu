// Relation-reduce tail for sm_100a: factorised first relation-MLP layer over
// gathered anchor/partner rows (with or without the current-row cache update),
// and the per-partner LayerNorm + active-K softmax + weighted sum.
//
// Semantics follow src/relation_lm/kernels/relation_reduce.py:72-146, 186-309
// and 360-417 of the reference project.

#include "rlm_common.cuh"

namespace rlm {
namespace {


// ------------------------------------------------------------------ hidden

constexpr int kHT = 64;            // hidden columns per CTA
constexpr int kHiddenThreads = 128;
constexpr int kMaxK = 16;          // partner slots per row
constexpr int kPad = 4;            // row padding (floats) of staged weight tiles: conflict-free float4 reads

struct HiddenArgs {
    void* expanded_cache;
    const void* operand_cache;
    const int32_t* anchor_index;
    const int32_t* partner_index;
    const void* anchor_weight;
    const void* partner_weight;
    const void* product_weight;
    const void* first_bias;
    const int64_t* position;
    const int32_t* row_batch;
    float* out;
    int32_t* status;
    int n_rows, n_seq, max_t, rdim, hdim, k_out;
    int cache_dtype, weight_dtype;
};

__device__ __forceinline__ void stage_weight_tile(const void* weight, int dtype, int h0, int hdim,
                                                  int rdim, float* dst) {
    const int segs = rdim / 8;
    for (int i = threadIdx.x; i < kHT * segs; i += kHiddenThreads) {
        int r = i / segs, sgm = i % segs;
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (h0 + r < hdim) {
            const char* row = static_cast<const char*>(weight) +
                              static_cast<size_t>(h0 + r) * rdim * (dtype == RLM_F32 ? 4 : 2);
            load8(row, 8 * sgm, dtype, f);
        }
        float4* d = reinterpret_cast<float4*>(dst + r * (rdim + kPad) + 8 * sgm);
        d[0] = make_float4(f[0], f[1], f[2], f[3]);
        d[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

__device__ __forceinline__ float gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}

template <bool kUpdate>
__global__ void __launch_bounds__(kHiddenThreads) relation_hidden_kernel(const HiddenArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x;
    const int R = a.rdim, H = a.hdim, K = a.k_out;
    const int stride = R + kPad;
    float* wm = reinterpret_cast<float*>(smem);
    float* wa = wm + kHT * stride;                        // only when kUpdate
    float* wp = wa + (kUpdate ? kHT * stride : 0);
    float* prod = wp + (kUpdate ? kHT * stride : 0);      // [K][R]
    float* cur = prod + kMaxK * R;                        // [R] current operand (kUpdate)
    float* fresh = cur + R;                               // [2][kHT] (kUpdate)
    __shared__ int idx[kMaxK + 1];

    const int h0 = blockIdx.y * kHT;
    int t = -1;
    if (kUpdate) {
        t = static_cast<int>(*a.position);
        if (t < 0 || t >= a.max_t) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
            return;
        }
    }
    stage_weight_tile(a.product_weight, a.weight_dtype, h0, H, R, wm);
    if (kUpdate) {
        stage_weight_tile(a.anchor_weight, a.weight_dtype, h0, H, R, wa);
        stage_weight_tile(a.partner_weight, a.weight_dtype, h0, H, R, wp);
    }
    const int h = tid % kHT, g = tid / kHT;        // two thread groups split the partner slots
    const int per = (K + 1) / 2;
    const int k_lo = g * per, k_hi = min(K, k_lo + per);
    const bool h_ok = h0 + h < H;
    const int cs = a.cache_dtype == RLM_F32 ? 4 : 2;

    for (int row = blockIdx.x; row < a.n_rows; row += gridDim.x) {
        __syncthreads();   // previous row's reads of prod/idx/fresh are done; weights are staged
        const int b = a.row_batch ? a.row_batch[row] : row;
        if (b < 0 || b >= a.n_seq) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
            continue;
        }
        if (tid <= K) {
            int v = tid == 0 ? a.anchor_index[row] : a.partner_index[static_cast<size_t>(row) * K + tid - 1];
            idx[tid] = min(max(v, 0), a.max_t - 1);
        }
        __syncthreads();
        const char* operand = static_cast<const char*>(a.operand_cache) + static_cast<size_t>(b) * a.max_t * R * cs;
        for (int i = tid; i < K * R; i += kHiddenThreads) {
            int k = i / R, r = i % R;
            float oa = load_scalar(operand, static_cast<int64_t>(idx[0]) * R + r, a.cache_dtype);
            float op = load_scalar(operand, static_cast<int64_t>(idx[k + 1]) * R + r, a.cache_dtype);
            prod[k * R + r] = op * oa;
        }
        if (kUpdate)
            for (int r = tid; r < R; r += kHiddenThreads)
                cur[r] = load_scalar(operand, static_cast<int64_t>(t) * R + r, a.cache_dtype);
        __syncthreads();

        char* expanded = static_cast<char*>(a.expanded_cache) + static_cast<size_t>(b) * a.max_t * 2 * H * cs;
        if (kUpdate) {
            // group 0: anchor half (+ bias); group 1: partner half of the current expanded row
            const float* w = (g == 0 ? wa : wp) + h * stride;
            float acc = 0.0f;
            for (int r = 0; r < R; r += 4) {
                float4 wv = *reinterpret_cast<const float4*>(w + r);
                float4 ov = *reinterpret_cast<const float4*>(cur + r);
                acc = fmaf(wv.x, ov.x, acc); acc = fmaf(wv.y, ov.y, acc);
                acc = fmaf(wv.z, ov.z, acc); acc = fmaf(wv.w, ov.w, acc);
            }
            if (g == 0 && h_ok) acc += load_scalar(a.first_bias, h0 + h, a.weight_dtype);
            fresh[g * kHT + h] = acc;
            if (h_ok)
                store_scalar(expanded, static_cast<int64_t>(t) * 2 * H + g * H + h0 + h, a.cache_dtype, acc);
            __syncthreads();
        }
        float acc[(kMaxK + 1) / 2];
#pragma unroll
        for (int i = 0; i < (kMaxK + 1) / 2; ++i) acc[i] = 0.0f;
        const float* w = wm + h * stride;
        for (int r = 0; r < R; r += 4) {
            float4 wv = *reinterpret_cast<const float4*>(w + r);
#pragma unroll
            for (int i = 0; i < (kMaxK + 1) / 2; ++i) {
                if (k_lo + i < k_hi) {
                    float4 pv = *reinterpret_cast<const float4*>(prod + (k_lo + i) * R + r);
                    acc[i] = fmaf(wv.x, pv.x, acc[i]); acc[i] = fmaf(wv.y, pv.y, acc[i]);
                    acc[i] = fmaf(wv.z, pv.z, acc[i]); acc[i] = fmaf(wv.w, pv.w, acc[i]);
                }
            }
        }
        if (h_ok) {
            const int ai = idx[0];
            float base_a = (kUpdate && ai == t) ? fresh[h]
                                                 : load_scalar(expanded, static_cast<int64_t>(ai) * 2 * H + h0 + h, a.cache_dtype);
#pragma unroll
            for (int i = 0; i < (kMaxK + 1) / 2; ++i) {
                int k = k_lo + i;
                if (k < k_hi) {
                    const int pi = idx[k + 1];
                    float base_p = (kUpdate && pi == t) ? fresh[kHT + h]
                                                         : load_scalar(expanded, static_cast<int64_t>(pi) * 2 * H + H + h0 + h, a.cache_dtype);
                    float x = acc[i] + (base_a + base_p);
                    a.out[(static_cast<size_t>(row) * K + k) * H + h0 + h] = gelu_erf(x);
                }
            }
        }
    }
}

int hidden_smem_bytes(bool update, int rdim) {
    int tiles = update ? 3 : 1;
    return (tiles * kHT * (rdim + kPad) + kMaxK * rdim + rdim + 2 * kHT) * 4;
}

int launch_hidden(HiddenArgs& a, bool update, void* stream) {
    if (a.n_rows == 0) return RLM_OK;
    if (!a.expanded_cache || !a.operand_cache || !a.anchor_index || !a.partner_index ||
        !a.product_weight || !a.out ||
        (update && (!a.anchor_weight || !a.partner_weight || !a.first_bias || !a.position))) {
        set_error("relation_hidden: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (a.n_rows < 0 || a.n_seq < 1 || a.max_t < 1 || a.rdim < 8 || a.rdim % 8 != 0 || a.hdim < 1 ||
        a.k_out < 1 || a.k_out > kMaxK) {
        set_error("relation_hidden: need relation_dim a multiple of 8, 1 <= K <= 16 and positive sizes");
        return RLM_ERR_SHAPE;
    }
    if (!a.row_batch && a.n_rows != a.n_seq) {
        set_error("relation_hidden: without row_batch the rows must equal the sequences");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(a.cache_dtype) || !valid_dtype(a.weight_dtype)) {
        set_error("relation_hidden: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    if (!aligned16(a.product_weight) || (update && (!aligned16(a.anchor_weight) || !aligned16(a.partner_weight)))) {
        set_error("relation_hidden: weight matrices must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    int smem_bytes = hidden_smem_bytes(update, a.rdim);
    if (smem_bytes > kSmemDynamicLimit) {
        set_error("relation_hidden: relation_dim too large for the staged weight tiles");
        return RLM_ERR_SMEM;
    }
    const void* fn = update ? reinterpret_cast<const void*>(relation_hidden_kernel<true>)
                            : reinterpret_cast<const void*>(relation_hidden_kernel<false>);
    if (smem_bytes > 48 * 1024) {
        int rc = allow_large_smem(fn, kSmemPerCta);
        if (rc != RLM_OK) return rc;
    }
    int tiles = (a.hdim + kHT - 1) / kHT;
    // enough CTAs to fill the machine a few times over; more rows per CTA amortise the weight tile
    int want = (148 * 4 + tiles - 1) / tiles;
    int gx = a.n_rows < want ? a.n_rows : want;
    dim3 grid(gx, tiles);
    if (update)
        relation_hidden_kernel<true><<<grid, kHiddenThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(a);
    else
        relation_hidden_kernel<false><<<grid, kHiddenThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(a);
    count_launch();
    return check_launch("relation_hidden_kernel");
}

// ------------------------------------------------------------------ norm + reduce

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kMaxPerLane = 32;    // feature columns per lane: dim <= 1024
constexpr int kNormMaxK = 64;

struct NormArgs {
    const void* raw;
    const float* scores;
    const void* weight;
    const void* bias;
    const int64_t* position;
    const int32_t* row_position;
    float* out;
    int32_t* status;
    float eps;
    int n_rows, k_out, dim, raw_dtype, param_dtype;
};

__global__ void __launch_bounds__(kNormThreads) relation_norm_reduce_kernel(const NormArgs a) {
    extern __shared__ __align__(16) float partial[];   // [warps][dim]
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = a.k_out, D = a.dim;
    const int t = a.row_position ? a.row_position[row] : static_cast<int>(*a.position);
    int k_limit = 32 - __clz(max(t, 0) + 1);   // ceil(log2(t + 2))
    k_limit = min(max(k_limit, 1), K);

    // softmax weights over the active slots (every warp computes them redundantly)
    float s0 = lane < K ? a.scores[static_cast<size_t>(row) * K + lane] : kNegInf;
    float s1 = lane + 32 < K ? a.scores[static_cast<size_t>(row) * K + lane + 32] : kNegInf;
    bool a0 = lane < K && lane < k_limit && s0 > -1.0e30f;
    bool a1 = lane + 32 < K && lane + 32 < k_limit && s1 > -1.0e30f;
    float f0 = a0 ? s0 : -1.0e4f, f1 = a1 ? s1 : -1.0e4f;
    float mx = fmaxf(f0, f1);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float e0 = a0 ? expf(f0 - mx) : 0.0f, e1 = a1 ? expf(f1 - mx) : 0.0f;
    float den = fmaxf(warp_sum(e0 + e1), 1.0e-9f);
    float w0 = e0 / den, w1 = e1 / den;

    const int per = (D + 31) / 32;
    float y[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) y[i] = 0.0f;
    for (int k = warp; k < K; k += kNormWarps) {
        float wk = __shfl_sync(0xffffffffu, k < 32 ? w0 : w1, k & 31);
        if (wk == 0.0f) continue;   // inactive slot: contributes nothing, its row is not read
        const int64_t base = (static_cast<int64_t>(row) * K + k) * D;
        float x[kMaxPerLane];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            int c = lane + 32 * i;
            x[i] = (i < per && c < D) ? load_scalar(a.raw, base + c, a.raw_dtype) : 0.0f;
            sum += x[i];
        }
        const float mean = warp_sum(sum) / static_cast<float>(D);
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            int c = lane + 32 * i;
            float d = (i < per && c < D) ? x[i] - mean : 0.0f;
            x[i] = d;
            sq = fmaf(d, d, sq);
        }
        const float inv = rsqrtf(warp_sum(sq) / static_cast<float>(D) + a.eps);
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            int c = lane + 32 * i;
            if (i < per && c < D) {
                float gm = load_scalar(a.weight, c, a.param_dtype);
                float bt = load_scalar(a.bias, c, a.param_dtype);
                y[i] = fmaf(wk, fmaf(x[i] * inv, gm, bt), y[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        int c = lane + 32 * i;
        if (i < per && c < D) partial[warp * D + c] = y[i];
    }
    __syncthreads();
    for (int c = tid; c < D; c += kNormThreads) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kNormWarps; ++w) total += partial[w * D + c];
        a.out[static_cast<size_t>(row) * D + c] = total;
    }
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_relation_hidden_cached(
    const void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const void* product_weight, const int32_t* row_batch, float* out,
    int n_rows, int n_seq, int max_t, int relation_dim, int hidden_dim, int k_out, int cache_dtype,
    int weight_dtype, int32_t* status, void* stream) {
    rlm::HiddenArgs a{};
    a.expanded_cache = const_cast<void*>(expanded_cache); a.operand_cache = operand_cache;
    a.anchor_index = anchor_index; a.partner_index = partner_index; a.product_weight = product_weight;
    a.row_batch = row_batch; a.out = out; a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.rdim = relation_dim; a.hdim = hidden_dim;
    a.k_out = k_out; a.cache_dtype = cache_dtype; a.weight_dtype = weight_dtype;
    return rlm::launch_hidden(a, false, stream);
}

extern "C" int rlm_relation_hidden_cache_update(
    void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const void* anchor_weight, const void* partner_weight,
    const void* product_weight, const void* first_bias, const int64_t* position, float* out,
    int batch, int max_t, int relation_dim, int hidden_dim, int k_out, int cache_dtype,
    int weight_dtype, int32_t* status, void* stream) {
    rlm::HiddenArgs a{};
    a.expanded_cache = expanded_cache; a.operand_cache = operand_cache;
    a.anchor_index = anchor_index; a.partner_index = partner_index;
    a.anchor_weight = anchor_weight; a.partner_weight = partner_weight;
    a.product_weight = product_weight; a.first_bias = first_bias; a.position = position;
    a.out = out; a.status = status;
    a.n_rows = batch; a.n_seq = batch; a.max_t = max_t; a.rdim = relation_dim; a.hdim = hidden_dim;
    a.k_out = k_out; a.cache_dtype = cache_dtype; a.weight_dtype = weight_dtype;
    return rlm::launch_hidden(a, true, stream);
}

extern "C" int rlm_relation_norm_reduce(
    const void* raw, const float* partner_scores, const void* norm_weight, const void* norm_bias,
    const int64_t* position, const int32_t* row_position, float norm_eps, float* out, int n_rows,
    int k_out, int dim, int raw_dtype, int param_dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (n_rows == 0) return RLM_OK;
    if (!raw || !partner_scores || !norm_weight || !norm_bias || !out || (!position && !row_position)) {
        set_error("relation_norm_reduce: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (n_rows < 0 || k_out < 1 || k_out > kNormMaxK || dim < 1 || dim > 32 * kMaxPerLane) {
        set_error("relation_norm_reduce: need 1 <= K <= 64 and 1 <= dim <= 1024");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(raw_dtype) || !valid_dtype(param_dtype)) {
        set_error("relation_norm_reduce: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    NormArgs a{};
    a.raw = raw; a.scores = partner_scores; a.weight = norm_weight; a.bias = norm_bias;
    a.position = position; a.row_position = row_position; a.out = out; a.status = status;
    a.eps = norm_eps; a.n_rows = n_rows; a.k_out = k_out; a.dim = dim;
    a.raw_dtype = raw_dtype; a.param_dtype = param_dtype;
    int smem_bytes = kNormWarps * dim * 4;
    relation_norm_reduce_kernel<<<n_rows, kNormThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(a);
    count_launch();
    return check_launch("relation_norm_reduce_kernel");
}
