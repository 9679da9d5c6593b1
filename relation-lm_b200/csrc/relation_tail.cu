// Fused relation tail for decode batches (sm_100a): second relation-MLP layer on the tensor
// cores + per-partner LayerNorm + active-K softmax + weighted sum + residual update, one launch.
//
//   raw[b, k, :]  = hidden[b, k, :] . W2^T + b2                       (split-K tcgen05 GEMM)
//   context[b, :] = sum_k softmax_k(score) * LayerNorm(raw[b, k, :])  (relation_norm_reduce)
//   residual[b, :] += mix * context[b, :]
//
// Grid = (d / 64 column tiles, K-splits of H, 128-row tiles).  Every CTA multiplies its
// slice (TMA ring -> tcgen05.mma -> TMEM), adds the fp32 partial tile into a SCRATCH
// accumulator in global memory with vector atomics, and bumps an arrival counter.  The CTA
// that arrives last for a row tile owns the finished sums: it applies bias, LayerNorm,
// softmax and the weighted sum, one warp per sequence, then zeroes the scratch rows and the
// counter again, so the scratch is clean for the next launch.
//
// Semantics of the reduction follow src/relation_lm/kernels/relation_reduce.py:360-417 of the
// reference project; the GEMM replaces the F.linear its callers run between the two
// operators (benchmarks/benchmark_relation_reduce.py:63).

#include <mutex>

#include "rlm_tcgen05.cuh"

namespace rlm {
namespace {

constexpr int kTailThreads = 256;
constexpr int kTailBN = 64;
constexpr int kTailStages = 8;
constexpr int kTailMaxK = 32;          // partner slots per sequence
constexpr int kTailMaxVec = 8;         // float4 per lane per row: d <= 1024

struct TailArgs {
    const void* bias2;
    const float* scores;
    const float* norm_w;
    const float* norm_b;
    const int64_t* position;
    float* residual;        // [B, d] fp32 or NULL
    const float* mix;
    float* context;         // [B, d] fp32 or NULL
    float* scratch;         // [row tiles * 128, d] fp32, all zero between launches
    int* counters;          // [row tiles], zero between launches
    int32_t* status;
    float eps;
    int rows, batch, k_out, d, h;
    int k_blocks_per_split;
    int w_dtype;
    uint32_t idesc;
    uint32_t a_bytes;
};

__global__ void __launch_bounds__(kTailThreads, 1) relation_tail_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
    const TailArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * kTailStages + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    __shared__ int is_last;
    griddep_sync();

    constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = kTailBN * kBK * 2;
    unsigned char* ring = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t ring_addr = smem_u32(ring);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kTailBN, m0 = blockIdx.z * kBM;
    const int total_blocks = (a.h + kBK - 1) / kBK;
    const int kb_lo = blockIdx.y * a.k_blocks_per_split;
    const int k_iters = max(0, min(a.k_blocks_per_split, total_blocks - kb_lo));
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kTailStages + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * kTailStages);

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int i = 0; i < 2 * kTailStages + 1; ++i) mbar_init(bar0 + 8u * i, 1);
        fence_barrier_init();
        failed = 0;
        is_last = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTailBN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (tid == 0) {
        for (int it = 0; it < k_iters; ++it) {
            const int s = it % kTailStages;
            if (it >= kTailStages && !mbar_wait(empty(s), ((it / kTailStages) - 1) & 1)) { failed = 1; break; }
            mbar_expect_tx(full(s), a.a_bytes + kBBytes);
            tma_load_2d(ring_addr + s * (kABytes + kBBytes), &map_a, (kb_lo + it) * kBK, m0, full(s));
            tma_load_2d(ring_addr + s * (kABytes + kBBytes) + kABytes, &map_w, (kb_lo + it) * kBK, n0, full(s));
        }
    } else if (tid == 32) {
        bool ok = true;
        for (int it = 0; it < k_iters && ok; ++it) {
            const int s = it % kTailStages;
            ok = mbar_wait(full(s), (it / kTailStages) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = smem_desc_sw128(ring_addr + s * (kABytes + kBBytes));
            const uint64_t db = smem_desc_sw128(ring_addr + s * (kABytes + kBBytes) + kABytes);
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk)
                umma_f16(tmem_base, da + 2 * kk, db + 2 * kk, a.idesc, (it > 0 || kk > 0) ? 1u : 0u);
            umma_commit(empty(s));
        }
        if (!ok) failed = 1;
        umma_commit(acc_full);
    }
    __syncwarp();

    bool ready = mbar_wait(acc_full, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ready = ready && (*reinterpret_cast<volatile int*>(&failed) == 0);
    const bool good = !__syncthreads_or(!ready);
    if (good && warp < 4 && k_iters > 0) {
        // partial tile -> scratch accumulator (vector atomics; rows that do not exist are skipped)
        const int row = m0 + warp * 32 + lane;
        if (m0 + warp * 32 < a.rows) {
#pragma unroll
            for (int c = 0; c < kTailBN; c += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < a.rows) {
                    float4* dst = reinterpret_cast<float4*>(a.scratch + static_cast<size_t>(row) * a.d + n0 + c);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        atomicAdd(dst + i, make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                       __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3])));
                }
            }
        }
    } else if (!good && tid == 0 && a.status) {
        atomicOr(a.status, RLM_DEV_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __threadfence();
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(kTailBN) : "memory");
    if (tid == 0) {
        const int arrivals = gridDim.x * gridDim.y;
        const int before = atomicAdd(a.counters + blockIdx.z, 1);
        is_last = before == arrivals - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();

    // ---- the last CTA of this row tile: bias + LayerNorm + softmax + weighted sum + residual
    const int K = a.k_out, D = a.d;
    const int t = static_cast<int>(*a.position);
    int k_limit = 32 - __clz(max(t, 0) + 1);   // ceil(log2(t + 2))
    k_limit = min(max(k_limit, 1), K);
    const int vecs = D / 4;
    const int seq_lo = m0 / K, seq_hi = min(a.batch, (m0 + kBM) / K);
    // per-lane slices of bias and affine parameters, loaded once
    float4 bias[kTailMaxVec], gam[kTailMaxVec], bet[kTailMaxVec];
#pragma unroll
    for (int i = 0; i < kTailMaxVec; ++i) {
        const int c4 = lane + 32 * i;
        bias[i] = gam[i] = bet[i] = make_float4(0, 0, 0, 0);
        if (c4 < vecs) {
            bias[i] = make_float4(load_scalar(a.bias2, 4 * c4, a.w_dtype), load_scalar(a.bias2, 4 * c4 + 1, a.w_dtype),
                                  load_scalar(a.bias2, 4 * c4 + 2, a.w_dtype), load_scalar(a.bias2, 4 * c4 + 3, a.w_dtype));
            gam[i] = *reinterpret_cast<const float4*>(a.norm_w + 4 * c4);
            bet[i] = *reinterpret_cast<const float4*>(a.norm_b + 4 * c4);
        }
    }
    for (int b = seq_lo + warp; b < seq_hi; b += kTailThreads / 32) {      // one warp per sequence
        float s = lane < K ? a.scores[static_cast<size_t>(b) * K + lane] : kNegInf;
        const bool active = lane < K && lane < k_limit && s > -1.0e30f;
        float safe = active ? s : -1.0e4f;
        float mx = safe;
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
        const float e = active ? expf(safe - mx) : 0.0f;
        const float wgt = e / fmaxf(warp_sum(e), 1.0e-9f);
        float4 ctx[kTailMaxVec];
#pragma unroll
        for (int i = 0; i < kTailMaxVec; ++i) ctx[i] = make_float4(0, 0, 0, 0);
        for (int k = 0; k < K; ++k) {
            const float wk = __shfl_sync(0xffffffffu, wgt, k);
            float4* src = reinterpret_cast<float4*>(a.scratch + (static_cast<size_t>(b) * K + k) * D);
            float4 x[kTailMaxVec];
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < kTailMaxVec; ++i) {
                const int c4 = lane + 32 * i;
                x[i] = make_float4(0, 0, 0, 0);
                if (c4 < vecs) {
                    x[i] = __ldcg(src + c4);
                    src[c4] = make_float4(0, 0, 0, 0);      // leave the scratch clean
                    x[i].x += bias[i].x; x[i].y += bias[i].y; x[i].z += bias[i].z; x[i].w += bias[i].w;
                    sum += (x[i].x + x[i].y) + (x[i].z + x[i].w);
                }
            }
            if (wk == 0.0f) continue;          // inactive slot
            const float mean = warp_sum(sum) / static_cast<float>(D);
            float sq = 0.0f;
#pragma unroll
            for (int i = 0; i < kTailMaxVec; ++i) {
                if (lane + 32 * i < vecs) {
                    x[i].x -= mean; x[i].y -= mean; x[i].z -= mean; x[i].w -= mean;
                    sq = fmaf(x[i].x, x[i].x, sq); sq = fmaf(x[i].y, x[i].y, sq);
                    sq = fmaf(x[i].z, x[i].z, sq); sq = fmaf(x[i].w, x[i].w, sq);
                }
            }
            const float c = wk * rsqrtf(warp_sum(sq) / static_cast<float>(D) + a.eps);
#pragma unroll
            for (int i = 0; i < kTailMaxVec; ++i) {
                if (lane + 32 * i < vecs) {
                    ctx[i].x = fmaf(c * x[i].x, gam[i].x, fmaf(wk, bet[i].x, ctx[i].x));
                    ctx[i].y = fmaf(c * x[i].y, gam[i].y, fmaf(wk, bet[i].y, ctx[i].y));
                    ctx[i].z = fmaf(c * x[i].z, gam[i].z, fmaf(wk, bet[i].z, ctx[i].z));
                    ctx[i].w = fmaf(c * x[i].w, gam[i].w, fmaf(wk, bet[i].w, ctx[i].w));
                }
            }
        }
        const float mix = a.residual ? *a.mix : 0.0f;
#pragma unroll
        for (int i = 0; i < kTailMaxVec; ++i) {
            const int c4 = lane + 32 * i;
            if (c4 < vecs) {
                if (a.context) reinterpret_cast<float4*>(a.context + static_cast<size_t>(b) * D)[c4] = ctx[i];
                if (a.residual) {
                    float4* r = reinterpret_cast<float4*>(a.residual + static_cast<size_t>(b) * D) + c4;
                    float4 h = *r;
                    h.x = fmaf(mix, ctx[i].x, h.x); h.y = fmaf(mix, ctx[i].y, h.y);
                    h.z = fmaf(mix, ctx[i].z, h.z); h.w = fmaf(mix, ctx[i].w, h.w);
                    *r = h;
                }
            }
        }
    }
    if (tid == 0) a.counters[blockIdx.z] = 0;
}

// Everything that can be wrong with the sizes, dtypes and alignment of a call, checked before
// any work is put on the stream (`a.scratch` may still be unset: it is checked when given).
int validate_relation_tail(const void* hidden, const void* w2, const TailArgs& a, int hidden_dtype) {
    if (a.batch < 0 || a.k_out < 1 || a.k_out > kTailMaxK || kBM % a.k_out != 0 || a.d < 64 ||
        a.d % 64 != 0 || a.d > 128 * kTailMaxVec || a.h < 64 || a.h % 8 != 0) {
        set_error("relation_tail: need K dividing 128 (K <= 32), d a multiple of 64 up to 1024, H a multiple of 8");
        return RLM_ERR_SHAPE;
    }
    if ((hidden_dtype != RLM_BF16 && hidden_dtype != RLM_F16) || a.w_dtype != hidden_dtype) {
        set_error("relation_tail: hidden states and weights must share bfloat16 or float16");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(hidden) || !aligned16(w2) || !aligned16(a.scratch) || !aligned16(a.norm_w) ||
        !aligned16(a.norm_b) || (a.residual && !aligned16(a.residual)) || (a.context && !aligned16(a.context))) {
        set_error("relation_tail: tensors must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    return RLM_OK;
}

// Host-side validation, tiling and launch.
int launch_relation_tail(const void* hidden, const void* w2, TailArgs& a, int hidden_dtype,
                         void* stream) {
    if (a.batch == 0) return RLM_OK;
    const int valid = validate_relation_tail(hidden, w2, a, hidden_dtype);
    if (valid != RLM_OK) return valid;
    a.rows = a.batch * a.k_out;
    const int m_tiles = (a.rows + kBM - 1) / kBM;
    const int n_tiles = a.d / kTailBN;
    const int total_blocks = (a.h + kBK - 1) / kBK;
    // enough K-splits for about one CTA per SM, at most eight ring stages' worth of work each
    int splits = (sm_count() + n_tiles * m_tiles - 1) / (n_tiles * m_tiles);
    if (splits > total_blocks) splits = total_blocks;
    if (splits < 1) splits = 1;
    a.k_blocks_per_split = (total_blocks + splits - 1) / splits;
    splits = (total_blocks + a.k_blocks_per_split - 1) / a.k_blocks_per_split;
    const int box_rows = a.rows >= kBM ? kBM : ((a.rows + 7) / 8) * 8;
    CUtensorMap ma, mw;
    if (!make_map(&ma, hidden, a.rows, a.h, a.h, box_rows, hidden_dtype) ||
        !make_map(&mw, w2, a.d, a.h, a.h, kTailBN, hidden_dtype)) {
        set_error("relation_tail: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    const uint32_t fmt = hidden_dtype == RLM_BF16 ? 1u : 0u;
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kTailBN >> 3) << 17) |
              (static_cast<uint32_t>(kBM >> 4) << 24);
    a.a_bytes = static_cast<uint32_t>(box_rows) * kBK * 2;
    const int smem_bytes = kTailStages * (kBM * kBK * 2 + kTailBN * kBK * 2) + 1024;
    int rc = allow_large_smem(reinterpret_cast<const void*>(relation_tail_kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    dim3 grid(n_tiles, splits, m_tiles);
    launch_kernel(relation_tail_kernel, dim3(grid), dim3(kTailThreads), smem_bytes, stream, ma, mw, a);
    count_launch();
    return check_launch("relation_tail_kernel");
}

// ------------------------------------------------------------------ built-in scratch
//
// Scratch for callers that may not allocate device memory themselves.  It is part of the
// library image, so every GPU that loads the library carries these bytes until the process
// exits.  Limits: one 128-row tile (batch * k_out <= 128) and d_model <= 1024.
constexpr int kStaticRows = kBM;
constexpr int kStaticDim = 1024;
constexpr size_t kStaticAccBytes = static_cast<size_t>(kStaticRows) * kStaticDim * sizeof(float);
constexpr size_t kStaticScratchBytes = kStaticAccBytes + 256;        // + the arrival counter

static __device__ __align__(256) unsigned char g_tail_scratch[kStaticScratchBytes];

// Device address of g_tail_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use; the address is asked for
// once per device (with that device current) and remembered.
int static_scratch_address(void** out) {
    static std::mutex guard;
    static void* address[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
        cudaGetLastError();
        set_error("relation_tail_static: cannot identify the current device");
        return RLM_ERR_LAUNCH;
    }
    std::lock_guard<std::mutex> lock(guard);
    if (!address[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_tail_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            set_error(e != cudaSuccess ? cudaGetErrorString(e) : "relation_tail_static: no address for the built-in scratch");
            return RLM_ERR_LAUNCH;
        }
        address[device] = p;
    }
    *out = address[device];
    return RLM_OK;
}

}  // namespace
}  // namespace rlm

extern "C" int64_t rlm_relation_tail_scratch_bytes(int batch, int k_out, int d_model) {
    if (batch < 0 || k_out < 1 || d_model < 1) return -1;
    const int64_t rows = static_cast<int64_t>(batch) * k_out;
    const int64_t tiles = (rows + rlm::kBM - 1) / rlm::kBM;
    // accumulator rows (padded to whole tiles) + one arrival counter per tile, 256-byte granules
    return ((tiles * rlm::kBM * d_model * 4 + 255) / 256) * 256 + ((tiles * 4 + 255) / 256) * 256;
}

extern "C" int rlm_relation_tail(const void* relation_hidden, const void* second_weight,
                                 const void* second_bias, const float* partner_scores,
                                 const float* norm_weight, const float* norm_bias,
                                 const int64_t* position, float norm_eps, float* residual,
                                 const float* mix, float* context, void* scratch,
                                 int64_t scratch_bytes, int batch, int k_out, int d_model,
                                 int hidden_dim, int dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (batch == 0) return RLM_OK;
    if (!relation_hidden || !second_weight || !second_bias || !partner_scores || !norm_weight ||
        !norm_bias || !position || !scratch || (!residual && !context) || (residual && !mix)) {
        set_error("relation_tail: NULL pointer");
        return RLM_ERR_NULL;
    }
    const int64_t need = rlm_relation_tail_scratch_bytes(batch, k_out, d_model);
    if (need < 0 || scratch_bytes < need) {
        set_error("relation_tail: scratch buffer smaller than rlm_relation_tail_scratch_bytes()");
        return RLM_ERR_SHAPE;
    }
    TailArgs a{};
    a.bias2 = second_bias; a.scores = partner_scores; a.norm_w = norm_weight; a.norm_b = norm_bias;
    a.position = position; a.residual = residual; a.mix = mix; a.context = context;
    a.scratch = static_cast<float*>(scratch);
    const int64_t rows = static_cast<int64_t>(batch) * k_out;
    const int64_t tiles = (rows + kBM - 1) / kBM;
    a.counters = reinterpret_cast<int*>(static_cast<char*>(scratch) +
                                        ((tiles * kBM * d_model * 4 + 255) / 256) * 256);
    a.status = status; a.eps = norm_eps; a.batch = batch; a.k_out = k_out; a.d = d_model; a.h = hidden_dim;
    a.w_dtype = dtype;
    return launch_relation_tail(relation_hidden, second_weight, a, dtype, stream);
}


// The fused relation tail for callers that cannot provide scratch memory: identical
// arithmetic to rlm_relation_tail, with the split-K accumulator in the library's built-in
// device array instead of a caller buffer.  Nothing is allocated, here or in anything this
// function calls.
extern "C" int rlm_relation_tail_static(const void* relation_hidden, const void* second_weight,
                                        const void* second_bias, const float* partner_scores,
                                        const float* norm_weight, const float* norm_bias,
                                        const int64_t* position, float norm_eps, float* residual,
                                        const float* mix, float* context, int batch, int k_out,
                                        int d_model, int hidden_dim, int dtype, int32_t* status,
                                        void* stream) {
    using namespace rlm;
    if (batch == 0) return RLM_OK;
    if (!relation_hidden || !second_weight || !second_bias || !partner_scores || !norm_weight ||
        !norm_bias || !position || (!residual && !context) || (residual && !mix)) {
        set_error("relation_tail_static: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (batch < 0 || k_out < 1 || static_cast<int64_t>(batch) * k_out > kStaticRows || d_model > kStaticDim) {
        set_error("relation_tail_static: the built-in scratch holds batch * k_out <= 128 rows of d_model <= 1024; "
                  "use rlm_relation_tail with a caller buffer for larger problems");
        return RLM_ERR_SHAPE;
    }
    TailArgs a{};
    a.bias2 = second_bias; a.scores = partner_scores; a.norm_w = norm_weight; a.norm_b = norm_bias;
    a.position = position; a.residual = residual; a.mix = mix; a.context = context;
    a.status = status; a.eps = norm_eps; a.batch = batch; a.k_out = k_out; a.d = d_model; a.h = hidden_dim;
    a.w_dtype = dtype;
    // sizes, dtypes and alignment are settled before anything is put on the stream
    int rc = validate_relation_tail(relation_hidden, second_weight, a, dtype);
    if (rc != RLM_OK) return rc;
    void* scratch = nullptr;
    rc = static_scratch_address(&scratch);
    if (rc != RLM_OK) return rc;
    // The array keeps whatever the previous call left.  A completed call leaves zeros, but a call
    // that was cut short would not, so the part this call uses is cleared on the stream first.
    const size_t acc_bytes = static_cast<size_t>(kStaticRows) * d_model * sizeof(float);
    if (cudaMemsetAsync(scratch, 0, acc_bytes, static_cast<cudaStream_t>(stream)) != cudaSuccess ||
        cudaMemsetAsync(static_cast<char*>(scratch) + kStaticAccBytes, 0, 256, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        cudaGetLastError();
        set_error("relation_tail_static: clearing the built-in scratch failed");
        return RLM_ERR_LAUNCH;
    }
    a.scratch = static_cast<float*>(scratch);
    a.counters = reinterpret_cast<int*>(static_cast<char*>(scratch) + kStaticAccBytes);
    return launch_relation_tail(relation_hidden, second_weight, a, dtype, stream);
}
