// Relation-reduce tail for sm_100a: factorised first relation-MLP layer over
// gathered anchor/partner rows (with or without the current-row cache update),
// and the per-partner LayerNorm + active-K softmax + weighted sum.
//
// Semantics follow src/relation_lm/kernels/relation_reduce.py:72-146, 186-309
// and 360-417 of the reference project.

#include "rlm_common.cuh"

namespace rlm {
// tensor-core form for launches with many relation rows (relation_hidden_tc.cu)
bool hidden_tc_applicable(bool update, int n_rows, int rdim, int hdim, int k_out, int cache_dtype,
                          int weight_dtype, const void* expanded_cache, const void* out);
int launch_hidden_tc(bool update, void* expanded_cache, const void* operand_cache,
                     const int32_t* anchor_index, const int32_t* partner_index,
                     const void* anchor_weight, const void* partner_weight, const void* product_weight,
                     const void* first_bias, const int64_t* position, const int32_t* row_batch, void* out,
                     int n_rows, int n_seq, int max_t, int rdim, int hdim, int k_out, int dtype,
                     int out_dtype, int32_t* status, void* stream);
namespace {


// ------------------------------------------------------------------ hidden
//
// Tile = kRB sequences (kRB*K relation rows) x kHT hidden columns per CTA pass.  The weight
// tiles of the CTA's hidden columns are staged once (fp32, padded rows); a CTA then walks
// its share of sequence groups.  Per group the gathered operand rows are multiplied into the
// product matrix in shared memory.  The 512 threads form four groups of 128 that each take a
// quarter of the relation dimension (sixteen warps per CTA hide the shared-memory latency);
// inside a group a thread accumulates an NR x 2 register tile (NR relation rows, two hidden
// columns) with float4 reads.  Partial sums meet in shared memory; the epilogue (expanded-cache
// terms, GELU, store) is spread over all threads, two adjacent hidden columns per thread.

constexpr int kHT = 32;            // hidden columns per CTA
constexpr int kRB = 4;             // sequences per tile
constexpr int kSplit = 4;          // thread groups along the relation dimension
constexpr int kGroupThreads = 128;
constexpr int kHiddenThreads = kSplit * kGroupThreads;
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
    void* out;
    int32_t* status;
    int n_rows, n_seq, max_t, rdim, hdim, k_out;
    int cache_dtype, weight_dtype, out_dtype;
};

__device__ __forceinline__ float gelu_erf(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}

__device__ __forceinline__ float dot4(const float4& a, const float4& b, float acc) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    return fmaf(a.w, b.w, acc);
}

__device__ __forceinline__ void store8(float* dst, const float (&f)[8]) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
}

// NR = relation rows per thread: the tile's kRB*K rows are dealt to 8 thread rows.
// kBf16: caches, weights and output are all bfloat16 (the decode step): dtype branches fold away.
template <bool kUpdate, int NR, bool kBf16>
__global__ void __launch_bounds__(kHiddenThreads) relation_hidden_kernel(const HiddenArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x;
    const int cache_dtype = kBf16 ? RLM_BF16 : a.cache_dtype, weight_dtype = kBf16 ? RLM_BF16 : a.weight_dtype,
              out_dtype = kBf16 ? RLM_BF16 : a.out_dtype;
    const int R = a.rdim, H = a.hdim, K = a.k_out;
    const int stride = R + kPad;
    const int tile_rows = kRB * K;
    constexpr int kRows = 8 * NR;                          // rows of the product matrix
    float* wm = reinterpret_cast<float*>(smem);
    float* wa = wm + kHT * stride;                        // only when kUpdate
    float* wp = wa + (kUpdate ? kHT * stride : 0);
    float* prod = wp + (kUpdate ? kHT * stride : 0);      // [kRows][R]
    float* red = prod + kRows * R;                        // [kSplit][kRows][kHT] partial sums
    float* cur = red + kSplit * kRows * kHT;              // [kRB][R] current operands (kUpdate)
    float* red2 = cur + (kUpdate ? kRB * R : 0);          // [kSplit][kRB][2][kHT] (kUpdate)
    __shared__ int idx[kRB][kMaxK + 1];
    __shared__ int seq[kRB];

    const int h0 = blockIdx.x * kHT;
    const int ws = weight_dtype == RLM_F32 ? 4 : 2;
    const int cs = cache_dtype == RLM_F32 ? 4 : 2;
    const int segs = R / 8;
    // quotients by the two run-time divisors of the index arithmetic: shifts when they are powers of two
    const int segs_shift = (segs & (segs - 1)) == 0 ? 31 - __clz(segs) : -1;
    const int k_shift = (K & (K - 1)) == 0 ? 31 - __clz(K) : -1;
    auto div_segs = [&](int x) { return segs_shift >= 0 ? x >> segs_shift : x / segs; };
    auto div_k = [&](int x) { return k_shift >= 0 ? x >> k_shift : x / K; };
    // weight tiles: every load of this thread is issued before the first conversion
    for (int i = tid; i < kHT * segs; i += kHiddenThreads) {
        const int r = div_segs(i), sgm = i - r * segs;
        Raw8 rm, ra, rp;
        rm.lo = rm.hi = make_uint4(0, 0, 0, 0);
        ra = rm;
        rp = rm;
        if (h0 + r < H) {
            const size_t off = static_cast<size_t>(h0 + r) * R * ws;
            rm = load8_raw(static_cast<const char*>(a.product_weight) + off, 8 * sgm, weight_dtype);
            if (kUpdate) {
                ra = load8_raw(static_cast<const char*>(a.anchor_weight) + off, 8 * sgm, weight_dtype);
                rp = load8_raw(static_cast<const char*>(a.partner_weight) + off, 8 * sgm, weight_dtype);
            }
        }
        float f[8];
        convert8(rm, weight_dtype, f);
        store8(wm + r * stride + 8 * sgm, f);
        if (kUpdate) {
            convert8(ra, weight_dtype, f);
            store8(wa + r * stride + 8 * sgm, f);
            convert8(rp, weight_dtype, f);
            store8(wp + r * stride + 8 * sgm, f);
        }
    }
    int t = -1;
    if (kUpdate) {
        t = static_cast<int>(*a.position);
        if (t < 0 || t >= a.max_t) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
            return;
        }
    }
    const int rq = tid / kGroupThreads, t7 = tid - rq * kGroupThreads;
    const int tx = t7 & 15, ty = t7 >> 4;                // hidden columns {tx, tx+16}; rows {ty + 8 i}
    const int steps = R / 4;                              // float4 steps along the relation dimension
    const int r_lo = 4 * (rq * steps / kSplit), r_hi = 4 * ((rq + 1) * steps / kSplit);
    const int groups = (a.n_rows + kRB - 1) / kRB;
    griddep_sync();      // the weight tiles are requested; indices and caches may come from the previous kernel

    for (int group = blockIdx.y; group < groups; group += gridDim.y) {
        __syncthreads();   // previous group's reads are done; weight tiles are staged
        const int row0 = group * kRB;
        if (tid < kRB * (K + 1)) {
            int rb = tid / (K + 1), j = tid - rb * (K + 1), row = row0 + rb;
            int v = 0;
            if (row < a.n_rows)
                v = j == 0 ? a.anchor_index[row] : a.partner_index[static_cast<size_t>(row) * K + j - 1];
            idx[rb][j] = min(max(v, 0), a.max_t - 1);
            if (j == 0) {
                int b = row < a.n_rows ? (a.row_batch ? a.row_batch[row] : row) : -1;
                if (row < a.n_rows && (b < 0 || b >= a.n_seq)) {
                    if (a.status) atomicOr(a.status, RLM_DEV_POSITION);
                    b = -1;
                }
                seq[rb] = b;
            }
        }
        __syncthreads();
        // product matrix: prod[rb*K + k][:] = operand[p_k] * operand[anchor]
        for (int i = tid; i < kRows * segs; i += kHiddenThreads) {
            const int prow = div_segs(i), sgm = i - prow * segs;
            const int rb = div_k(prow), k = prow - rb * K;
            float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (prow < tile_rows && seq[rb] >= 0) {
                const char* operand = static_cast<const char*>(a.operand_cache) +
                                      static_cast<size_t>(seq[rb]) * a.max_t * R * cs;
                Raw8 ra = load8_raw(operand + static_cast<size_t>(idx[rb][0]) * R * cs, 8 * sgm, cache_dtype);
                Raw8 rp = load8_raw(operand + static_cast<size_t>(idx[rb][k + 1]) * R * cs, 8 * sgm, cache_dtype);
                float oa[8], op[8];
                convert8(ra, cache_dtype, oa);
                convert8(rp, cache_dtype, op);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = op[e] * oa[e];
            }
            store8(prod + prow * R + 8 * sgm, f);
        }
        if (kUpdate) {
            for (int i = tid; i < kRB * segs; i += kHiddenThreads) {
                const int rb = div_segs(i), sgm = i - rb * segs;
                float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (seq[rb] >= 0)
                    load8(static_cast<const char*>(a.operand_cache) +
                              (static_cast<size_t>(seq[rb]) * a.max_t + t) * R * cs,
                          8 * sgm, cache_dtype, o);
                store8(cur + rb * R + 8 * sgm, o);
            }
        }
        // expanded-cache terms of this thread's epilogue outputs, requested before the
        // arithmetic so that their latency is hidden; pair q covers hidden columns 2q, 2q+1
        constexpr int kPairs = kRows * (kHT / 2) / kHiddenThreads;
        float2 base_a[kPairs], base_p[kPairs];
        int out_row[kPairs], out_k[kPairs];
        bool sub_a[kPairs], sub_p[kPairs];
#pragma unroll
        for (int e = 0; e < kPairs; ++e) {
            const int o = tid + e * kHiddenThreads;
            const int prow = o / (kHT / 2), hh = 2 * (o - prow * (kHT / 2));
            const int rb = div_k(prow), k = prow - rb * K;
            const bool live = prow < tile_rows && row0 + rb < a.n_rows && seq[rb < kRB ? rb : 0] >= 0 &&
                              h0 + hh < H;
            out_row[e] = live ? row0 + rb : -1;
            out_k[e] = k;
            base_a[e] = base_p[e] = make_float2(0.0f, 0.0f);
            sub_a[e] = sub_p[e] = false;
            if (!live) continue;
            const int64_t ebase = static_cast<int64_t>(seq[rb]) * a.max_t * 2 * H;
            const int ai = idx[rb][0], pi = idx[rb][k + 1];
            sub_a[e] = kUpdate && ai == t;
            sub_p[e] = kUpdate && pi == t;
            const bool two = h0 + hh + 1 < H;
            if (!sub_a[e]) {
                const int64_t at = ebase + static_cast<int64_t>(ai) * 2 * H + h0 + hh;
                base_a[e].x = load_scalar(a.expanded_cache, at, cache_dtype);
                if (two) base_a[e].y = load_scalar(a.expanded_cache, at + 1, cache_dtype);
            }
            if (!sub_p[e]) {
                const int64_t at = ebase + static_cast<int64_t>(pi) * 2 * H + H + h0 + hh;
                base_p[e].x = load_scalar(a.expanded_cache, at, cache_dtype);
                if (two) base_p[e].y = load_scalar(a.expanded_cache, at + 1, cache_dtype);
            }
        }
        __syncthreads();

        // partial sums over this group's quarter of the relation dimension
        float acc[NR][2];
#pragma unroll
        for (int i = 0; i < NR; ++i) acc[i][0] = acc[i][1] = 0.0f;
        {
            const float* w0 = wm + tx * stride;
            const float* w1 = w0 + 16 * stride;
            const float* p0 = prod + ty * R;
#pragma unroll 2
            for (int r = r_lo; r < r_hi; r += 4) {
                float4 a0 = *reinterpret_cast<const float4*>(w0 + r);
                float4 a1 = *reinterpret_cast<const float4*>(w1 + r);
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    float4 pv = *reinterpret_cast<const float4*>(p0 + i * 8 * R + r);
                    acc[i][0] = dot4(a0, pv, acc[i][0]);
                    acc[i][1] = dot4(a1, pv, acc[i][1]);
                }
            }
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                red[(rq * kRows + ty + 8 * i) * kHT + tx] = acc[i][0];
                red[(rq * kRows + ty + 8 * i) * kHT + tx + 16] = acc[i][1];
            }
        }
        if (kUpdate) {
            // current expanded rows: thread row ty -> (sequence ty/2, anchor or partner half)
            const int rb = ty >> 1, half = ty & 1;
            const float* w0 = (half ? wp : wa) + tx * stride;
            const float* w1 = w0 + 16 * stride;
            const float* c = cur + rb * R;
            float f0 = 0.0f, f1 = 0.0f;
            for (int r = r_lo; r < r_hi; r += 4) {
                float4 cv = *reinterpret_cast<const float4*>(c + r);
                f0 = dot4(*reinterpret_cast<const float4*>(w0 + r), cv, f0);
                f1 = dot4(*reinterpret_cast<const float4*>(w1 + r), cv, f1);
            }
            red2[((rq * kRB + rb) * 2 + half) * kHT + tx] = f0;
            red2[((rq * kRB + rb) * 2 + half) * kHT + tx + 16] = f1;
        }
        __syncthreads();

        if (kUpdate && tid < kRB * 2 * (kHT / 2)) {
            // fresh expanded rows -> cache row t (rounded to the cache dtype)
            const int pair = tid % (kHT / 2), rh = tid / (kHT / 2);      // rh = rb * 2 + half
            const int rb = rh >> 1, half = rh & 1, hh = 2 * pair;
            if (seq[rb] >= 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (h0 + hh + j >= H) continue;
                    float v = 0.0f;
#pragma unroll
                    for (int q = 0; q < kSplit; ++q) v += red2[((q * kRB + rb) * 2 + half) * kHT + hh + j];
                    if (half == 0) v += load_scalar(a.first_bias, h0 + hh + j, weight_dtype);
                    store_scalar(a.expanded_cache,
                                 (static_cast<int64_t>(seq[rb]) * a.max_t + t) * 2 * H + half * H + h0 + hh + j,
                                 cache_dtype, v);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < kPairs; ++e) {
            if (out_row[e] < 0) continue;
            const int o = tid + e * kHiddenThreads;
            const int prow = o / (kHT / 2), hh = 2 * (o - prow * (kHT / 2));
            const int rb = div_k(prow);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (h0 + hh + j >= H) continue;
                float v = 0.0f;
#pragma unroll
                for (int q = 0; q < kSplit; ++q) v += red[(q * kRows + prow) * kHT + hh + j];
                float ba = j == 0 ? base_a[e].x : base_a[e].y;
                float bp = j == 0 ? base_p[e].x : base_p[e].y;
                if (kUpdate && (sub_a[e] || sub_p[e])) {
                    float fa = 0.0f, fp = 0.0f;
#pragma unroll
                    for (int q = 0; q < kSplit; ++q) {
                        fa += red2[((q * kRB + rb) * 2 + 0) * kHT + hh + j];
                        fp += red2[((q * kRB + rb) * 2 + 1) * kHT + hh + j];
                    }
                    if (sub_a[e]) ba = fa + load_scalar(a.first_bias, h0 + hh + j, weight_dtype);
                    if (sub_p[e]) bp = fp;
                }
                store_scalar(a.out, (static_cast<int64_t>(out_row[e]) * K + out_k[e]) * H + h0 + hh + j,
                             out_dtype, gelu_erf(v + (ba + bp)));
            }
        }
    }
}

int hidden_smem_bytes(bool update, int rdim, int nr) {
    int tiles = update ? 3 : 1;
    int floats = tiles * kHT * (rdim + kPad) + 8 * nr * rdim + kSplit * 8 * nr * kHT;
    if (update) floats += kRB * rdim + kSplit * kRB * 2 * kHT;
    return floats * 4;
}

template <bool kUpdate, int NR>
int launch_hidden_as(const HiddenArgs& a, void* stream) {
    const int smem_bytes = hidden_smem_bytes(kUpdate, a.rdim, NR);
    if (smem_bytes > kSmemDynamicLimit) {
        set_error("relation_hidden: relation_dim too large for the staged weight tiles");
        return RLM_ERR_SMEM;
    }
    const bool bf16 = a.cache_dtype == RLM_BF16 && a.weight_dtype == RLM_BF16 && a.out_dtype == RLM_BF16;
    auto kernel = bf16 ? relation_hidden_kernel<kUpdate, NR, true> : relation_hidden_kernel<kUpdate, NR, false>;
    if (smem_bytes > 48 * 1024) {
        int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
        if (rc != RLM_OK) return rc;
    }
    const int tiles = (a.hdim + kHT - 1) / kHT;
    const int groups = (a.n_rows + kRB - 1) / kRB;
    // a few CTAs per SM; beyond that a CTA keeps its weight tiles and walks several groups
    int gy = (sm_count() * 4 + tiles - 1) / tiles;
    if (gy > groups) gy = groups;
    dim3 grid(tiles, gy);
    launch_kernel(kernel, dim3(grid), dim3(kHiddenThreads), smem_bytes, stream, a);
    count_launch();
    return check_launch("relation_hidden_kernel");
}

int launch_hidden(HiddenArgs& a, bool update, void* stream) {
    if (a.n_rows == 0) return RLM_OK;
    if (!a.expanded_cache || !a.operand_cache || !a.anchor_index || !a.partner_index ||
        !a.product_weight || !a.out ||
        (update && (!a.anchor_weight || !a.partner_weight || !a.first_bias || !a.position))) {
        set_error("relation_hidden: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (a.n_rows < 0 || a.n_seq < 1 || a.max_t < 1 || a.rdim < 16 || a.rdim % 16 != 0 || a.hdim < 1 ||
        a.k_out < 1 || a.k_out > kMaxK) {
        set_error("relation_hidden: need relation_dim a multiple of 16, 1 <= K <= 16 and positive sizes");
        return RLM_ERR_SHAPE;
    }
    if (!a.row_batch && a.n_rows != a.n_seq) {
        set_error("relation_hidden: without row_batch the rows must equal the sequences");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(a.cache_dtype) || !valid_dtype(a.weight_dtype) || !valid_dtype(a.out_dtype)) {
        set_error("relation_hidden: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    if (!aligned16(a.product_weight) || !aligned16(a.operand_cache) ||
        (update && (!aligned16(a.anchor_weight) || !aligned16(a.partner_weight)))) {
        set_error("relation_hidden: weight matrices and the operand cache must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    if (hidden_tc_applicable(update, a.n_rows, a.rdim, a.hdim, a.k_out, a.cache_dtype, a.weight_dtype,
                             a.expanded_cache, a.out))
        return launch_hidden_tc(update, a.expanded_cache, a.operand_cache, a.anchor_index, a.partner_index,
                                a.anchor_weight, a.partner_weight, a.product_weight, a.first_bias,
                                a.position, a.row_batch, a.out, a.n_rows, a.n_seq, a.max_t, a.rdim, a.hdim,
                                a.k_out, a.cache_dtype, a.out_dtype, a.status, stream);
    const bool wide = kRB * a.k_out > 32;      // more than 4 relation rows per thread
    if (update) return wide ? launch_hidden_as<true, 8>(a, stream) : launch_hidden_as<true, 4>(a, stream);
    return wide ? launch_hidden_as<false, 8>(a, stream) : launch_hidden_as<false, 4>(a, stream);
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
    float* out;               // context [N, D], or NULL when only the residual is wanted
    float* residual;          // optional [N, D] fp32: residual += (*mix) * context
    const float* mix;
    int raw_splits;           // raw is the sum of this many slices, raw_split_stride elements apart (split-K GEMM)
    int64_t raw_split_stride;
    const void* raw_bias;     // optional [D] (param dtype): added to every partner row
    const float* next_w;      // optional: LayerNorm of the updated residual row, written as 16-bit
    const float* next_b;      //   values to next_out [N, D] (the next layer's normalised input)
    void* next_out;
    float next_eps;
    int next_dtype;
    int32_t* status;
    float eps;
    int n_rows, k_out, dim, raw_dtype, param_dtype;
    // fused projection of the normalised row (relation_norm_reduce_project_kernel only)
    const void* proj_weight;  // [proj_out_dim, dim], the next_out dtype
    void* proj_out;           // [N, proj_out_dim], the next_out dtype
    int proj_out_dim;
};

__global__ void __launch_bounds__(kNormThreads) relation_norm_reduce_kernel(const NormArgs a) {
    extern __shared__ __align__(16) float partial[];   // [warps][dim]
    griddep_sync();
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = a.k_out, D = a.dim;
    const int per = (D + 31) / 32;

    // Every load that does not depend on another is issued first: position, scores, this
    // warp's first partner row and the affine parameters.  (raw is dense [N, K, D], so the
    // row of an inactive slot is readable; it is simply not accumulated.)
    const int t = a.row_position ? a.row_position[row] : static_cast<int>(*a.position);
    float s0 = lane < K ? a.scores[static_cast<size_t>(row) * K + lane] : kNegInf;
    float s1 = lane + 32 < K ? a.scores[static_cast<size_t>(row) * K + lane + 32] : kNegInf;
    float x[kMaxPerLane];
    if (warp < K) {
        const int64_t base = (static_cast<int64_t>(row) * K + warp) * D;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            int c = lane + 32 * i;
            x[i] = (i < per && c < D) ? load_scalar(a.raw, base + c, a.raw_dtype) : 0.0f;
        }
    }
    float gm[kMaxPerLane], bt[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        int c = lane + 32 * i;
        bool in = i < per && c < D;
        gm[i] = in ? load_scalar(a.weight, c, a.param_dtype) : 0.0f;
        bt[i] = in ? load_scalar(a.bias, c, a.param_dtype) : 0.0f;
    }

    // softmax weights over the active slots (every warp computes them redundantly)
    int k_limit = 32 - __clz(max(t, 0) + 1);   // ceil(log2(t + 2))
    k_limit = min(max(k_limit, 1), K);
    bool a0 = lane < K && lane < k_limit && s0 > -1.0e30f;
    bool a1 = lane + 32 < K && lane + 32 < k_limit && s1 > -1.0e30f;
    float f0 = a0 ? s0 : -1.0e4f, f1 = a1 ? s1 : -1.0e4f;
    float mx = fmaxf(f0, f1);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float e0 = a0 ? expf(f0 - mx) : 0.0f, e1 = a1 ? expf(f1 - mx) : 0.0f;
    float den = fmaxf(warp_sum(e0 + e1), 1.0e-9f);
    float w0 = e0 / den, w1 = e1 / den;

    float y[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) y[i] = 0.0f;
    for (int k = warp; k < K; k += kNormWarps) {
        float wk = __shfl_sync(0xffffffffu, k < 32 ? w0 : w1, k & 31);
        if (k != warp && wk != 0.0f) {
            const int64_t base = (static_cast<int64_t>(row) * K + k) * D;
#pragma unroll
            for (int i = 0; i < kMaxPerLane; ++i) {
                int c = lane + 32 * i;
                x[i] = (i < per && c < D) ? load_scalar(a.raw, base + c, a.raw_dtype) : 0.0f;
            }
        }
        if (wk == 0.0f) continue;   // inactive slot contributes nothing
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) sum += x[i];
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
        for (int i = 0; i < kMaxPerLane; ++i) y[i] = fmaf(wk, fmaf(x[i] * inv, gm[i], bt[i]), y[i]);
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
        if (a.out) a.out[static_cast<size_t>(row) * D + c] = total;
        if (a.residual) {
            const size_t at = static_cast<size_t>(row) * D + c;
            a.residual[at] = fmaf(*a.mix, total, a.residual[at]);
        }
    }
}

// Vector form for feature widths that are a multiple of 8 (16-byte aligned rows): a lane owns
// the 8-column chunks lane, lane + 32, ... (kVecChunks of them, at most four: dim <= 1024), so a partner row is
// fetched with a few 16-byte loads per lane instead of one scalar load per column.
// One row by one CTA; `partial` is [warps][dim] floats of shared memory.  With `normalized_copy`
// (shared memory, dim 16-bit values) the next layer's normalised row is left there as well.
// kEarly (kernels without an occupancy target): the affine parameters, the residual row and the
// mixing weight are requested into registers at the top instead of where the chain reaches them.
template <int kVecChunks, bool kEarly, bool kPlain>
__device__ __forceinline__ void norm_reduce_vec_row(const NormArgs& a, int row, float* partial,
                                                    void* normalized_copy) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // kPlain: bf16 partner rows in one slice without a bias, fp32 parameters, bf16 normalised
    // output (the decode step): the dtype and slice branches fold away
    const int raw_dtype = kPlain ? RLM_BF16 : a.raw_dtype, param_dtype = kPlain ? RLM_F32 : a.param_dtype;
    const int next_dtype = kPlain ? RLM_BF16 : a.next_dtype, raw_splits = kPlain ? 1 : a.raw_splits;
    const void* raw_bias = kPlain ? nullptr : a.raw_bias;
    const int K = a.k_out, D = a.dim;
    const int chunks = D / 8;
    const size_t raw_elem = raw_dtype == RLM_F32 ? 4 : 2;

    // loads that depend on nothing first: position, scores, this warp's first partner row, affine
    const int t = a.row_position ? a.row_position[row] : static_cast<int>(*a.position);
    float s0 = lane < K ? a.scores[static_cast<size_t>(row) * K + lane] : kNegInf;
    float s1 = lane + 32 < K ? a.scores[static_cast<size_t>(row) * K + lane + 32] : kNegInf;
    float x[kVecChunks][8];
    float gm_early[kEarly ? kVecChunks : 1][8], bt_early[kEarly ? kVecChunks : 1][8];
    float4 res_early = make_float4(0.0f, 0.0f, 0.0f, 0.0f), next_g = res_early, next_b = res_early;
    float mix_early = 0.0f;
    if (kEarly) {
#pragma unroll
        for (int i = 0; i < kVecChunks; ++i)
            if (lane + 32 * i < chunks) {
                load8(a.weight, 8 * (lane + 32 * i), param_dtype, gm_early[i]);
                load8(a.bias, 8 * (lane + 32 * i), param_dtype, bt_early[i]);
            }
        if (4 * tid < D) {
            if (a.residual) res_early = *reinterpret_cast<const float4*>(a.residual + static_cast<size_t>(row) * D + 4 * tid);
            if (a.next_out) {
                next_g = *reinterpret_cast<const float4*>(a.next_w + 4 * tid);
                next_b = *reinterpret_cast<const float4*>(a.next_b + 4 * tid);
            }
        }
        if (a.residual) mix_early = *a.mix;
    }
    // one 8-column chunk of partner row k: the slices of a split-K GEMM are summed and the bias added here
    auto load_raw = [&](const char* row_k, int chunk, float (&dst)[8]) {
        load8(row_k, 8 * chunk, raw_dtype, dst);
        for (int sp = 1; sp < raw_splits; ++sp) {
            float more[8];
            load8(row_k + static_cast<size_t>(sp) * a.raw_split_stride * raw_elem, 8 * chunk, raw_dtype, more);
#pragma unroll
            for (int e = 0; e < 8; ++e) dst[e] += more[e];
        }
        if (raw_bias) {
            float bias8[8];
            load8(raw_bias, 8 * chunk, param_dtype, bias8);
#pragma unroll
            for (int e = 0; e < 8; ++e) dst[e] += bias8[e];
        }
    };
    const char* raw_row = static_cast<const char*>(a.raw) + static_cast<size_t>(row) * K * D * raw_elem;
    if (warp < K) {
#pragma unroll
        for (int i = 0; i < kVecChunks; ++i)
            if (lane + 32 * i < chunks) load_raw(raw_row + static_cast<size_t>(warp) * D * raw_elem, lane + 32 * i, x[i]);
    }

    int k_limit = 32 - __clz(max(t, 0) + 1);   // ceil(log2(t + 2))
    k_limit = min(max(k_limit, 1), K);
    bool a0 = lane < K && lane < k_limit && s0 > -1.0e30f;
    bool a1 = lane + 32 < K && lane + 32 < k_limit && s1 > -1.0e30f;
    float f0 = a0 ? s0 : -1.0e4f, f1 = a1 ? s1 : -1.0e4f;
    float mx = fmaxf(f0, f1);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float e0 = a0 ? expf(f0 - mx) : 0.0f, e1 = a1 ? expf(f1 - mx) : 0.0f;
    float den = fmaxf(warp_sum(e0 + e1), 1.0e-9f);
    float w0 = e0 / den, w1 = e1 / den;

    float y[kVecChunks][8];
#pragma unroll
    for (int i = 0; i < kVecChunks; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) y[i][e] = 0.0f;
    for (int k = warp; k < K; k += kNormWarps) {
        float wk = __shfl_sync(0xffffffffu, k < 32 ? w0 : w1, k & 31);
        if (k != warp && wk != 0.0f) {
#pragma unroll
            for (int i = 0; i < kVecChunks; ++i)
                if (lane + 32 * i < chunks) load_raw(raw_row + static_cast<size_t>(k) * D * raw_elem, lane + 32 * i, x[i]);
        }
        if (wk == 0.0f) continue;   // inactive slot contributes nothing
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kVecChunks; ++i)
            if (lane + 32 * i < chunks)
#pragma unroll
                for (int e = 0; e < 8; ++e) sum += x[i][e];
        const float mean = warp_sum(sum) / static_cast<float>(D);
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < kVecChunks; ++i)
            if (lane + 32 * i < chunks)
#pragma unroll
                for (int e = 0; e < 8; ++e) { x[i][e] -= mean; sq = fmaf(x[i][e], x[i][e], sq); }
        const float inv = rsqrtf(warp_sum(sq) / static_cast<float>(D) + a.eps);
#pragma unroll
        for (int i = 0; i < kVecChunks; ++i)
            if (lane + 32 * i < chunks) {
                float gm[8], bt[8];       // cache-resident affine parameters, read where they are used
                if (kEarly) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) { gm[e] = gm_early[i][e]; bt[e] = bt_early[i][e]; }
                } else {
                    load8(a.weight, 8 * (lane + 32 * i), param_dtype, gm);
                    load8(a.bias, 8 * (lane + 32 * i), param_dtype, bt);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) y[i][e] = fmaf(wk, fmaf(x[i][e] * inv, gm[e], bt[e]), y[i][e]);
            }
    }
#pragma unroll
    for (int i = 0; i < kVecChunks; ++i)
        if (lane + 32 * i < chunks) {
            float4* dst = reinterpret_cast<float4*>(partial + warp * D + 8 * (lane + 32 * i));
            dst[0] = make_float4(y[i][0], y[i][1], y[i][2], y[i][3]);
            dst[1] = make_float4(y[i][4], y[i][5], y[i][6], y[i][7]);
        }
    __syncthreads();
    const float mix = kEarly ? mix_early : (a.residual ? *a.mix : 0.0f);
    const int c = 4 * tid;                 // dim <= 1024: every thread owns at most four columns
    const bool live = c < D;
    float updated[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
        float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const int used = K < kNormWarps ? K : kNormWarps;      // warps beyond K hold zeros
#pragma unroll
        for (int w = 0; w < kNormWarps; ++w) {
            if (w >= used) break;
            const float4 v = *reinterpret_cast<const float4*>(partial + w * D + c);
            total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
        }
        const size_t at = static_cast<size_t>(row) * D + c;
        if (a.out) *reinterpret_cast<float4*>(a.out + at) = total;
        if (a.residual) {
            float4 r = kEarly ? res_early : *reinterpret_cast<float4*>(a.residual + at);
            r.x = fmaf(mix, total.x, r.x); r.y = fmaf(mix, total.y, r.y);
            r.z = fmaf(mix, total.z, r.z); r.w = fmaf(mix, total.w, r.w);
            *reinterpret_cast<float4*>(a.residual + at) = r;
            updated[0] = r.x; updated[1] = r.y; updated[2] = r.z; updated[3] = r.w;
        }
    }
    if (a.next_out) {
        __shared__ float scratch[18];
        NormTarget t0{a.next_w, a.next_b, static_cast<uint16_t*>(a.next_out) + static_cast<size_t>(row) * D};
        NormTarget t1{a.next_w, a.next_b, normalized_copy};
        block_layer_norm4(updated, live, c, D, a.next_eps, t0, t1, next_dtype, scratch,
                          kEarly ? &next_g : nullptr, kEarly ? &next_b : nullptr);
    }
}

template <int kVecChunks, bool kPlain>
__global__ void __launch_bounds__(kNormThreads, kVecChunks <= 2 ? 4 : (kVecChunks == 3 ? 3 : 2)) relation_norm_reduce_vec_kernel(const NormArgs a) {
    extern __shared__ __align__(16) float partial[];   // [warps][dim]
    griddep_sync();
    norm_reduce_vec_row<kVecChunks, false, kPlain>(a, blockIdx.x, partial, nullptr);
}

// ---- thousands of rows (whole-sequence passes): a warp per row
//
// The CTA-per-row kernels above spread a row's K partners over the warps and meet in shared
// memory: right for a decode batch, where a row's latency counts, but a pass over 10^4 .. 10^5 rows
// is a stream of K x dim 16-bit values per row and should run at memory speed.  Here a warp owns a
// row: it requests all its active partners' rows at once (K x dim / 16 sixteen-byte loads in
// flight per lane), then normalises and accumulates them one after the other with warp shuffles
// only — no shared memory, no block-wide barrier.  Plain form only: 16-bit raw rows in one slice,
// fp32 parameters, context output.  Same formulas as relation_norm_reduce_vec_kernel
// (src/relation_lm/kernels/relation_reduce.py:360-417 of the reference project).
constexpr int kRowWarpK = 8;          // partners per row this form holds in registers

template <int kChunks, bool kBf16>
__global__ void __launch_bounds__(256) relation_norm_reduce_warp_kernel(const NormArgs a) {
    griddep_sync();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= a.n_rows) return;
    const int K = a.k_out;
    constexpr int D = 256 * kChunks;
    const int t = a.row_position ? a.row_position[row] : static_cast<int>(*a.position);
    const float s = lane < K ? a.scores[static_cast<size_t>(row) * K + lane] : kNegInf;
    int k_limit = 32 - __clz(max(t, 0) + 1);   // ceil(log2(t + 2))
    k_limit = min(max(k_limit, 1), K);
    const bool active = lane < K && lane < k_limit && s > -1.0e30f;
    const unsigned live = __ballot_sync(0xffffffffu, active);
    // every active partner's row, requested before anything is computed
    const uint4* raw_row = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.raw) + static_cast<size_t>(row) * K * D);
    uint4 raw[kRowWarpK][kChunks];
#pragma unroll
    for (int k = 0; k < kRowWarpK; ++k)
#pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            raw[k][i] = make_uint4(0, 0, 0, 0);
            if ((live >> k) & 1u) raw[k][i] = raw_row[k * (D / 8) + lane + 32 * i];
        }
    const float f = active ? s : -1.0e4f;
    float mx = f;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    const float e = active ? expf(f - mx) : 0.0f;
    const float w = e / fmaxf(warp_sum(e), 1.0e-9f);
    float gm[kChunks][8], bt[kChunks][8], y[kChunks][8];
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
        load8(a.weight, 8 * (lane + 32 * i), RLM_F32, gm[i]);
        load8(a.bias, 8 * (lane + 32 * i), RLM_F32, bt[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[i][j] = 0.0f;
    }
#pragma unroll
    for (int k = 0; k < kRowWarpK; ++k) {
        const float wk = __shfl_sync(0xffffffffu, w, k);
        if (!((live >> k) & 1u) || wk == 0.0f) continue;       // (warp-uniform) inactive slots contribute nothing
        float x[kChunks][8], sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kChunks; ++i) {
            Raw8 r8;
            r8.lo = raw[k][i];
            r8.hi = make_uint4(0, 0, 0, 0);
            convert8(r8, kBf16 ? RLM_BF16 : RLM_F16, x[i]);
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += x[i][j];
        }
        const float mean = warp_sum(sum) / static_cast<float>(D);
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < kChunks; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) { x[i][j] -= mean; sq = fmaf(x[i][j], x[i][j], sq); }
        const float inv = rsqrtf(warp_sum(sq) / static_cast<float>(D) + a.eps);
#pragma unroll
        for (int i = 0; i < kChunks; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) y[i][j] = fmaf(wk, fmaf(x[i][j] * inv, gm[i][j], bt[i][j]), y[i][j]);
    }
#pragma unroll
    for (int i = 0; i < kChunks; ++i) {
        float4* dst = reinterpret_cast<float4*>(a.out + static_cast<size_t>(row) * D + 8 * (lane + 32 * i));
        dst[0] = make_float4(y[i][0], y[i][1], y[i][2], y[i][3]);
        dst[1] = make_float4(y[i][4], y[i][5], y[i][6], y[i][7]);
    }
}

// ---- norm-reduce + residual + next LayerNorm + the next layer's query projection, for decode
// batches of a few rows.  A cluster of proj_out_dim / 32 CTAs serves one row: every CTA requests
// its 32 x dim slice of the projection weight before the dependency wait (eight lanes per output
// row, 16-byte pieces interleaved so that the lanes read contiguous bytes), CTA 0 of the cluster
// does the row's norm-reduce and stores the normalised row (16-bit, as the tensor-core projection
// would read it) into every CTA's shared memory through distributed shared memory, and after one
// cluster barrier everybody finishes its 32 outputs with fp32 accumulation.  One launch instead of two, and the
// weight fetch overlaps the norm-reduce chain.
constexpr int kProjCols = 32;     // projection outputs per CTA

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Stores 16 bytes at the address that `local_ptr` has in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ void store_cluster_shared16(const void* local_ptr, uint32_t rank, const uint4& v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};"
                 ::"r"(remote), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int kVecChunks, bool kPlain>
__global__ void __launch_bounds__(kNormThreads) relation_norm_reduce_project_kernel(const NormArgs a) {
    extern __shared__ __align__(16) float partial[];            // [warps][dim], CTA 0 of the cluster
    __shared__ __align__(16) uint16_t normalized_row[1024];
    constexpr int kPieces = 4 * kVecChunks;                      // 16-byte weight pieces per thread: dim <= 256 * kVecChunks
    const int tid = threadIdx.x;
    const int D = a.dim, pieces = D / 64;                        // dim is a multiple of 64
    const int next_dtype = kPlain ? RLM_BF16 : a.next_dtype;
    const uint32_t rank = cluster_rank();
    const int slices = a.proj_out_dim / kProjCols;
    const int row = blockIdx.x / slices;
    const int col = static_cast<int>(rank) * kProjCols + (tid >> 3), part = tid & 7;
    uint4 w[kPieces];
    {
        const uint4* wrow = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.proj_weight) +
                                                           static_cast<size_t>(col) * D);
#pragma unroll
        for (int j = 0; j < kPieces; ++j)
            if (j < pieces) w[j] = wrow[part + 8 * j];
    }
    griddep_sync();
    if (rank == 0) {
        norm_reduce_vec_row<kVecChunks, true, kPlain>(a, row, partial, normalized_row);
        __syncthreads();
        if (tid < D / 8) {          // hand the normalised row to the other CTAs of the cluster
            const uint4 v = reinterpret_cast<const uint4*>(normalized_row)[tid];
            for (int r = 1; r < slices; ++r)
                store_cluster_shared16(reinterpret_cast<uint4*>(normalized_row) + tid, static_cast<uint32_t>(r), v);
        }
    }
    cluster_sync_all();             // release / acquire: the row is visible in every CTA's shared memory
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < kPieces; ++j) {
        if (j < pieces) {
            float wf[8], xf[8];
            Raw8 raw;
            raw.lo = w[j];
            raw.hi = make_uint4(0, 0, 0, 0);
            convert8(raw, next_dtype, wf);
            load8(normalized_row, 8 * (part + 8 * j), next_dtype, xf);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fmaf(wf[e], xf[e], acc);
        }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (part == 0)
        store_scalar(a.proj_out, static_cast<int64_t>(row) * a.proj_out_dim + col, next_dtype, acc);
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_relation_hidden_cached(
    const void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const void* product_weight, const int32_t* row_batch, void* out,
    int n_rows, int n_seq, int max_t, int relation_dim, int hidden_dim, int k_out, int cache_dtype,
    int weight_dtype, int out_dtype, int32_t* status, void* stream) {
    rlm::HiddenArgs a{};
    a.expanded_cache = const_cast<void*>(expanded_cache); a.operand_cache = operand_cache;
    a.anchor_index = anchor_index; a.partner_index = partner_index; a.product_weight = product_weight;
    a.row_batch = row_batch; a.out = out; a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.rdim = relation_dim; a.hdim = hidden_dim;
    a.k_out = k_out; a.cache_dtype = cache_dtype; a.weight_dtype = weight_dtype; a.out_dtype = out_dtype;
    return rlm::launch_hidden(a, false, stream);
}

extern "C" int rlm_relation_hidden_cache_update(
    void* expanded_cache, const void* operand_cache, const int32_t* anchor_index,
    const int32_t* partner_index, const void* anchor_weight, const void* partner_weight,
    const void* product_weight, const void* first_bias, const int64_t* position, void* out,
    int batch, int max_t, int relation_dim, int hidden_dim, int k_out, int cache_dtype,
    int weight_dtype, int out_dtype, int32_t* status, void* stream) {
    rlm::HiddenArgs a{};
    a.expanded_cache = expanded_cache; a.operand_cache = operand_cache;
    a.anchor_index = anchor_index; a.partner_index = partner_index;
    a.anchor_weight = anchor_weight; a.partner_weight = partner_weight;
    a.product_weight = product_weight; a.first_bias = first_bias; a.position = position;
    a.out = out; a.status = status;
    a.n_rows = batch; a.n_seq = batch; a.max_t = max_t; a.rdim = relation_dim; a.hdim = hidden_dim;
    a.k_out = k_out; a.cache_dtype = cache_dtype; a.weight_dtype = weight_dtype; a.out_dtype = out_dtype;
    return rlm::launch_hidden(a, true, stream);
}

namespace rlm {
namespace {
int norm_reduce_launch(
    const void* raw, const float* partner_scores, const void* norm_weight, const void* norm_bias,
    const int64_t* position, const int32_t* row_position, float norm_eps, float* out,
    float* residual, const float* mix, const float* next_norm_weight, const float* next_norm_bias,
    float next_norm_eps, void* next_normalized, int next_dtype, int raw_splits,
    int64_t raw_split_stride, const void* raw_bias, const void* proj_weight, void* proj_out, int proj_out_dim,
    int n_rows, int k_out, int dim, int raw_dtype, int param_dtype, int32_t* status, void* stream) {
    if (n_rows == 0) return RLM_OK;
    if (!raw || !partner_scores || !norm_weight || !norm_bias || (!out && !residual) ||
        (residual && !mix) || (!position && !row_position)) {
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
    a.residual = residual; a.mix = mix;
    a.next_w = next_norm_weight; a.next_b = next_norm_bias; a.next_out = next_normalized;
    a.next_eps = next_norm_eps; a.next_dtype = next_dtype;
    a.raw_splits = raw_splits < 1 ? 1 : raw_splits; a.raw_split_stride = raw_split_stride; a.raw_bias = raw_bias;
    a.eps = norm_eps; a.n_rows = n_rows; a.k_out = k_out; a.dim = dim;
    a.raw_dtype = raw_dtype; a.param_dtype = param_dtype;
    int smem_bytes = kNormWarps * dim * 4;
    const bool vec = dim % 8 == 0 && aligned16(raw) && aligned16(norm_weight) && aligned16(norm_bias) &&
                     (!out || aligned16(out)) && (!residual || aligned16(residual));
    if ((raw_splits > 1 || raw_bias) && (!vec || (raw_bias && !aligned16(raw_bias)) ||
                                          (raw_splits > 1 && (raw_split_stride * dtype_size(raw_dtype)) % 16 != 0))) {
        set_error("relation_norm_reduce: summed slices / a bias need dim a multiple of 8 and 16-byte aligned tensors");
        return RLM_ERR_UNSUPPORTED;
    }
    if (next_normalized) {
        if (!residual || !next_norm_weight || !next_norm_bias || !vec || !aligned16(next_norm_weight) ||
            !aligned16(next_norm_bias) || !aligned16(next_normalized) ||
            (next_dtype != RLM_BF16 && next_dtype != RLM_F16)) {
            set_error("relation_norm_reduce: the normalised output needs the residual form, dim a multiple "
                      "of 8, 16-byte aligned tensors and a 16-bit dtype");
            return RLM_ERR_UNSUPPORTED;
        }
    }
    if (proj_out) {
        if (!proj_weight || !next_normalized || dim % 64 != 0 || proj_out_dim < kProjCols ||
            proj_out_dim % kProjCols != 0 || proj_out_dim > 8 * kProjCols || !aligned16(proj_weight)) {
            set_error("relation_norm_reduce_project: needs the normalised output, dim a multiple of 64, "
                      "32..256 projection outputs in steps of 32 and a 16-byte aligned weight");
            return RLM_ERR_UNSUPPORTED;
        }
        a.proj_weight = proj_weight; a.proj_out = proj_out; a.proj_out_dim = proj_out_dim;
        const unsigned slices = static_cast<unsigned>(proj_out_dim / kProjCols);
        const dim3 grid(static_cast<unsigned>(n_rows) * slices);
        const bool plain = raw_dtype == RLM_BF16 && param_dtype == RLM_F32 && next_dtype == RLM_BF16 &&
                           a.raw_splits == 1 && !raw_bias;
        auto kernel = dim <= 512 ? (plain ? relation_norm_reduce_project_kernel<2, true> : relation_norm_reduce_project_kernel<2, false>)
                    : dim <= 768 ? (plain ? relation_norm_reduce_project_kernel<3, true> : relation_norm_reduce_project_kernel<3, false>)
                                 : (plain ? relation_norm_reduce_project_kernel<4, true> : relation_norm_reduce_project_kernel<4, false>);
        launch_kernel_cluster(kernel, grid, dim3(kNormThreads), slices, smem_bytes, stream, a);
        count_launch();
        return check_launch("relation_norm_reduce_project_kernel");
    }
    // thousands of rows in the plain form: a warp per row, all of a row's partner rows in flight at once
    if (vec && n_rows >= 2048 && k_out <= kRowWarpK && dim % 256 == 0 && out && !residual && !next_normalized &&
        a.raw_splits == 1 && !raw_bias && param_dtype == RLM_F32 && (raw_dtype == RLM_BF16 || raw_dtype == RLM_F16)) {
        using Kernel = void (*)(const NormArgs);
        const bool bf16 = raw_dtype == RLM_BF16;
        Kernel kernel = dim == 256 ? (bf16 ? relation_norm_reduce_warp_kernel<1, true> : relation_norm_reduce_warp_kernel<1, false>)
                      : dim == 512 ? (bf16 ? relation_norm_reduce_warp_kernel<2, true> : relation_norm_reduce_warp_kernel<2, false>)
                      : dim == 768 ? (bf16 ? relation_norm_reduce_warp_kernel<3, true> : relation_norm_reduce_warp_kernel<3, false>)
                                   : (bf16 ? relation_norm_reduce_warp_kernel<4, true> : relation_norm_reduce_warp_kernel<4, false>);
        launch_kernel(kernel, dim3((n_rows + 7) / 8), dim3(256), 0, stream, a);
        count_launch();
        return check_launch("relation_norm_reduce_warp_kernel");
    }
    // the decode step's dtypes (bf16 rows in one slice, fp32 parameters) take builds without dtype branches
    const bool plain_rows = raw_dtype == RLM_BF16 && param_dtype == RLM_F32 && a.raw_splits == 1 && !raw_bias &&
                            (!next_normalized || next_dtype == RLM_BF16);
    if (vec) {
        auto kernel = dim <= 512 ? (plain_rows ? relation_norm_reduce_vec_kernel<2, true> : relation_norm_reduce_vec_kernel<2, false>)
                    : dim <= 768 ? (plain_rows ? relation_norm_reduce_vec_kernel<3, true> : relation_norm_reduce_vec_kernel<3, false>)
                                 : (plain_rows ? relation_norm_reduce_vec_kernel<4, true> : relation_norm_reduce_vec_kernel<4, false>);
        launch_kernel(kernel, dim3(n_rows), dim3(kNormThreads), smem_bytes, stream, a);
    } else
        launch_kernel(relation_norm_reduce_kernel, dim3(n_rows), dim3(kNormThreads), smem_bytes, stream, a);
    count_launch();
    return check_launch("relation_norm_reduce_kernel");
}
}  // namespace
}  // namespace rlm

extern "C" int rlm_relation_norm_reduce(
    const void* raw, const float* partner_scores, const void* norm_weight, const void* norm_bias,
    const int64_t* position, const int32_t* row_position, float norm_eps, float* out,
    float* residual, const float* mix, const float* next_norm_weight, const float* next_norm_bias,
    float next_norm_eps, void* next_normalized, int next_dtype, int raw_splits,
    int64_t raw_split_stride, const void* raw_bias, int n_rows,
    int k_out, int dim, int raw_dtype, int param_dtype, int32_t* status, void* stream) {
    return rlm::norm_reduce_launch(raw, partner_scores, norm_weight, norm_bias, position, row_position, norm_eps,
                                   out, residual, mix, next_norm_weight, next_norm_bias, next_norm_eps,
                                   next_normalized, next_dtype, raw_splits, raw_split_stride, raw_bias, nullptr,
                                   nullptr, 0, n_rows, k_out, dim, raw_dtype, param_dtype, status, stream);
}

extern "C" int rlm_relation_norm_reduce_project(
    const void* raw, const float* partner_scores, const void* norm_weight, const void* norm_bias,
    const int64_t* position, float norm_eps, float* residual, const float* mix,
    const float* next_norm_weight, const float* next_norm_bias, float next_norm_eps, void* next_normalized,
    const void* proj_weight, void* proj_out, int proj_out_dim, int next_dtype, const void* raw_bias, int n_rows,
    int k_out, int dim, int raw_dtype, int param_dtype, int32_t* status, void* stream) {
    if (!proj_weight || !proj_out) {
        rlm::set_error("relation_norm_reduce_project: NULL projection weight or output");
        return RLM_ERR_NULL;
    }
    return rlm::norm_reduce_launch(raw, partner_scores, norm_weight, norm_bias, position, nullptr, norm_eps, nullptr,
                                   residual, mix, next_norm_weight, next_norm_bias, next_norm_eps, next_normalized,
                                   next_dtype, 1, 0, raw_bias, proj_weight, proj_out, proj_out_dim, n_rows, k_out,
                                   dim, raw_dtype, param_dtype, status, stream);
}


// ------------------------------------------------------------------ multi-anchor slot mixing
//
// Last step of a multi-anchor relation layer (src/relation_lm/models/multi_relation_blocks.py:170-178
// of the reference project): the slots' contexts are mixed with learned softmax weights
// renormalised over the slots that are active for the query, and the result enters the residual
// stream through a sigmoid gate:
//   w[n, s]  = slot_weight[s] * active[n, s] / max(sum_s' slot_weight[s'] * active[n, s'], 1e-9)
//   hidden[n] += gate * sum_s w[n, s] * slot_context[n, s]
namespace rlm {
namespace {
constexpr int kMixMaxSlots = 8;

__global__ void __launch_bounds__(256) slot_mix_residual_kernel(
    const float* __restrict__ slot_context, const uint8_t* __restrict__ active, const float* __restrict__ slot_weight,
    const float* __restrict__ gate, float* __restrict__ hidden, int n_rows, int slots, int dim) {
    griddep_sync();
    const int vecs = dim >> 2;                                  // float4 columns per row
    const float g = *gate;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
         i < static_cast<int64_t>(n_rows) * vecs; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int n = static_cast<int>(i / vecs), c = static_cast<int>(i - static_cast<int64_t>(n) * vecs);
        float w[kMixMaxSlots], total = 0.0f;
#pragma unroll
        for (int s = 0; s < kMixMaxSlots; ++s) {
            w[s] = s < slots && active[static_cast<size_t>(n) * slots + s] ? slot_weight[s] : 0.0f;
            total += w[s];
        }
        const float inv = 1.0f / fmaxf(total, 1.0e-9f);
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int s = 0; s < kMixMaxSlots; ++s) {
            if (w[s] == 0.0f) continue;
            const float4 v = reinterpret_cast<const float4*>(slot_context + (static_cast<size_t>(n) * slots + s) * dim)[c];
            const float ws = w[s] * inv;
            acc.x = fmaf(ws, v.x, acc.x); acc.y = fmaf(ws, v.y, acc.y); acc.z = fmaf(ws, v.z, acc.z); acc.w = fmaf(ws, v.w, acc.w);
        }
        float4* h = reinterpret_cast<float4*>(hidden + static_cast<size_t>(n) * dim) + c;
        float4 hv = *h;
        hv.x = fmaf(g, acc.x, hv.x); hv.y = fmaf(g, acc.y, hv.y); hv.z = fmaf(g, acc.z, hv.z); hv.w = fmaf(g, acc.w, hv.w);
        *h = hv;
    }
}
}  // namespace
}  // namespace rlm

extern "C" int rlm_slot_mix_residual(const float* slot_context, const uint8_t* anchor_active, const float* slot_weight,
                                     const float* gate, float* hidden, int n_rows, int slots, int d_model,
                                     void* stream) {
    using namespace rlm;
    if (n_rows == 0) return RLM_OK;
    if (!slot_context || !anchor_active || !slot_weight || !gate || !hidden) {
        set_error("slot_mix_residual: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (n_rows < 0 || slots < 1 || slots > kMixMaxSlots || d_model < 4 || d_model % 4 != 0) {
        set_error("slot_mix_residual: 1..8 slots and a width that is a multiple of 4");
        return RLM_ERR_SHAPE;
    }
    if (!aligned16(slot_context) || !aligned16(hidden)) {
        set_error("slot_mix_residual: contexts and residual rows must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    const int64_t work = static_cast<int64_t>(n_rows) * (d_model / 4);
    const int64_t most = static_cast<int64_t>(sm_count()) * 8;
    const int blocks = static_cast<int>(work / 256 + 1 < most ? work / 256 + 1 : most);
    launch_kernel(slot_mix_residual_kernel, dim3(blocks), dim3(256), 0, stream, slot_context, anchor_active,
                  slot_weight, gate, hidden, n_rows, slots, d_model);
    count_launch();
    return check_launch("slot_mix_residual_kernel");
}
