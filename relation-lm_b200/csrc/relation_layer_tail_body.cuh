// Body of the relation layer tail (see relation_layer_tail.cu for the description) and its host-side
// helpers, shared by the standalone kernel and by the whole-layer kernel that runs the selector
// in front of it (relation_select.cu).
#pragma once

#include <mutex>

#include "rlm_tcgen05.cuh"

namespace rlm {
namespace {

constexpr int kLtThreads = 256;
constexpr int kLtHC = 128;            // hidden columns per CTA
constexpr int kLtMaxPairs = 64;       // (sequence, partner) pairs per cluster
constexpr int kLtMaxSeq = 8;          // sequences per cluster
constexpr int kLtOwn = 32;            // output columns a CTA owns after the reduce-scatter (d / C)
constexpr int kLtOwnStride = 33;      // padded row of the owned raw values (floats)
constexpr uint32_t kLtTermStride = kLtHC * 2 + 16;   // padded row of the staged expanded-cache terms

struct LayerTailArgs {
    const void* expanded_cache;      // [B, T, 2H]
    const void* operand_cache;       // [B, T, R]
    const int32_t* anchor_index;     // [B]
    const int32_t* partner_index;    // [B, K]
    const float* partner_scores;     // [B, K]
    const void* second_bias;         // [d]
    const float* norm_w;             // [d] relation LayerNorm
    const float* norm_b;
    const int64_t* position;
    float* residual;                 // [B, d] in/out
    const float* mix;
    const float* next_w;             // [d] next LayerNorm
    const float* next_b;
    void* normalized;                // [B, d] 16-bit out
    const void* query_weight;        // [NQ, d] or NULL
    void* query;                     // [B, NQ] 16-bit out
    int32_t* status;
    float eps, next_eps;
    int n_seq, k_out, max_t, rdim, hdim, d, n_query, dtype;
    int seqs_per_cluster, cluster;   // cluster = H / 128
};

// Shared-memory plan (byte offsets from the 1024-aligned dynamic base).
struct LtPlan {
    uint32_t wm, w2, p, hid, term_p, term_a, op_a, total;
};

__host__ __device__ inline LtPlan lt_plan(int rdim, int d, int pairs_pad) {
    LtPlan p;
    uint32_t off = 0;
    p.wm = off;     off += static_cast<uint32_t>(rdim / kBK) * kBM * 128u;           // W_m slice; later the W_q slice
    p.w2 = off;     off += static_cast<uint32_t>(d / kBM) * 2u * kBM * 128u;         // W_2 slice; later the partial dump
    p.p = off;      off += static_cast<uint32_t>(rdim / kBK) * pairs_pad * 128u;     // product tile; later the owned raw values
    if (off - p.p < kLtMaxPairs * kLtOwnStride * 4u) off = p.p + kLtMaxPairs * kLtOwnStride * 4u;
    off = (off + 1023u) & ~1023u;
    p.hid = off;    off += 2u * pairs_pad * 128u;                                    // hidden tile; later the normalised rows
    if (off - p.hid < static_cast<uint32_t>(kLtMaxSeq) * d * 2u) off = p.hid + kLtMaxSeq * d * 2u;
    p.term_p = off; off += kLtMaxPairs * kLtTermStride;
    p.term_a = off; off += kLtMaxSeq * kLtTermStride;
    p.op_a = off;   off += kLtMaxSeq * static_cast<uint32_t>(rdim) * 2u;
    p.total = off;
    return p;
}

__device__ __forceinline__ uint32_t lt_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void lt_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `local_addr` (a shared-memory address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t lt_peer(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ float4 lt_ld_peer16(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void lt_st_peer8(uint32_t addr, float x, float y) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ void lt_st_peer2(uint32_t addr, uint16_t v) {
    asm volatile("st.shared::cluster.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}

__device__ __forceinline__ float lt_from16(uint16_t bits, int dtype) {
    return dtype == RLM_BF16 ? bf16_bits_to_float(bits) : __half2float(*reinterpret_cast<const __half*>(&bits));
}
__device__ __forceinline__ uint16_t lt_to16(float v, int dtype) {
    if (dtype == RLM_BF16) { __nv_bfloat16 h = __float2bfloat16_rn(v); return *reinterpret_cast<uint16_t*>(&h); }
    __half h = __float2half_rn(v);
    return *reinterpret_cast<uint16_t*>(&h);
}

// A stage that runs in front of the gathers, in the shared memory behind the weight slices (product
// tile, hidden tile, term and operand rows: unused until the gathers).  The standalone kernel has
// none; the whole-layer kernel runs the selector there.  A stage returns true when it has done the
// dependency wait itself (at the point its own inputs need it).
struct NoStage {
    static constexpr bool kActive = false;
    __device__ __forceinline__ bool operator()(unsigned char*, uint32_t, int, int) const { return false; }
};

template <bool kBf16, typename Stage>
__device__ __forceinline__ void layer_tail_body(const CUtensorMap& map_wm, const CUtensorMap& map_w2,
                                                const LayerTailArgs& a, unsigned char* lt_smem_raw, const Stage& stage) {
    __shared__ __align__(8) unsigned long long bars[4];          // W_m, W_2, product GEMM done, second GEMM done
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    __shared__ int pair_seq_s[kLtMaxPairs];
    __shared__ float weight_s[kLtMaxPairs];
    __shared__ __align__(8) float2 ln_s[kLtMaxPairs];            // (mean, rstd) per pair over the full width

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int dtype = kBf16 ? static_cast<int>(RLM_BF16) : static_cast<int>(RLM_F16);
    const uint32_t rank = lt_cluster_rank();
    const int C = a.cluster, K = a.k_out, R = a.rdim, H = a.hdim, D = a.d;
    const int s0 = blockIdx.y * a.seqs_per_cluster;
    const int nseq = min(a.n_seq - s0, a.seqs_per_cluster);
    const int pairs = nseq * K;
    const int pairs_pad = pairs <= 16 ? 16 : (pairs <= 32 ? 32 : 64);
    const int kblocks = R / kBK, chunks = R / 8, mtiles = D / kBM;
    const int h0 = static_cast<int>(rank) * kLtHC;
    const uint32_t fmt = dtype == RLM_BF16 ? 1u : 0u;
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(pairs_pad >> 3) << 17) |
                           (static_cast<uint32_t>(kBM >> 4) << 24);

    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(lt_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const LtPlan plan = lt_plan(R, D, pairs_pad);
    unsigned char* wm_tile = base + plan.wm;
    unsigned char* w2_tile = base + plan.w2;
    unsigned char* p_tile = base + plan.p;
    unsigned char* hid_tile = base + plan.hid;
    unsigned char* term_p = base + plan.term_p;
    unsigned char* term_a = base + plan.term_a;
    unsigned char* op_a = base + plan.op_a;
    const uint32_t p_kblock = static_cast<uint32_t>(pairs_pad) * 128u;
    // Once every CTA has dumped its partial sums, the term rows are dead in the whole cluster: their
    // place receives the LayerNorm statistics that the CTAs push to one another, [sender][pair]
    // and [sender][sequence] of (mean, M2) over the sender's 32 columns.
    float2* stats_in = reinterpret_cast<float2*>(term_p);
    float2* stats2_in = reinterpret_cast<float2*>(term_a);
    // LayerNorm parameters of this thread's owned column (thread = sequence x owned column at the
    // end of the kernel): parameters, read before the dependency wait
    const int own0 = static_cast<int>(rank) * kLtOwn;
    const float pre_g = a.norm_w[own0 + lane], pre_bt = a.norm_b[own0 + lane];
    const float pre_nw = a.next_w[own0 + lane], pre_nb = a.next_b[own0 + lane];
    const int row_chunks = pairs_pad / 4;                      // 16-byte chunks per row of partial sums: 4, 8 or 16
    const float pre_bias = tid < kLtOwn * row_chunks ? load_scalar(a.second_bias, own0 + tid / row_chunks, dtype) : 0.0f;

    const uint32_t bar_wm = smem_u32(&bars[0]), bar_w2 = smem_u32(&bars[1]);
    const uint32_t bar_d1 = smem_u32(&bars[2]), bar_d2 = smem_u32(&bars[3]);
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_wm) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w2) : "memory");
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bars[i]), 1);
        fence_barrier_init();
        failed = 0;
        // the weight slices do not depend on earlier kernels: requested before the dependency wait
        mbar_expect_tx(bar_wm, static_cast<uint32_t>(kblocks) * kBM * 128u);
        for (int kb = 0; kb < kblocks; ++kb)
            tma_load_2d(smem_u32(wm_tile) + kb * kBM * 128u, &map_wm, kb * kBK, h0, bar_wm);
        mbar_expect_tx(bar_w2, static_cast<uint32_t>(mtiles) * 2u * kBM * 128u);
        for (int mt = 0; mt < mtiles; ++mt)
            for (int kb = 0; kb < 2; ++kb)
                tma_load_2d(smem_u32(w2_tile) + (mt * 2 + kb) * kBM * 128u, &map_w2, h0 + kb * kBK, mt * kBM, bar_w2);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (Stage::kActive) {
        // the stage's results reach the other CTAs of the cluster through global memory, ordered by
        // the cluster barrier
        if (!stage(p_tile, rank, s0, nseq)) griddep_sync();
        lt_cluster_sync();
    } else {
        griddep_sync();
    }
    // the residual stream was written by the previous kernel: requested now, used at the very end
    float pre_res = 0.0f;
    if (warp < nseq) pre_res = a.residual[static_cast<size_t>(s0 + warp) * D + own0 + lane];
    const float pre_mix = *a.mix;

    // ---- gathers.  Four threads share a row to gather: they read its index themselves (one
    // broadcast load) and issue their quarter of its copies at once, so no shared-memory round
    // trip lies between the selector's indices and the first gather.  Partner operand rows go
    // straight into the swizzled product tile; copy group 0 = operand rows (needed by the
    // product GEMM), group 1 = this CTA's 128 columns of the two expanded-cache terms (needed by
    // its epilogue).
    const size_t op_row = static_cast<size_t>(R) * 2, ex_row = static_cast<size_t>(H) * 4;
    const int entry = tid >> 2, quarter = tid & 3;
    int my_pair_row = 0, my_anchor_row = 0;
    if (entry < pairs) {
        const int bl = entry / K;
        const int p = a.partner_index[static_cast<size_t>(s0) * K + entry];
        my_pair_row = min(max(p, 0), a.max_t - 1);            // empty slots carry a sentinel that may be negative
        if (quarter == 0) pair_seq_s[entry] = bl;
        const char* src = static_cast<const char*>(a.operand_cache) +
                          (static_cast<size_t>(s0 + bl) * a.max_t + my_pair_row) * op_row;
        for (int c = quarter; c < chunks; c += 4)
            cp_async16(smem_u32(p_tile) + swizzled(entry, c, p_kblock), src + 16 * c);
    } else if (entry < pairs_pad) {
        for (int c = quarter; c < chunks; c += 4)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};"
                         ::"r"(smem_u32(p_tile) + swizzled(entry, c, p_kblock)), "r"(0) : "memory");
    }
    if (entry < nseq) {
        const int an = a.anchor_index[s0 + entry];
        my_anchor_row = min(max(an, 0), a.max_t - 1);
        const char* src = static_cast<const char*>(a.operand_cache) +
                          (static_cast<size_t>(s0 + entry) * a.max_t + my_anchor_row) * op_row;
        for (int c = quarter; c < chunks; c += 4)
            cp_async16(smem_u32(op_a) + static_cast<uint32_t>(entry * R * 2 + 16 * c), src + 16 * c);
    }
    cp_async_commit();
    if (entry < pairs) {
        const char* src = static_cast<const char*>(a.expanded_cache) +
                          (static_cast<size_t>(s0 + entry / K) * a.max_t + my_pair_row) * ex_row +
                          static_cast<size_t>(H + h0) * 2;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            cp_async16(smem_u32(term_p) + entry * kLtTermStride + 16 * (4 * quarter + i), src + 16 * (4 * quarter + i));
    }
    if (entry < nseq) {
        const char* src = static_cast<const char*>(a.expanded_cache) +
                          (static_cast<size_t>(s0 + entry) * a.max_t + my_anchor_row) * ex_row +
                          static_cast<size_t>(h0) * 2;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            cp_async16(smem_u32(term_a) + entry * kLtTermStride + 16 * (4 * quarter + i), src + 16 * (4 * quarter + i));
    }
    cp_async_commit();
    // softmax weights over the active partner slots of every sequence (needed much later): a few
    // threads of the last warp read the scores themselves while the gathers are in flight
    const int t = static_cast<int>(*a.position);
    const bool bad_position = t < 0 || t >= a.max_t;          // the same in every CTA of the grid
    if (tid >= kLtThreads - kLtMaxSeq && tid - (kLtThreads - kLtMaxSeq) < nseq) {
        const int b = tid - (kLtThreads - kLtMaxSeq);
        const float* sc = a.partner_scores + static_cast<size_t>(s0 + b) * K;
        int k_limit = 32 - __clz(max(t, 0) + 1);               // ceil(log2(t + 2))
        k_limit = min(max(k_limit, 1), K);
        float mx = -1.0e4f;
        for (int k = 0; k < K; ++k)
            if (k < k_limit && sc[k] > -1.0e30f) mx = fmaxf(mx, sc[k]);
        float den = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float e = (k < k_limit && sc[k] > -1.0e30f) ? expf(sc[k] - mx) : 0.0f;
            weight_s[b * K + k] = e;
            den += e;
        }
        den = 1.0f / fmaxf(den, 1.0e-9f);
        for (int k = 0; k < K; ++k) weight_s[b * K + k] *= den;
    }
    cp_async_wait_group1();                                    // the operand rows have arrived
    __syncthreads();
    // products o[a] * o[p], in fp32, rounded to the operand dtype, in place
    for (int i = tid; i < pairs * chunks; i += kLtThreads) {
        const int j = i / chunks, c = i - j * chunks;
        unsigned char* at = p_tile + swizzled(j, c, p_kblock);
        float pv[8], av[8];
        unpack8(*reinterpret_cast<const uint4*>(at), dtype, pv);
        unpack8(*reinterpret_cast<const uint4*>(op_a + pair_seq_s[j] * R * 2 + 16 * c), dtype, av);
        uint4 out;
        out.x = pack2(pv[0] * av[0], pv[1] * av[1], dtype);
        out.y = pack2(pv[2] * av[2], pv[3] * av[3], dtype);
        out.z = pack2(pv[4] * av[4], pv[5] * av[5], dtype);
        out.w = pack2(pv[6] * av[6], pv[7] * av[7], dtype);
        *reinterpret_cast<uint4*>(at) = out;
    }
    fence_proxy_async();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t tmem_d2 = tmem_base + 64u;                 // second GEMM: mtiles x pairs_pad columns from column 64

    // ---- product GEMM: D1[hidden column, pair] = W_m slice x products^T
    if (tid == 0) {
        if (mbar_wait(bar_wm, 0)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = 0; kb < kblocks; ++kb) {
                const uint64_t dw = smem_desc_sw128(smem_u32(wm_tile) + kb * kBM * 128u);
                const uint64_t dp = smem_desc_sw128(smem_u32(p_tile) + kb * p_kblock);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)
                    umma_f16(tmem_base, dw + 2 * kk, dp + 2 * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
        } else {
            failed = 1;
        }
        umma_commit(bar_d1);
    }
    __syncwarp();
    if (!mbar_wait(bar_d1, 0)) failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    const int nq_own = a.query_weight ? a.n_query / C : 0;
    int tpo = 16;                                              // threads per projection output: 2 .. 16
    while (tpo > 2 && (nseq * nq_own * tpo > kLtThreads || (D / 8) / tpo < 2)) tpo >>= 1;
    const uint32_t wq_stride = static_cast<uint32_t>(D) * 2u + 16u * static_cast<uint32_t>(tpo);
    cp_async_wait_all();                                       // the expanded-cache terms have arrived
    __syncthreads();

    // ---- epilogue of the product GEMM: + expanded-cache terms, GELU, hidden slice as the K-major
    // B tile of the second GEMM (row = pair, K = this CTA's hidden columns).  Warps 0-3 take the
    // first half of the pair columns, warps 4-7 the second half (eight columns at a time).
    const int half_cols = pairs_pad >> 1;                     // 8, 16 or 32 pair columns per warp half
    {
        const int hc = 32 * (warp & 3) + lane;                // hidden column == TMEM lane
        const int col0 = half_cols * (warp >> 2);
        const uint32_t lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        const unsigned char* ta = term_a + hc * 2;
        const unsigned char* tp = term_p + hc * 2;
        unsigned char* hrow = hid_tile + static_cast<uint32_t>(hc >> 6) * p_kblock + (hc & 7) * 2;
        const int hchunk = (hc >> 3) & 7;
        for (int c = col0; c < col0 + half_cols; c += 8) {
            uint32_t v[8];
            tmem_ld8(tmem_base + lane_base + c, v);
            float term[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int pr = c + j;
                term[j] = 0.0f;
                if (pr < pairs)
                    term[j] = lt_from16(*reinterpret_cast<const uint16_t*>(ta + pair_seq_s[pr] * kLtTermStride), dtype) +
                              lt_from16(*reinterpret_cast<const uint16_t*>(tp + pr * kLtTermStride), dtype);
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int pr = c + j;
                const float x = pr < pairs ? gelu_tc(__uint_as_float(v[j]) + term[j]) : 0.0f;
                *reinterpret_cast<uint16_t*>(hrow + (pr >> 3) * 1024 + (pr & 7) * 128 + ((hchunk ^ (pr & 7)) << 4)) = lt_to16(x, dtype);
            }
        }
    }
    fence_proxy_async();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- second GEMM, split over the cluster along the hidden width:
    // D2[output row, pair] (partial) = W_2[:, this CTA's hidden columns] x hidden slice^T
    if (tid == 0) {
        if (mbar_wait(bar_w2, 0)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int mt = 0; mt < mtiles; ++mt)
                for (int kb = 0; kb < 2; ++kb) {
                    const uint64_t dw = smem_desc_sw128(smem_u32(w2_tile) + (mt * 2 + kb) * kBM * 128u);
                    const uint64_t dh = smem_desc_sw128(smem_u32(hid_tile) + kb * p_kblock);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk)
                        umma_f16(tmem_d2 + static_cast<uint32_t>(mt * pairs_pad), dw + 2 * kk, dh + 2 * kk, idesc,
                                 (kb > 0 || kk > 0) ? 1u : 0u);
                }
        } else {
            failed = 1;
        }
        umma_commit(bar_d2);
    }
    __syncwarp();
    // the W_m slice was consumed by the first GEMM: while the second one runs, its place takes this
    // CTA's rows of the query-projection weight (rows padded by one 16-byte chunk per cooperating
    // thread: conflict-free reads in the projection below)
    if (nq_own > 0) {
        const int w_chunks = D / 8;
        for (int i = tid; i < nq_own * w_chunks; i += kLtThreads) {
            const int j = i / w_chunks, c = i - j * w_chunks;
            cp_async16(smem_u32(wm_tile) + j * wq_stride + 16 * c,
                       static_cast<const char*>(a.query_weight) +
                           (static_cast<size_t>(rank) * nq_own + j) * D * 2 + 16 * c);
        }
        cp_async_commit();
    }
    if (!mbar_wait(bar_d2, 0)) failed = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    // ---- dump the partial raw^T [d, pairs_pad] (fp32) over the consumed W_2 slice; 16-byte chunk
    // j of row r sits at chunk j ^ (r mod chunks per row): conflict-free for writers and readers
    const uint32_t part_row = static_cast<uint32_t>(pairs_pad) * 4u;
    {
        const int lr = 32 * (warp & 3) + lane;
        const int col0 = half_cols * (warp >> 2);
        const uint32_t lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        for (int mt = 0; mt < mtiles; ++mt) {
            const int r = mt * kBM + lr;
            for (int c = col0; c < col0 + half_cols; c += 8) {
                uint32_t v[8];
                tmem_ld8(tmem_d2 + lane_base + static_cast<uint32_t>(mt * pairs_pad + c), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int ch = ((c >> 2) + q) ^ (r & (row_chunks - 1));
                    *reinterpret_cast<uint4*>(w2_tile + r * part_row + ch * 16) =
                        make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    lt_cluster_sync();                                         // (1) every CTA's partial is in its shared memory
    // every warp has read its accumulators: the tensor memory goes back now, off the kernel's exit path
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }

    // ---- reduce-scatter: this CTA owns output rows [own0, own0 + 32); partial sums are pulled
    // from the CTAs in rank order, so the result does not depend on timing
    float* own_raw = reinterpret_cast<float*>(p_tile);        // [pair][kLtOwnStride]
    {
        const uint32_t part_base = smem_u32(w2_tile);
        for (int i = tid; i < kLtOwn * row_chunks; i += kLtThreads) {
            const int r = i / row_chunks, j = i - r * row_chunks;
            const int row = own0 + r;
            const uint32_t off = static_cast<uint32_t>(row) * part_row + static_cast<uint32_t>((j ^ (row & (row_chunks - 1))) * 16);
            float4 v[16];
#pragma unroll
            for (int q = 0; q < 16; ++q)
                v[q] = q < C ? lt_ld_peer16(lt_peer(part_base, static_cast<uint32_t>(q)) + off)
                             : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int q = 0; q < 16; ++q) { acc.x += v[q].x; acc.y += v[q].y; acc.z += v[q].z; acc.w += v[q].w; }
            const float bias = i == tid ? pre_bias : load_scalar(a.second_bias, row, dtype);
            const int pr = 4 * j;
            own_raw[(pr + 0) * kLtOwnStride + r] = acc.x + bias;
            own_raw[(pr + 1) * kLtOwnStride + r] = acc.y + bias;
            own_raw[(pr + 2) * kLtOwnStride + r] = acc.z + bias;
            own_raw[(pr + 3) * kLtOwnStride + r] = acc.w + bias;
        }
    }
    __syncthreads();

    // ---- LayerNorm statistics of every pair over the full width: (mean, M2) of this CTA's 32
    // columns, combined over the cluster (equal counts: Chan's parallel variance)
    {
        const int pr = tid >> 2, q = tid & 3;                  // four threads per pair, eight columns each
        float x[8], sum = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            x[i] = pr < pairs ? own_raw[pr * kLtOwnStride + 8 * q + i] : 0.0f;
            sum += x[i];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float mean = sum * (1.0f / kLtOwn);
        float m2 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float dv = x[i] - mean; m2 = fmaf(dv, dv, m2); }
        m2 += __shfl_xor_sync(0xffffffffu, m2, 1);
        m2 += __shfl_xor_sync(0xffffffffu, m2, 2);
        // pushed to every CTA of the cluster (the four threads of a pair share the receivers), so that
        // nobody waits for a remote load after the barrier
        if (pr < pairs) {
            const uint32_t at = smem_u32(&stats_in[rank * kLtMaxPairs + pr]);
            for (int i = 0; i < (C >> 2); ++i) lt_st_peer8(lt_peer(at, static_cast<uint32_t>(q * (C >> 2) + i)), mean, m2);
        }
    }
    lt_cluster_sync();                                         // (2) every CTA's pair statistics are written
    {
        // four lanes per pair, each reading the statistics of C / 4 CTAs (C = 4, 8 or 16)
        const int pr = tid >> 2, q = tid & 3, per = C >> 2;
        float2 st[4];
        float msum = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            st[i] = make_float2(0.0f, 0.0f);
            if (i < per && pr < pairs)
                st[i] = stats_in[(q * per + i) * kLtMaxPairs + pr];
            msum += st[i].x;
        }
        msum += __shfl_xor_sync(0xffffffffu, msum, 1);
        msum += __shfl_xor_sync(0xffffffffu, msum, 2);
        const float mean = msum / static_cast<float>(C);
        float m2 = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (i < per) { const float dm = st[i].x - mean; m2 += st[i].y + static_cast<float>(kLtOwn) * dm * dm; }
        m2 += __shfl_xor_sync(0xffffffffu, m2, 1);
        m2 += __shfl_xor_sync(0xffffffffu, m2, 2);
        if (q == 0 && pr < pairs) ln_s[pr] = make_float2(mean, rsqrtf(m2 / static_cast<float>(D) + a.eps));
    }
    __syncthreads();

    // ---- context, residual update and the next LayerNorm: thread (sequence = warp, owned column = lane)
    const int bl = warp, col = own0 + lane;
    const bool live = bl < nseq && !bad_position;
    float hval = 0.0f;
    if (live) {
        const float g = pre_g, bt = pre_bt;
        float ctx = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float wk = weight_s[bl * K + k];
            if (wk == 0.0f) continue;                          // inactive slots contribute nothing
            const float2 ms = ln_s[bl * K + k];
            const float x = own_raw[(bl * K + k) * kLtOwnStride + lane];
            ctx = fmaf(wk, fmaf((x - ms.x) * ms.y, g, bt), ctx);
        }
        float* res = a.residual + static_cast<size_t>(s0 + bl) * D + col;
        hval = fmaf(pre_mix, ctx, pre_res);
        *res = hval;
    }
    {
        const float mean = warp_sum(hval) * (1.0f / kLtOwn);
        const float dv = hval - mean;
        const float m2 = warp_sum(dv * dv);
        if (lane < C && bl < kLtMaxSeq)
            lt_st_peer8(lt_peer(smem_u32(&stats2_in[rank * kLtMaxSeq + bl]), static_cast<uint32_t>(lane)), mean, m2);
    }
    lt_cluster_sync();                                         // (3) every CTA's residual statistics are written
    {
        float2 st = make_float2(0.0f, 0.0f);
        if (lane < C && bl < nseq) st = stats2_in[lane * kLtMaxSeq + bl];
        const float mean = warp_sum(st.x) / static_cast<float>(C);
        const float dm = st.x - mean;
        const float m2 = warp_sum(lane < C ? st.y + static_cast<float>(kLtOwn) * dm * dm : 0.0f);
        const float rstd = rsqrtf(m2 / static_cast<float>(D) + a.next_eps);
        if (live) {
            const uint16_t nv = lt_to16(fmaf((hval - mean) * rstd, pre_nw, pre_nb), dtype);
            static_cast<uint16_t*>(a.normalized)[static_cast<size_t>(s0 + bl) * D + col] = nv;
            if (nq_own > 0) {
                // the normalised rows go to every CTA of the cluster for its share of the projection
                const uint32_t at = smem_u32(hid_tile) + static_cast<uint32_t>((bl * D + col) * 2);
                for (int p = 0; p < C; ++p) lt_st_peer2(lt_peer(at, static_cast<uint32_t>(p)), nv);
            }
        }
    }
    cp_async_wait_all();                                       // this thread's pieces of the W_q slice
    lt_cluster_sync();                                         // (4) normalised rows everywhere; no remote access after this

    // ---- this CTA's share of the next query projection: outputs [rank * nq_own, + nq_own) of every
    // sequence, two threads per (sequence, output), fp32 accumulation
    if (nq_own > 0 && !bad_position) {
        const int n_out = nseq * nq_own, per_pass = kLtThreads / tpo, my_chunks = (D / 8) / tpo;
        const int part = tid & (tpo - 1);
        for (int o0 = 0; o0 < n_out; o0 += per_pass) {        // whole warps walk the loop together
            const int o = o0 + tid / tpo;
            const bool in = o < n_out;
            const int b = in ? o / nq_own : 0, j = in ? o - b * nq_own : 0;
            const unsigned char* wrow = wm_tile + j * wq_stride;
            const unsigned char* xrow = hid_tile + (b * D) * 2;
            float acc0 = 0.0f, acc1 = 0.0f;
            for (int i = 0; i < my_chunks; i += 2) {
                float wf[8], xf[8], wg[8], xg[8];
                const int c = part + tpo * i, c2 = part + tpo * (i + 1);
                unpack8(*reinterpret_cast<const uint4*>(wrow + 16 * c), dtype, wf);
                unpack8(*reinterpret_cast<const uint4*>(xrow + 16 * c), dtype, xf);
                unpack8(*reinterpret_cast<const uint4*>(wrow + 16 * c2), dtype, wg);
                unpack8(*reinterpret_cast<const uint4*>(xrow + 16 * c2), dtype, xg);
#pragma unroll
                for (int e = 0; e < 8; ++e) { acc0 = fmaf(wf[e], xf[e], acc0); acc1 = fmaf(wg[e], xg[e], acc1); }
            }
            float acc = acc0 + acc1;
            for (int sh = 1; sh < tpo; sh <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
            if (in && part == 0)
                static_cast<uint16_t*>(a.query)[static_cast<size_t>(s0 + b) * a.n_query + rank * nq_own + j] = lt_to16(acc, dtype);
        }
    }
    if (tid == 0 && a.status) {
        if (*reinterpret_cast<volatile int*>(&failed)) atomicOr(a.status, RLM_DEV_TIMEOUT);
        if (bad_position) atomicOr(a.status, RLM_DEV_POSITION);
    }
}

int lt_validate(const LayerTailArgs& a) {
    if (a.n_seq < 1 || a.k_out < 1 || a.k_out > kLtMaxPairs || a.max_t < 1) {
        set_error("relation_layer_tail: sizes must be positive and K at most 64");
        return RLM_ERR_SHAPE;
    }
    if (a.dtype != RLM_BF16 && a.dtype != RLM_F16) {
        set_error("relation_layer_tail: caches and weights must share bfloat16 or float16");
        return RLM_ERR_UNSUPPORTED;
    }
    if (a.hdim % kLtHC != 0 || (a.hdim / kLtHC != 4 && a.hdim / kLtHC != 8 && a.hdim / kLtHC != 16) ||
        a.d % kBM != 0 || a.d > 512 || a.d / (a.hdim / kLtHC) != kLtOwn || a.rdim % kBK != 0 || a.rdim > 256) {
        set_error("relation_layer_tail: needs H = 4 d with d in {128, 256, 512} and R a multiple of 64 up to 256");
        return RLM_ERR_UNSUPPORTED;
    }
    const int cluster = a.hdim / kLtHC;
    if (a.query_weight && (a.n_query < cluster || a.n_query % (16 * cluster) != 0 || a.n_query / cluster > 64 || !a.query ||
                           static_cast<size_t>(a.n_query / cluster) * (a.d * 2 + 256) > static_cast<size_t>(a.rdim / kBK) * kBM * 128)) {
        set_error("relation_layer_tail: query projection width must be a multiple of 16 outputs per CTA (H / 128 CTAs), at most 64 each");
        return RLM_ERR_UNSUPPORTED;
    }
    if (lt_plan(a.rdim, a.d, kLtMaxPairs).total + 1024 > static_cast<uint32_t>(kSmemDynamicLimit)) {
        set_error("relation_layer_tail: the weight slices exceed 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    return RLM_OK;
}

int lt_prepare(const void* kernel, int cluster) {
    // clusters of more than 8 CTAs are an opt-in of every kernel, on every device
    static std::mutex guard;
    static const void* done_kernel[64 * 4] = {};
    static int done_device[64 * 4] = {};
    static int done_count = 0;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return RLM_ERR_LAUNCH; }
    int rc = allow_large_smem(kernel, kSmemPerCta);
    if (rc != RLM_OK) return rc;
    std::lock_guard<std::mutex> lock(guard);
    for (int i = 0; i < done_count; ++i)
        if (done_kernel[i] == kernel && done_device[i] == device) return RLM_OK;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        set_error("relation_layer_tail: clusters of 16 CTAs are not available on this device");
        return RLM_ERR_UNSUPPORTED;
    }
    if (done_count < 64 * 4) {
        done_kernel[done_count] = kernel;
        done_device[done_count] = device;
        ++done_count;
    }
    (void)cluster;
    return RLM_OK;
}


}  // namespace
}  // namespace rlm
