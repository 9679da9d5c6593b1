// Routed anchor/partner selection for sm_100a.
//
// One CTA per query row.  Everything a row needs is staged in shared memory by
// untiled bulk (TMA) copies that complete on mbarriers: both streams' block
// statistics and local key windows are requested at kernel entry; the chosen
// remote blocks and the partner-anchor cache row are requested as soon as the
// indices that address them are known.  Scores are computed from shared memory
// with 8 lanes per 64-wide row (16-byte reads, bank-conflict free for 16-bit
// caches) in the canonical order documented in rlm_common.cuh, so the selected
// indices do not depend on the launch geometry.
//
// Semantics follow src/relation_lm/kernels/relation_select.py:50-308 and
// src/relation_lm/kernels/triton_select.py:23-252 of the reference project.

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kD = 64;        // exact-score width == router heads * head width
constexpr int kHeads = 4;

enum Mode { kPacked = 0, kAnchorOnly = 1, kPartnerOnly = 2 };

struct SelectArgs {
    const void* anchor_query;
    const void* anchor_keys;
    const void* anchor_router_query;
    const void* anchor_mean;
    const void* anchor_std;
    const void* anchor_gamma;
    const void* anchor_bias;
    const void* partner_base;            // packed: [N,128]; partner-only: exact query [N,64]
    const void* partner_router_query;    // partner-only: router query [N,64]
    const void* partner_anchor_cache;
    const void* partner_keys;
    const void* partner_mean;
    const void* partner_std;
    const void* partner_gamma;
    const void* partner_bias;
    const int64_t* position;
    const int32_t* row_batch;
    const int32_t* row_position;
    const int32_t* anchor_index_in;      // partner-only
    int32_t* out_anchor;
    float* out_anchor_score;
    int32_t* out_partner;
    float* out_partner_score;
    int32_t* status;
    int64_t aq_stride, arq_stride, pbase_stride, prq_stride;   // query row strides, elements
    int n_rows, n_seq, max_t, n_blocks, block_size, buckets;
    int local_window, top_blocks, k_out, strict_valid;
    int query_dtype, key_dtype, stats_dtype, param_dtype;
    int mode;
};

// Shared-memory plan (byte offsets from the dynamic shared base).
struct Plan {
    int a_mean, a_std, p_mean, p_std;   // [NB,64] stats elements
    int a_local, p_local;               // [L,64] key elements
    int remote;                         // [TOP*BS,64] key elements (anchor phase, then partner phase)
    int pa_row;                         // [128] key elements
    int queries;                        // f32: aq[64] arq[64] pq[64] prq[64]
    int params;                         // f32: softplus(gamma) a[4] p[4], bias a[4*buckets] p[4*buckets]
    int block_scores;                   // f32 [NB]
    int cand;                           // f32 [L + TOP*BS]
    int sel;                            // int [3*TOP]: block, usable, valid row count
    int bars;                           // 5 mbarriers
    int total;
};

__host__ __device__ inline int align16(int x) { return (x + 15) & ~15; }

__host__ __device__ inline Plan make_plan(int nb, int bs, int local, int top, int buckets,
                                          int key_size, int stats_size, int mode) {
    Plan p;
    int off = 0;
    int stats_bytes = nb * kD * stats_size;
    int local_bytes = local * kD * key_size;
    bool anchor = mode != kPartnerOnly, partner = mode != kAnchorOnly;
    p.a_mean = off; off += anchor ? stats_bytes : 0;
    p.a_std = off; off += anchor ? stats_bytes : 0;
    p.p_mean = off; off += partner ? stats_bytes : 0;
    p.p_std = off; off += partner ? stats_bytes : 0;
    p.a_local = off; off += anchor ? local_bytes : 0;
    p.p_local = off; off += partner ? local_bytes : 0;
    p.remote = off; off += top * bs * kD * key_size;
    p.pa_row = off; off += 2 * kD * key_size;
    p.queries = off; off += 4 * kD * 4;
    p.params = off; off += align16((8 + 8 * buckets) * 4);
    p.block_scores = off; off += align16(nb * 4);
    p.cand = off; off += align16((local + top * bs) * 4);
    p.sel = off; off += align16(3 * (top > 0 ? top : 1) * 4);
    p.bars = off; off += 5 * 8;
    p.total = align16(off);
    return p;
}

// Scores `n_rows` staged key rows against the query held in shared memory
// (f32 [64]).  Row r of `rows` is candidate slot `slot0 + r`; rows at or past
// `n_valid`, and the row whose position equals `exclude`, score -inf.
__device__ __forceinline__ void score_rows(const unsigned char* rows, int key_dtype, int n_rows,
                                           int n_valid_first, int n_valid_end, int pos0,
                                           int exclude, const float* query, float* cand,
                                           int slot0) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = lane & 7, sub = lane >> 3;
    const int row_bytes = kD * (key_dtype == RLM_F32 ? 4 : 2);
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = query[8 * j + i];
    for (int base = warp * 4; base < n_rows; base += 4 * kWarps) {
        int r = base + sub;
        bool valid = r < n_rows && r >= n_valid_first && r < n_valid_end && (pos0 + r) != exclude;
        float acc = 0.0f;
        if (valid) {
            float k[8];
            load8(rows + static_cast<size_t>(r) * row_bytes, 8 * j, key_dtype, k);
            acc = seg8(k, q);
        }
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
        if (j == 0 && r < n_rows) cand[slot0 + r] = valid ? __fmul_rn(acc, 0.125f) : kNegInf;
    }
}

// Block scores of the first `n_complete` blocks (the others are not eligible).
__device__ __forceinline__ void score_blocks(const unsigned char* mean, const unsigned char* stdv,
                                             int stats_dtype, int nb, int n_complete, int bs,
                                             int t, int ls, int strict, int buckets,
                                             const float* rq, const float* softplus,
                                             const float* bias, float* out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = lane & 7, sub = lane >> 3, head = j >> 1;
    const int row_bytes = kD * (stats_dtype == RLM_F32 ? 4 : 2);
    float q[8], aq[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { q[i] = rq[8 * j + i]; aq[i] = fabsf(q[i]); }
    const float sp = softplus[head];
    for (int n = threadIdx.x; n < nb; n += kThreads)
        if (n >= n_complete) out[n] = kNegInf;
    for (int base = warp * 4; base < n_complete; base += 4 * kWarps) {
        int n = base + sub;
        bool live = n < n_complete;
        float md = 0.0f, sd = 0.0f;
        int end = (n + 1) * bs - 1;
        if (live) {
            float m[8], s[8];
            load8(mean + static_cast<size_t>(n) * row_bytes, 8 * j, stats_dtype, m);
            load8(stdv + static_cast<size_t>(n) * row_bytes, 8 * j, stats_dtype, s);
            md = seg8(m, q);
            sd = seg8(s, aq);
        }
        md = __fadd_rn(md, __shfl_xor_sync(0xffffffffu, md, 1));
        sd = __fadd_rn(sd, __shfl_xor_sync(0xffffffffu, sd, 1));
        int dist = t - end;
        if (dist < 0) dist = 0;
        int bucket = 31 - __clz(dist + 1);
        if (bucket > buckets - 1) bucket = buckets - 1;
        float sh = __fadd_rn(__fmul_rn(__fadd_rn(md, __fmul_rn(sp, sd)), 0.25f),
                             live ? bias[head * buckets + bucket] : 0.0f);
        const int g = lane & ~7;
        float acc = __shfl_sync(0xffffffffu, sh, g);
#pragma unroll
        for (int h = 1; h < kHeads; ++h) {
            float s = __shfl_sync(0xffffffffu, sh, g + 2 * h);
            float mx = fmaxf(acc, s);
            acc = __fadd_rn(mx, canon_log(__fadd_rn(canon_exp(__fsub_rn(acc, mx)),
                                                    canon_exp(__fsub_rn(s, mx)))));
        }
        if (j == 0 && live) {
            bool eligible = !strict || end < ls;
            out[n] = eligible ? acc : kNegInf;
        }
    }
}

// Warp 0: pick `top` blocks by descending score (ties: lowest index), record
// (block, usable, number of rows before the local window) per rank.
__device__ __forceinline__ void pick_blocks(float* scores, int nb, int top, int bs, int ls,
                                            int* sel) {
    const int lane = threadIdx.x & 31;
    for (int r = 0; r < top; ++r) {
        float bv = kNegInf;
        int bi = 0x7fffffff;
        for (int n = lane; n < nb; n += 32) {
            float v = scores[n];
            if (v > bv || bi == 0x7fffffff) { bv = v; bi = n; }
        }
        warp_argmax_low(bv, bi);
        if (bi == 0x7fffffff) bi = 0;
        if (lane == 0) {
            int usable = bv > -1.0e30f;
            int rows = ls - bi * bs;
            rows = rows < 0 ? 0 : (rows > bs ? bs : rows);
            sel[3 * r] = bi;
            sel[3 * r + 1] = usable;
            sel[3 * r + 2] = usable ? rows : 0;
            scores[bi] = kNegInf;
        }
        __syncwarp();
    }
}

__global__ void __launch_bounds__(kThreads) relation_select_kernel(const SelectArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = a.row_batch ? a.row_batch[row] : row;
    const int t = a.row_position ? a.row_position[row] : static_cast<int>(*a.position);
    if (b < 0 || b >= a.n_seq || t < 0 || t >= a.max_t) {
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
        return;
    }
    const int nb = a.n_blocks, bs = a.block_size, L = a.local_window, top = a.top_blocks;
    const int ks = a.key_dtype == RLM_F32 ? 4 : 2, ss = a.stats_dtype == RLM_F32 ? 4 : 2;
    const Plan p = make_plan(nb, bs, L, top, a.buckets, ks, ss, a.mode);
    const bool do_anchor = a.mode != kPartnerOnly, do_partner = a.mode != kAnchorOnly;

    float* queries = reinterpret_cast<float*>(smem + p.queries);
    float* aq = queries, *arq = queries + kD, *pq = queries + 2 * kD, *prq = queries + 3 * kD;
    float* params = reinterpret_cast<float*>(smem + p.params);
    float* sp_a = params, *sp_p = params + 4, *bias_a = params + 8, *bias_p = bias_a + 4 * a.buckets;
    float* bscore = reinterpret_cast<float*>(smem + p.block_scores);
    float* cand = reinterpret_cast<float*>(smem + p.cand);
    int* sel = reinterpret_cast<int*>(smem + p.sel);
    const uint32_t bars = smem_u32(smem + p.bars);
    const uint32_t bar_a = bars, bar_p = bars + 8, bar_ra = bars + 16, bar_row = bars + 24,
                   bar_rp = bars + 32;

    const int ls = max(t - L + 1, 0);
    const int first_local = ls - (t - L + 1);       // first valid slot of the local window
    const int n_local = t - ls + 1;
    const int n_complete = min((t + 1) / bs, nb);
    const size_t key_row = static_cast<size_t>(kD) * ks, stat_row = static_cast<size_t>(kD) * ss;
    const size_t seq_keys = static_cast<size_t>(b) * a.max_t * key_row;
    const size_t seq_stats = static_cast<size_t>(b) * nb * stat_row;

    if (tid == 0) {
        for (int i = 0; i < 5; ++i) mbar_init(bars + 8 * i, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0) {
        const uint32_t sbytes = static_cast<uint32_t>(n_complete * stat_row);
        const uint32_t lbytes = static_cast<uint32_t>(n_local * key_row);
        const size_t loff = seq_keys + static_cast<size_t>(ls) * key_row;
        const uint32_t ldst = static_cast<uint32_t>(first_local * key_row);
        if (do_anchor) {
            mbar_expect_tx(bar_a, 2 * sbytes + lbytes);
            if (sbytes) {
                bulk_g2s(smem_u32(smem + p.a_mean), static_cast<const char*>(a.anchor_mean) + seq_stats, sbytes, bar_a);
                bulk_g2s(smem_u32(smem + p.a_std), static_cast<const char*>(a.anchor_std) + seq_stats, sbytes, bar_a);
            }
            bulk_g2s(smem_u32(smem + p.a_local) + ldst, static_cast<const char*>(a.anchor_keys) + loff, lbytes, bar_a);
        }
        if (do_partner) {
            mbar_expect_tx(bar_p, 2 * sbytes + lbytes);
            if (sbytes) {
                bulk_g2s(smem_u32(smem + p.p_mean), static_cast<const char*>(a.partner_mean) + seq_stats, sbytes, bar_p);
                bulk_g2s(smem_u32(smem + p.p_std), static_cast<const char*>(a.partner_std) + seq_stats, sbytes, bar_p);
            }
            bulk_g2s(smem_u32(smem + p.p_local) + ldst, static_cast<const char*>(a.partner_keys) + loff, lbytes, bar_p);
        }
    }
    // Small operands through ordinary loads while the bulk copies fly.
    if (do_anchor) {
        if (tid < kD) aq[tid] = load_scalar(a.anchor_query, row * a.aq_stride + tid, a.query_dtype);
        else if (tid < 2 * kD) arq[tid - kD] = load_scalar(a.anchor_router_query, row * a.arq_stride + tid - kD, a.query_dtype);
    }
    if (a.mode == kPartnerOnly) {
        if (tid < kD) pq[tid] = load_scalar(a.partner_base, row * a.pbase_stride + tid, a.query_dtype);
        else if (tid < 2 * kD) prq[tid - kD] = load_scalar(a.partner_router_query, row * a.prq_stride + tid - kD, a.query_dtype);
    }
    if (tid >= 2 * kD && tid < 2 * kD + 8) {
        int h = (tid - 2 * kD) & 3;
        bool partner_side = tid - 2 * kD >= 4;
        const void* g = partner_side ? a.partner_gamma : a.anchor_gamma;
        if (g) {
            float gamma = load_scalar(g, h, a.param_dtype);
            (partner_side ? sp_p : sp_a)[h] = canon_log(__fadd_rn(1.0f, canon_exp(gamma)));
        }
    }
    for (int i = tid; i < 4 * a.buckets; i += kThreads) {
        if (do_anchor) bias_a[i] = load_scalar(a.anchor_bias, i, a.param_dtype);
        if (do_partner) bias_p[i] = load_scalar(a.partner_bias, i, a.param_dtype);
    }
    __syncthreads();

    int anchor_pos = 0;
    if (do_anchor) {
        bool ok = mbar_wait(bar_a, 0);
        if (__syncthreads_or(!ok)) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
            return;
        }
        score_blocks(smem + p.a_mean, smem + p.a_std, a.stats_dtype, nb, n_complete, bs, t, ls,
                     a.strict_valid, a.buckets, arq, sp_a, bias_a, bscore);
        score_rows(smem + p.a_local, a.key_dtype, L, first_local, L, t - L + 1, -1, aq, cand, 0);
        __syncthreads();
        if (warp == 0) {
            pick_blocks(bscore, nb, top, bs, ls, sel);
            if (lane == 0 && top > 0) {
                fence_proxy_async();
                uint32_t total = 0;
                for (int r = 0; r < top; ++r) total += static_cast<uint32_t>(sel[3 * r + 2] * key_row);
                mbar_expect_tx(bar_ra, total);
                for (int r = 0; r < top; ++r)
                    if (sel[3 * r + 2] > 0)
                        bulk_g2s(smem_u32(smem + p.remote) + static_cast<uint32_t>(r * bs * key_row),
                                 static_cast<const char*>(a.anchor_keys) + seq_keys + static_cast<size_t>(sel[3 * r]) * bs * key_row,
                                 static_cast<uint32_t>(sel[3 * r + 2] * key_row), bar_ra);
            }
        }
        __syncthreads();
        if (top > 0) {
            ok = mbar_wait(bar_ra, 0);
            if (__syncthreads_or(!ok)) {
                if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
                return;
            }
            for (int r = 0; r < top; ++r)
                score_rows(smem + p.remote + static_cast<size_t>(r) * bs * key_row, a.key_dtype, bs, 0,
                           sel[3 * r + 2], sel[3 * r] * bs, -1, aq, cand, L + r * bs);
            __syncthreads();
        }
        // Every warp reduces redundantly so that all threads know the anchor.
        float best = kNegInf;
        int best_c = 0x7fffffff;
        for (int c = lane; c < L; c += 32) {
            float v = cand[c];
            if (v > best || best_c == 0x7fffffff) { best = v; best_c = c; }
        }
        warp_argmax_low(best, best_c);
        anchor_pos = t - L + 1 + best_c;
        for (int r = 0; r < top; ++r) {
            float cv = kNegInf;
            int co = 0x7fffffff;
            for (int o = lane; o < bs; o += 32) {
                float v = cand[L + r * bs + o];
                if (v > cv || co == 0x7fffffff) { cv = v; co = o; }
            }
            warp_argmax_low(cv, co);
            if (co == 0x7fffffff) co = 0;
            int cpos = sel[3 * r] * bs + co;
            if (cv > best || (cv == best && cpos < anchor_pos)) { best = cv; anchor_pos = cpos; }
        }
        if (tid == 0) {
            a.out_anchor[row] = anchor_pos;
            a.out_anchor_score[row] = best;
        }
        if (!do_partner) return;
        __syncthreads();   // all reads of cand / sel / remote are done before they are reused
        if (tid == 0) {
            mbar_expect_tx(bar_row, static_cast<uint32_t>(2 * key_row));
            bulk_g2s(smem_u32(smem + p.pa_row),
                     static_cast<const char*>(a.partner_anchor_cache) + (static_cast<size_t>(b) * a.max_t + anchor_pos) * 2 * key_row,
                     static_cast<uint32_t>(2 * key_row), bar_row);
        }
        bool ok_row = mbar_wait(bar_row, 0);
        if (__syncthreads_or(!ok_row)) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
            return;
        }
        if (tid < 2 * kD) {
            float base = load_scalar(a.partner_base, row * a.pbase_stride + tid, a.query_dtype);
            float add = load_scalar(smem + p.pa_row, tid, a.key_dtype);
            pq[tid] = __fadd_rn(base, add);   // pq[64..127] is prq
        }
    } else {
        anchor_pos = a.anchor_index_in[row];
    }

    bool okp = mbar_wait(bar_p, 0);
    if (__syncthreads_or(!okp)) {   // also publishes pq / prq
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
        return;
    }
    score_blocks(smem + p.p_mean, smem + p.p_std, a.stats_dtype, nb, n_complete, bs, t, ls,
                 a.strict_valid, a.buckets, prq, sp_p, bias_p, bscore);
    __syncthreads();
    if (warp == 0) {
        pick_blocks(bscore, nb, top, bs, ls, sel);
        if (lane == 0 && top > 0) {
            fence_proxy_async();
            uint32_t total = 0;
            for (int r = 0; r < top; ++r) total += static_cast<uint32_t>(sel[3 * r + 2] * key_row);
            mbar_expect_tx(bar_rp, total);
            for (int r = 0; r < top; ++r)
                if (sel[3 * r + 2] > 0)
                    bulk_g2s(smem_u32(smem + p.remote) + static_cast<uint32_t>(r * bs * key_row),
                             static_cast<const char*>(a.partner_keys) + seq_keys + static_cast<size_t>(sel[3 * r]) * bs * key_row,
                             static_cast<uint32_t>(sel[3 * r + 2] * key_row), bar_rp);
        }
    }
    score_rows(smem + p.p_local, a.key_dtype, L, first_local, L, t - L + 1, anchor_pos, pq, cand, 0);
    __syncthreads();
    if (top > 0) {
        bool ok = mbar_wait(bar_rp, 0);
        if (__syncthreads_or(!ok)) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
            return;
        }
        for (int r = 0; r < top; ++r)
            score_rows(smem + p.remote + static_cast<size_t>(r) * bs * key_row, a.key_dtype, bs, 0,
                       sel[3 * r + 2], sel[3 * r] * bs, anchor_pos, pq, cand, L + r * bs);
        __syncthreads();
    }
    if (warp == 0) {
        const int cap = L + top * bs;
        for (int k = 0; k < a.k_out; ++k) {
            float bv = kNegInf;
            int bc = 0x7fffffff;
            for (int c = lane; c < cap; c += 32) {
                float v = cand[c];
                if (v > bv || bc == 0x7fffffff) { bv = v; bc = c; }
            }
            warp_argmax_low(bv, bc);
            if (lane == 0) {
                int pos;
                if (bc < L) pos = t - L + 1 + bc;
                else { int r = (bc - L) / bs; pos = sel[3 * r] * bs + (bc - L - r * bs); }
                a.out_partner[static_cast<size_t>(row) * a.k_out + k] = pos;
                a.out_partner_score[static_cast<size_t>(row) * a.k_out + k] = bv;
                cand[bc] = kNegInf;
            }
            __syncwarp();
        }
    }
}

int launch(SelectArgs& a, void* stream) {
    if (a.n_rows == 0) return RLM_OK;
    if (a.n_rows < 0 || a.n_seq < 1 || a.max_t < 1 || a.n_blocks < 1 || a.buckets < 1 ||
        a.local_window < 1 || a.top_blocks < 0 || a.max_t % a.n_blocks != 0) {
        set_error("relation_select: sizes must be positive and T a multiple of the block count");
        return RLM_ERR_SHAPE;
    }
    if (a.mode != kAnchorOnly && a.k_out < 1) {
        set_error("relation_select: k_out must be at least 1");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(a.query_dtype) || !valid_dtype(a.key_dtype) || !valid_dtype(a.stats_dtype) ||
        !valid_dtype(a.param_dtype)) {
        set_error("relation_select: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    if (!a.position && !a.row_position) {
        set_error("relation_select: either position or row_position is required");
        return RLM_ERR_NULL;
    }
    if (!a.row_batch && a.n_rows != a.n_seq) {
        set_error("relation_select: without row_batch the query rows must equal the sequences");
        return RLM_ERR_SHAPE;
    }
    bool anchor = a.mode != kPartnerOnly, partner = a.mode != kAnchorOnly;
    const void* need_a[] = {a.anchor_query, a.anchor_keys, a.anchor_router_query, a.anchor_mean,
                            a.anchor_std, a.anchor_gamma, a.anchor_bias, a.out_anchor, a.out_anchor_score};
    const void* need_p[] = {a.partner_base, a.partner_keys, a.partner_mean, a.partner_std,
                            a.partner_gamma, a.partner_bias, a.out_partner, a.out_partner_score};
    if (anchor) for (const void* q : need_a) if (!q) { set_error("relation_select: NULL anchor-side pointer"); return RLM_ERR_NULL; }
    if (partner) for (const void* q : need_p) if (!q) { set_error("relation_select: NULL partner-side pointer"); return RLM_ERR_NULL; }
    if (a.mode == kPacked && !a.partner_anchor_cache) { set_error("relation_select: NULL partner_anchor_cache"); return RLM_ERR_NULL; }
    if (a.mode == kPartnerOnly && (!a.partner_router_query || !a.anchor_index_in)) { set_error("partner_topk: NULL router query or anchor index"); return RLM_ERR_NULL; }
    const void* bulk[] = {a.anchor_keys, a.anchor_mean, a.anchor_std, a.partner_keys, a.partner_mean,
                          a.partner_std, a.partner_anchor_cache};
    for (const void* q : bulk)
        if (q && !aligned16(q)) {
            set_error("relation_select: key caches, block statistics and the partner-anchor cache must be 16-byte aligned");
            return RLM_ERR_ALIGN;
        }
    a.block_size = a.max_t / a.n_blocks;
    Plan plan = make_plan(a.n_blocks, a.block_size, a.local_window, a.top_blocks, a.buckets,
                          dtype_size(a.key_dtype), dtype_size(a.stats_dtype), a.mode);
    if (plan.total > kSmemDynamicLimit) {
        set_error("relation_select: block statistics + local window + remote blocks exceed 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    int rc = allow_large_smem(reinterpret_cast<const void*>(relation_select_kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    relation_select_kernel<<<a.n_rows, kThreads, plan.total, static_cast<cudaStream_t>(stream)>>>(a);
    count_launch();
    return check_launch("relation_select_kernel");
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_relation_select_packed(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma,
    const void* anchor_bias, const void* partner_base, const void* partner_anchor_cache,
    const void* partner_keys, const void* partner_mean, const void* partner_std,
    const void* partner_gamma, const void* partner_bias, const int64_t* position,
    const int32_t* row_batch, const int32_t* row_position, int32_t* out_anchor,
    float* out_anchor_score, int32_t* out_partner, float* out_partner_score,
    int64_t anchor_query_stride, int64_t anchor_router_query_stride, int64_t partner_base_stride,
    int n_rows, int n_seq,
    int max_t, int n_blocks, int buckets, int local_window, int top_blocks, int k_out,
    int strict_valid, int query_dtype, int key_dtype, int stats_dtype, int param_dtype,
    int32_t* status, void* stream) {
    rlm::SelectArgs a{};
    a.aq_stride = anchor_query_stride; a.arq_stride = anchor_router_query_stride; a.pbase_stride = partner_base_stride;
    a.anchor_query = anchor_query; a.anchor_keys = anchor_keys; a.anchor_router_query = anchor_router_query;
    a.anchor_mean = anchor_mean; a.anchor_std = anchor_std; a.anchor_gamma = anchor_gamma; a.anchor_bias = anchor_bias;
    a.partner_base = partner_base; a.partner_anchor_cache = partner_anchor_cache; a.partner_keys = partner_keys;
    a.partner_mean = partner_mean; a.partner_std = partner_std; a.partner_gamma = partner_gamma; a.partner_bias = partner_bias;
    a.position = position; a.row_batch = row_batch; a.row_position = row_position;
    a.out_anchor = out_anchor; a.out_anchor_score = out_anchor_score; a.out_partner = out_partner; a.out_partner_score = out_partner_score;
    a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks; a.buckets = buckets;
    a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = k_out; a.strict_valid = strict_valid != 0;
    a.query_dtype = query_dtype; a.key_dtype = key_dtype; a.stats_dtype = stats_dtype; a.param_dtype = param_dtype;
    a.mode = rlm::kPacked;
    return rlm::launch(a, stream);
}

extern "C" int rlm_anchor_select(
    const void* anchor_query, const void* anchor_keys, const void* router_query,
    const void* block_mean, const void* block_std, const void* gamma, const void* bias,
    const int64_t* position, const int32_t* row_batch, const int32_t* row_position,
    int32_t* out_index, float* out_score, int n_rows, int n_seq, int max_t, int n_blocks,
    int buckets, int local_window, int top_blocks, int strict_valid, int query_dtype,
    int key_dtype, int stats_dtype, int param_dtype, int32_t* status, void* stream) {
    rlm::SelectArgs a{};
    a.aq_stride = 64; a.arq_stride = 64;
    a.anchor_query = anchor_query; a.anchor_keys = anchor_keys; a.anchor_router_query = router_query;
    a.anchor_mean = block_mean; a.anchor_std = block_std; a.anchor_gamma = gamma; a.anchor_bias = bias;
    a.position = position; a.row_batch = row_batch; a.row_position = row_position;
    a.out_anchor = out_index; a.out_anchor_score = out_score; a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks; a.buckets = buckets;
    a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = 0; a.strict_valid = strict_valid != 0;
    a.query_dtype = query_dtype; a.key_dtype = key_dtype; a.stats_dtype = stats_dtype; a.param_dtype = param_dtype;
    a.mode = rlm::kAnchorOnly;
    return rlm::launch(a, stream);
}

extern "C" int rlm_partner_topk(
    const void* partner_query, const void* partner_keys, const void* router_query,
    const void* block_mean, const void* block_std, const void* gamma, const void* bias,
    const int64_t* position, const int32_t* row_batch, const int32_t* row_position,
    const int32_t* anchor_index, int32_t* out_index, float* out_score, int n_rows, int n_seq,
    int max_t, int n_blocks, int buckets, int local_window, int top_blocks, int k_out,
    int strict_valid, int query_dtype, int key_dtype, int stats_dtype, int param_dtype,
    int32_t* status, void* stream) {
    rlm::SelectArgs a{};
    a.pbase_stride = 64; a.prq_stride = 64;
    a.partner_base = partner_query; a.partner_router_query = router_query; a.partner_keys = partner_keys;
    a.partner_mean = block_mean; a.partner_std = block_std; a.partner_gamma = gamma; a.partner_bias = bias;
    a.position = position; a.row_batch = row_batch; a.row_position = row_position;
    a.anchor_index_in = anchor_index; a.out_partner = out_index; a.out_partner_score = out_score; a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks; a.buckets = buckets;
    a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = k_out; a.strict_valid = strict_valid != 0;
    a.query_dtype = query_dtype; a.key_dtype = key_dtype; a.stats_dtype = stats_dtype; a.param_dtype = param_dtype;
    a.mode = rlm::kPartnerOnly;
    return rlm::launch(a, stream);
}
