// Device code of the routed selector shared by its kernels: the shared-memory plan, the scoring,
// block-picking and top-K functions, and select_row (one query row by a whole CTA); plus the host-side
// validation of a selector launch.  Included by relation_select.cu (per-row, multi-anchor and
// whole-sequence kernels) and relation_layer.cu (the selector in front of the relation tail): the
// two are separate translation units on purpose, because the out-of-line helpers below are
// compiled once per unit and their register budget follows the unit's most generous launch
// bounds, which made the per-row kernels spill when the one-CTA-per-SM layer kernel lived beside them.
#pragma once

#include "rlm_common.cuh"

namespace rlm {
namespace {


constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxKOut = 32;  // partner slots per query
constexpr int kMaxExclude = 8; // extra excluded positions per query (multi-anchor selection)
constexpr int kD = 64;        // exact-score width == router heads * head width

enum Mode { kPacked = 0, kAnchorOnly = 1, kPartnerOnly = 2 };

// Shared-memory plan (byte offsets from the dynamic shared base).
struct Plan {
    int a_mean, a_std, p_mean, p_std;   // [NB,64] stats elements
    int a_local, p_local;               // [L,64] key elements
    int remote;                         // [TOP*BS,64] key elements (anchor phase, then partner phase)
    int queries;                        // f32: aq[64] arq[64] pq[64] prq[64]
    int params;                         // f32: softplus(gamma) a[4] p[4], bias a[4*buckets] p[4*buckets]
    int block_scores;                   // f32 [NB]
    int cand;                           // f32 [L + TOP*BS]
    int sel;                            // int [3*TOP]: block, usable, valid row count
    int bars;                           // 4 mbarriers
    int total;
};

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
    const int32_t* exclude_list;         // optional [N, exclude_count]: positions barred as candidates (< 0: unused entry)
    int exclude_count;
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
    int shared_streams;                  // the partner's staging buffers alias the anchor's (see make_plan)
    int sm_count;                        // streaming multiprocessors of the device the launch goes to
    int resident;                        // decode form with the whole key caches staged (see select_row)
    Plan plan;
};

__host__ __device__ inline int align16(int x) { return (x + 15) & ~15; }

// With `shared_streams` (packed mode only) the partner's statistics and local window take the
// anchor's place once the anchor's first scoring pass has read them: a smaller footprint, so
// more rows per SM, for launches of many rows.
// resident_rows > 0: the whole key cache of the sequence (that many rows) takes the place of the
// local window, and no buffer is kept for remote blocks (see SelectArgs::resident).
__host__ __device__ inline Plan make_plan(int nb, int bs, int local, int top, int buckets,
                                          int key_size, int stats_size, int mode, bool shared_streams,
                                          int resident_rows = 0) {
    Plan p;
    int off = 0;
    int stats_bytes = nb * kD * stats_size;
    int local_bytes = (resident_rows > 0 ? resident_rows : local) * kD * key_size;
    bool anchor = mode != kPartnerOnly, partner = mode != kAnchorOnly;
    p.a_mean = off; off += anchor ? stats_bytes : 0;
    p.a_std = off; off += anchor ? stats_bytes : 0;
    p.p_mean = shared_streams ? p.a_mean : off; off += partner && !shared_streams ? stats_bytes : 0;
    p.p_std = shared_streams ? p.a_std : off; off += partner && !shared_streams ? stats_bytes : 0;
    p.a_local = off; off += anchor ? local_bytes : 0;
    p.p_local = shared_streams ? p.a_local : off; off += partner && !shared_streams ? local_bytes : 0;
    p.remote = off; off += resident_rows > 0 ? 0 : top * bs * kD * key_size;
    p.queries = off; off += 4 * kD * 4;
    p.params = off; off += align16(8 * buckets * 4);
    p.block_scores = off; off += align16(((nb + 3) & ~3) * 4);
    p.cand = off; off += align16((local + top * bs) * 4);
    p.sel = off; off += align16(3 * (top > 0 ? top : 1) * 4);
    p.bars = off; off += 4 * 8;
    p.total = align16(off);
    return p;
}

// ---- key-row scoring
//
// The canonical dot of a 64-wide row is eight 8-element fma chains p0..p7 combined as
// ((p0+p1)+(p2+p3))+((p4+p5)+(p6+p7)).  One, two or four lanes share a row (kLpr): with many
// rows per warp a lane owns a whole row and needs no shuffles; with few rows the chains are
// spread over two or four lanes (two xor-shuffle additions at most) so that all lanes of the
// group work and the dependent chain per lane is shorter.  Rows are 128 (or 256) bytes apart in
// shared memory, so the lanes of a quarter warp must not read the same 16-byte chunk index at
// the same time: the order in which a lane walks its chunks is rotated by its row number.
// Because a + b == b + a exactly, the sums are bit-identical to the fixed order whatever the
// split; tree4() undoes the rotation.

// (s0 + s1) + (s2 + s3) from x[jj] = s[(jj + r) & 3]
__device__ __forceinline__ float tree4(const float (&x)[4], int r) {
    const bool odd = (r & 1) != 0;
    const float a = __fadd_rn(odd ? x[3] : x[0], odd ? x[0] : x[1]);
    const float b = __fadd_rn(odd ? x[1] : x[2], odd ? x[2] : x[3]);
    return __fadd_rn(a, b);
}

__device__ __forceinline__ float chunk_dot(const unsigned char* row, const float* query, int c, int key_dtype) {
    float k[8], q[8];
    load8(row, 8 * c, key_dtype, k);
    load8(query, 8 * c, RLM_F32, q);
    return seg8(k, q);
}

// Scores staged key rows against the query held in shared memory (f32 [64]) with the
// `nw` warps of a group (this warp is number `wi`).  Two layouts:
//   local window (sel == nullptr): row r is position pos0 + r, valid from `first_valid` on;
//   remote blocks (sel != nullptr): row r belongs to the block of rank r / bs at offset
//     o = r % bs, position sel[3 rank] * bs + o, valid while o < sel[3 rank + 2].
// The rows at position `exclude` and at the positions excl[0 .. n_excl) score -inf.  With a
// barrier address in `bar` the rows are still being copied: the warp waits for them after it has
// worked out its first rows' positions (`arrived` = false when the wait gave up).  With `cand`
// the scores go to candidate slots slot0 + r and nothing else happens; without, the warp's best
// (score, lowest position on ties) is folded into (best_key, best_pos), identical in all lanes.
// kAtPosition: `rows` is the sequence's whole key cache and a candidate row is read where it lies
// (row = its position), straight from global memory / L2, instead of from a staged copy.
template <bool kBf16, int kLpr, bool kAtPosition = false>
__device__ __noinline__ void score_rows_split(const unsigned char* rows, int key_dtype_arg, int n_rows,
                                              const int* sel, int bs, int first_valid, int pos0,
                                              int exclude, const int* excl, int n_excl, const float* query,
                                              float* cand, int slot0, int wi, int nw, uint32_t& best_key,
                                              int& best_pos, uint32_t bar, bool& arrived) {
    constexpr int kRows = 32 / kLpr;                 // rows per warp pass
    const int lane = threadIdx.x & 31;
    const int sub = lane & (kLpr - 1), rl = lane / kLpr;
    const int key_dtype = kBf16 ? RLM_BF16 : key_dtype_arg;
    const int row_bytes = kD * (key_dtype == RLM_F32 ? 4 : 2);
    uint32_t my_key = 0;
    int my_pos = 0x7fffffff;
    for (int base = wi * kRows; base < n_rows; base += kRows * nw) {
        const int r = base + rl;
        int pos;
        bool valid;
        if (sel) {
            const int rank = (bs & (bs - 1)) == 0 ? r >> (31 - __clz(bs)) : r / bs, o = r - rank * bs;
            const bool in = r < n_rows;
            pos = in ? sel[3 * rank] * bs + o : -1;
            valid = in && o < sel[3 * rank + 2];
        } else {
            pos = pos0 + r;
            valid = r < n_rows && r >= first_valid;
        }
        valid = valid && pos != exclude;
        for (int x = 0; x < n_excl; ++x) valid = valid && pos != excl[x];
        float part = 0.0f;
        if (bar != 0u) {          // the rows' bulk copies were given the time of the set-up above
            arrived = mbar_wait(bar, 0);
            bar = 0u;
        }
        valid = valid && arrived;
        if (valid) {
            const unsigned char* row = rows + static_cast<size_t>(kAtPosition ? pos : r) * row_bytes;
            if (kLpr == 1) {
                // pair sums (p0+p1) .. (p6+p7), pair index rotated by the row, lanes 4..7 of
                // each group of eight taking the pair's second chunk first
                float pair[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int c0 = 2 * ((jj + rl) & 3) + ((rl >> 2) & 1);
                    pair[jj] = __fadd_rn(chunk_dot(row, query, c0, key_dtype), chunk_dot(row, query, c0 ^ 1, key_dtype));
                }
                part = tree4(pair, rl & 3);
            } else if (kLpr == 2) {
                // this lane: (p0+p1)+(p2+p3) or (p4+p5)+(p6+p7), chunk order rotated by the row
                float x[4];
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) x[jj] = chunk_dot(row, query, 4 * sub + ((jj + rl) & 3), key_dtype);
                part = tree4(x, rl & 3);
            } else {
                // this lane: one pair sum, odd rows taking the second chunk first
                const int c0 = 2 * sub + (rl & 1);
                part = __fadd_rn(chunk_dot(row, query, c0, key_dtype), chunk_dot(row, query, c0 ^ 1, key_dtype));
            }
        }
        if (kLpr >= 2) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, 1));
        if (kLpr == 4) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, 2));
        const float sc = valid ? __fmul_rn(part, 0.125f) : kNegInf;
        if (cand) {                 // the partner stream only fills the candidate table
            if (r < n_rows && sub == 0) cand[slot0 + r] = sc;
            continue;
        }
        const uint32_t key = float_key(sc);
        if (valid && (key > my_key || my_pos == 0x7fffffff || (key == my_key && pos < my_pos))) {
            my_key = key;
            my_pos = pos;
        }
    }
    if (cand) return;
    warp_argmax_key(my_key, my_pos);
    if (my_pos != 0x7fffffff &&
        (my_key > best_key || best_pos == 0x7fffffff || (my_key == best_key && my_pos < best_pos))) {
        best_key = my_key;
        best_pos = my_pos;
    }
}

// Picks the split that keeps every lane of the group busy in the fewest passes (launches of at
// most one CTA per SM, where a row's latency is what counts).
template <bool kBf16, bool kAtPosition = false>
__device__ __forceinline__ void score_rows(const unsigned char* rows, int key_dtype, int n_rows,
                                           const int* sel, int bs, int first_valid, int pos0,
                                           int exclude, const int* excl, int n_excl, const float* query,
                                           float* cand, int slot0, int wi, int nw, uint32_t& best_key,
                                           int& best_pos, uint32_t bar, bool& arrived, int sm_count_arg) {
    const int lanes = static_cast<int>(gridDim.x) <= sm_count_arg ? 32 * nw : 0;   // a row per lane when CTAs share the SMs: fewer instructions in total
    if (4 * n_rows <= lanes)
        score_rows_split<kBf16, 4, kAtPosition>(rows, key_dtype, n_rows, sel, bs, first_valid, pos0, exclude, excl, n_excl,
                                   query, cand, slot0, wi, nw, best_key, best_pos, bar, arrived);
    else if (2 * n_rows <= lanes)
        score_rows_split<kBf16, 2, kAtPosition>(rows, key_dtype, n_rows, sel, bs, first_valid, pos0, exclude, excl, n_excl,
                                   query, cand, slot0, wi, nw, best_key, best_pos, bar, arrived);
    else
        score_rows_split<kBf16, 1, kAtPosition>(rows, key_dtype, n_rows, sel, bs, first_valid, pos0, exclude, excl, n_excl,
                                   query, cand, slot0, wi, nw, best_key, best_pos, bar, arrived);
}

// Block scores of the first `n_complete` blocks with the `nw` warps of a group; the other
// entries of `out` (up to the next multiple of four) are set to -inf.
template <bool kBf16>
__device__ __noinline__ void score_blocks(const unsigned char* mean, const unsigned char* stdv,
                                          int stats_dtype_arg, int nb, int n_complete, int bs, int t,
                                          int ls, int strict, int buckets, const float* rq,
                                          const float* sp4, const float* bias, float* out, int wi, int nw) {
    const int lane = threadIdx.x & 31;
    const int j = lane & 7, sub = lane >> 3, head = j >> 1;
    const int stats_dtype = kBf16 ? RLM_BF16 : stats_dtype_arg;
    const int row_bytes = kD * (stats_dtype == RLM_F32 ? 4 : 2);
    const float sp = sp4[head];
    float q[8], aq[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { q[i] = rq[8 * j + i]; aq[i] = fabsf(q[i]); }
    for (int n = n_complete + wi * 32 + lane; n < ((nb + 3) & ~3); n += 32 * nw) out[n] = kNegInf;
    for (int base = wi * 4; base < n_complete; base += 4 * nw) {
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
        // log-sum-exp over the four heads, max-shifted: every lane evaluates the exponential
        // of its own head, the sum is (e0 + e1) + (e2 + e3) through two xor shuffles.
        float mx = fmaxf(sh, __shfl_xor_sync(0xffffffffu, sh, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        float e = canon_exp(__fsub_rn(sh, mx));
        e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, 2));
        e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, 4));
        float acc = __fadd_rn(mx, canon_log(e));
        if (j == 0 && live) {
            bool eligible = !strict || end < ls;
            out[n] = eligible ? acc : kNegInf;
        }
    }
}

// The same block scores with four lanes per block, a head (16 statistics elements = chunks 2h and
// 2h + 1) per lane: fewer instructions per block and eight blocks per warp pass, for caches of
// more than 16 blocks.  Odd blocks of a pass take a head's second chunk first so that the eight
// lanes of a quarter warp read eight different 16-byte chunk indices (rows are 128 or 256 bytes
// apart in shared memory).  Every sum is one of the eight-lane form's sums with its operands
// possibly swapped, so the scores are bit-identical.
template <bool kBf16>
__device__ __noinline__ void score_blocks_head(const unsigned char* mean, const unsigned char* stdv,
                                               int stats_dtype_arg, int nb, int n_complete, int bs, int t,
                                               int ls, int strict, int buckets, const float* rq,
                                               const float* sp4, const float* bias, float* out, int wi, int nw) {
    const int lane = threadIdx.x & 31;
    const int head = lane & 3, bl = lane >> 2;
    const int stats_dtype = kBf16 ? RLM_BF16 : stats_dtype_arg;
    const int row_bytes = kD * (stats_dtype == RLM_F32 ? 4 : 2);
    const int c0 = 2 * head + (bl & 1), c1 = c0 ^ 1;
    float q0[8], q1[8], a0[8], a1[8];
    load8(rq, 8 * c0, RLM_F32, q0);
    load8(rq, 8 * c1, RLM_F32, q1);
#pragma unroll
    for (int i = 0; i < 8; ++i) { a0[i] = fabsf(q0[i]); a1[i] = fabsf(q1[i]); }
    const float sp = sp4[head];
    for (int n = n_complete + wi * 32 + lane; n < ((nb + 3) & ~3); n += 32 * nw) out[n] = kNegInf;
    for (int base = wi * 8; base < n_complete; base += 8 * nw) {
        const int n = base + bl;
        const bool live = n < n_complete;
        const int end = (n + 1) * bs - 1;
        int dist = t - end;
        if (dist < 0) dist = 0;
        int bucket = 31 - __clz(dist + 1);
        if (bucket > buckets - 1) bucket = buckets - 1;
        float md = 0.0f, sd = 0.0f;
        if (live) {
            const unsigned char* m = mean + static_cast<size_t>(n) * row_bytes;
            const unsigned char* sdev = stdv + static_cast<size_t>(n) * row_bytes;
            float v[8], w[8];
            load8(m, 8 * c0, stats_dtype, v);
            load8(m, 8 * c1, stats_dtype, w);
            md = __fadd_rn(seg8(v, q0), seg8(w, q1));
            load8(sdev, 8 * c0, stats_dtype, v);
            load8(sdev, 8 * c1, stats_dtype, w);
            sd = __fadd_rn(seg8(v, a0), seg8(w, a1));
        }
        const float sh = __fadd_rn(__fmul_rn(__fadd_rn(md, __fmul_rn(sp, sd)), 0.25f),
                                   live ? bias[head * buckets + bucket] : 0.0f);
        float mx = fmaxf(sh, __shfl_xor_sync(0xffffffffu, sh, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        float e = canon_exp(__fsub_rn(sh, mx));
        e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, 1));       // e0 + e1 | e2 + e3
        e = __fadd_rn(e, __shfl_xor_sync(0xffffffffu, e, 2));       // (e0 + e1) + (e2 + e3)
        const float acc = __fadd_rn(mx, canon_log(e));
        if (head == 0 && live) {
            const bool eligible = !strict || end < ls;
            out[n] = eligible ? acc : kNegInf;
        }
    }
}

// Eight lanes per block up to 16 complete blocks (one pass of four warps), a head per lane beyond.
template <bool kBf16>
__device__ __forceinline__ void score_blocks_any(const unsigned char* mean, const unsigned char* stdv,
                                                 int stats_dtype, int nb, int n_complete, int bs, int t,
                                                 int ls, int strict, int buckets, const float* rq,
                                                 const float* sp4, const float* bias, float* out, int wi, int nw) {
    if (n_complete > 16)
        score_blocks_head<kBf16>(mean, stdv, stats_dtype, nb, n_complete, bs, t, ls, strict, buckets, rq, sp4,
                                 bias, out, wi, nw);
    else
        score_blocks<kBf16>(mean, stdv, stats_dtype, nb, n_complete, bs, t, ls, strict, buckets, rq, sp4, bias,
                            out, wi, nw);
}

// Warp 0: rank the block scores by counting (descending score, ties to the lowest index)
// and record (block, usable, rows before the local window) for ranks below `top`.  Ranks of
// blocks that are not usable (-inf) never matter: they contribute no candidates.  `scores`
// is padded with -inf to a multiple of four.
__device__ __noinline__ void pick_blocks(const float* scores, int nb, int top, int bs, int ls,
                                         int* sel) {
    const int lane = threadIdx.x & 31;
    for (int r = lane; r < top; r += 32) { sel[3 * r] = 0; sel[3 * r + 1] = 0; sel[3 * r + 2] = 0; }
    __syncwarp();
    const float4* s4 = reinterpret_cast<const float4*>(scores);
    const int groups = (nb + 3) >> 2;
    for (int n = lane; n < nb; n += 32) {
        const float mine = scores[n];
        if (!(mine > -1.0e30f)) continue;
        int rank = 0;
        for (int g = 0; g < groups; ++g) {
            float4 o = s4[g];
            const int m = g << 2;
            rank += (o.x > mine || (o.x == mine && m < n)) + (o.y > mine || (o.y == mine && m + 1 < n)) +
                    (o.z > mine || (o.z == mine && m + 2 < n)) + (o.w > mine || (o.w == mine && m + 3 < n));
        }
        if (rank < top) {
            int rows = ls - n * bs;
            rows = rows < 0 ? 0 : (rows > bs ? bs : rows);
            sel[3 * rank] = n;
            sel[3 * rank + 1] = 1;
            sel[3 * rank + 2] = rows;
        }
    }
    __syncwarp();
}

// Exact top-K of up to 32 * kN candidate scores by one warp.  Lane l holds slots kN*l ..
// kN*l + kN - 1 as (score key, inverted slot) composites sorted in descending order (a fixed
// compare-exchange network), so its head is its best remaining candidate.  Each of the K rounds
// takes the largest head of the warp (one redux); among equal keys the lowest lane wins, which is
// the lowest slot because lanes hold ascending slot ranges and equal keys are sorted by slot
// inside a lane.  The winner pops its head.  Slots past the candidates hold key 0 and never
// beat a score; a result whose score is -inf (or missing) reports position t - L + 1.
template <int kN>
__device__ __noinline__ void topk_tournament(const float* cand, int cap4, int K, int L, int t, int bs,
                                                int bs_shift, const int* sel, int32_t* out_pos, float* out_score) {
    const int lane = threadIdx.x & 31;
    const float4* cand4 = reinterpret_cast<const float4*>(cand);
    uint64_t c[kN];
#pragma unroll
    for (int h = 0; h < kN / 4; ++h) {
        const int g = lane * (kN / 4) + h;
        const bool in = 4 * g < cap4;
        const float4 v = in ? cand4[g] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t key = in ? float_key(x[i] + 0.0f) : 0u;       // -0 and +0 tie
            c[4 * h + i] = (static_cast<uint64_t>(key) << 32) | (0xffffffffu - static_cast<uint32_t>(4 * g + i));
        }
    }
#define RLM_CE(i, j) do { const uint64_t hi_ = c[i] > c[j] ? c[i] : c[j], lo_ = c[i] > c[j] ? c[j] : c[i]; c[i] = hi_; c[j] = lo_; } while (0)
    if (kN == 4) {
        RLM_CE(0, 1); RLM_CE(2, 3); RLM_CE(0, 2); RLM_CE(1, 3); RLM_CE(1, 2);
    } else if (kN > 8) {
        // odd-even transposition sort, descending (up to 512 candidate slots per warp)
#pragma unroll
        for (int round = 0; round < kN; ++round)
#pragma unroll
            for (int i = round & 1; i + 1 < kN; i += 2) RLM_CE(i, i + 1);
    } else {
        RLM_CE(0, 1); RLM_CE(2, 3); RLM_CE(4, 5); RLM_CE(6, 7); RLM_CE(0, 2); RLM_CE(1, 3); RLM_CE(4, 6);
        RLM_CE(5, 7); RLM_CE(1, 2); RLM_CE(5, 6); RLM_CE(0, 4); RLM_CE(3, 7); RLM_CE(1, 5); RLM_CE(2, 6);
        RLM_CE(1, 4); RLM_CE(3, 6); RLM_CE(2, 4); RLM_CE(3, 5); RLM_CE(3, 4);
    }
#undef RLM_CE
    uint32_t won_key = 0, won_slot = 0;
    for (int r = 0; r < K; ++r) {
        const uint32_t head = static_cast<uint32_t>(c[0] >> 32);
        const uint32_t best = __reduce_max_sync(0xffffffffu, head);
        const int w = __ffs(__ballot_sync(0xffffffffu, head == best)) - 1;
        const uint32_t slot = 0xffffffffu - __shfl_sync(0xffffffffu, static_cast<uint32_t>(c[0]), w);
        if (lane == r) { won_key = best; won_slot = slot; }
        if (lane == w) {
#pragma unroll
            for (int i = 0; i + 1 < kN; ++i) c[i] = c[i + 1];
            c[kN - 1] = 0;
        }
    }
    if (lane < K) {
        const float sc = won_key == 0u ? kNegInf : cand[won_slot];
        const int cs = static_cast<int>(won_slot);
        int pos;
        if (!(sc > kNegInf)) pos = t - L + 1;
        else if (cs < L) pos = t - L + 1 + cs;
        else { const int rr = bs_shift >= 0 ? (cs - L) >> bs_shift : (cs - L) / bs; pos = sel[3 * rr] * bs + (cs - L - rr * bs); }
        out_pos[lane] = pos;
        out_score[lane] = sc;
    }
}

// Exact top-K of more than 256 candidate slots, by the whole CTA (out of line: the decode shapes
// never come here, and the selector's common path stays compact).
__device__ __noinline__ void topk_large(float* cand, int cap, int K, int L, int t, int bs, const int* sel,
                                        int32_t* out_pos, float* out_score) {
    __shared__ uint32_t surv_key[kWarps * kMaxKOut];
    __shared__ int surv_slot[kWarps * kMaxKOut];
    __shared__ uint32_t group_max[2 * kWarps];
    __shared__ int short_count;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) short_count = 0;
    __syncthreads();
    // Threshold filter: the K-th largest of the sixteen half-warp maxima is a lower bound of
    // the K-th largest score, so only candidates at or above it can be selected.  They are
    // compacted into a short list and ranked exactly there; when the list is long (many equal
    // or -inf scores) the tournament through shared memory below takes over with the score
    // table untouched.
    if (K <= 2 * kWarps && cap > 16 * (K - 1)) {
        uint32_t kmax = 0;
        for (int c = tid; c < cap; c += kThreads) kmax = max(kmax, float_key(cand[c] + 0.0f));
#pragma unroll
        for (int s = 8; s > 0; s >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, s));
        if ((lane & 15) == 0) group_max[tid >> 4] = kmax;
        __syncthreads();
        const uint32_t g = group_max[lane & 15];
        int grank = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t o = __shfl_sync(0xffffffffu, g, j);
            grank += (o > g) || (o == g && j < (lane & 15));
        }
        const unsigned holder = __ballot_sync(0xffffffffu, grank == K - 1) & 0xffffu;
        const uint32_t tau = __shfl_sync(0xffffffffu, g, __ffs(holder) - 1);
        for (int c0 = 0; c0 < cap; c0 += kThreads) {
            const int c = c0 + tid;
            const uint32_t key = c < cap ? float_key(cand[c] + 0.0f) : 0u;
            const bool pass = c < cap && key >= tau;
            const unsigned m = __ballot_sync(0xffffffffu, pass);
            int base = 0;
            if (lane == 0 && m) base = atomicAdd(&short_count, __popc(m));
            base = __shfl_sync(0xffffffffu, base, 0);
            const int at = base + __popc(m & ((1u << lane) - 1u));
            if (pass && at < kWarps * kMaxKOut) { surv_key[at] = key; surv_slot[at] = c; }
        }
        __syncthreads();
        const int n = short_count;
        if (tau > float_key(kNegInf) && n <= kThreads / 4) {
            const int i = tid >> 2, part = tid & 3;
            int rank = 0, c = 0;
            uint32_t key = 0;
            if (i < n) {
                key = surv_key[i];
                c = surv_slot[i];
                for (int j = part; j < n; j += 4) {
                    const uint32_t ok = surv_key[j];
                    rank += (ok > key) || (ok == key && surv_slot[j] < c);
                }
            }
            rank += __shfl_xor_sync(0xffffffffu, rank, 1);
            rank += __shfl_xor_sync(0xffffffffu, rank, 2);
            if (i < n && part == 0 && rank < K) {
                int pos;
                if (c < L) pos = t - L + 1 + c;
                else { int r = (c - L) / bs; pos = sel[3 * r] * bs + (c - L - r * bs); }
                out_pos[rank] = pos;
                out_score[rank] = cand[c];
            }
            return;
        }
    }
    {
        // Fallback for large candidate sets: tournament through shared memory.  Each warp extracts the top K of the slots it
        // owns (K rounds of redux arg-max, knocking winners out of the table); warp 0 then
        // extracts the top K of the 8 K survivors.  Any global top-K candidate is among the
        // top K of its own warp, and (score, lowest slot) ordering is kept at both levels.
        for (int r = 0; r < K; ++r) {
            uint32_t bk = 0;
            int bc = 0x7fffffff;
            for (int c = warp * 32 + lane; c < cap; c += kThreads) {
                uint32_t key = float_key(cand[c]);
                if (key > bk || bc == 0x7fffffff) { bk = key; bc = c; }
            }
            warp_argmax_key(bk, bc);
            if (lane == 0) {
                surv_key[warp * kMaxKOut + r] = bc == 0x7fffffff ? 0u : bk;
                surv_slot[warp * kMaxKOut + r] = bc;
                if (bc != 0x7fffffff) cand[bc] = __uint_as_float(0xffffffffu);   // below every score: key 0
            }
            __syncwarp();
        }
        __syncthreads();
        if (warp == 0) {
            for (int r = 0; r < K; ++r) {
                uint32_t bk = 0;
                int bc = 0x7fffffff, bi = -1;
                for (int i = lane; i < kWarps * K; i += 32) {
                    const int e = (i / K) * kMaxKOut + (i - (i / K) * K);
                    uint32_t key = surv_key[e];
                    int c = surv_slot[e];
                    if (key != 0u && (key > bk || (key == bk && c < bc) || bc == 0x7fffffff)) { bk = key; bc = c; bi = e; }
                }
                const int mine = bc;
                warp_argmax_key(bk, bc);
                if (bc != 0x7fffffff && mine == bc && bi >= 0) surv_key[bi] = 0u;
                if (lane == 0) {
                    const float sc = bc == 0x7fffffff ? kNegInf : key_float(bk);
                    int pos;
                    if (!(sc > kNegInf)) pos = t - L + 1;
                    else if (bc < L) pos = t - L + 1 + bc;
                    else { int rr = (bc - L) / bs; pos = sel[3 * rr] * bs + (bc - L - rr * bs); }
                    out_pos[r] = pos;
                    out_score[r] = sc;
                }
                __syncwarp();
            }
        }
    }
}

// Warp 0, at most 128 blocks and 32 remote blocks: block picking and the bulk-copy requests in
// one pass.  Lane l holds the scores of blocks l, l + 32, ...; each of the `top` rounds takes
// the best remaining block of the warp (two redux instructions; ties to the lowest index) and
// hands it to lane `round`, which then requests its own block, after lane 0 has posted the byte
// count of all of them.  Same result as pick_blocks + issue_remote.
__device__ __noinline__ void pick_and_issue(const float* scores, int nb, int top, int bs, int ls, int* sel,
                                            const unsigned char* keys, unsigned char* dst, size_t key_row,
                                            size_t seq_keys, uint32_t bar) {
    const int lane = threadIdx.x & 31;
    uint32_t k[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) k[i] = lane + 32 * i < nb ? float_key(scores[lane + 32 * i]) : 0u;
    int my_block = 0, my_rows = 0;
    for (int r = 0; r < top; ++r) {
        uint32_t bk = 0;
        int bn = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (k[i] > bk) { bk = k[i]; bn = lane + 32 * i; }
        warp_argmax_key(bk, bn);
        if (!(key_float(bk) > -1.0e30f)) break;          // no usable block is left
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (lane + 32 * i == bn) k[i] = 0u;
        if (lane == r) {
            int rows = ls - bn * bs;
            my_rows = rows < 0 ? 0 : (rows > bs ? bs : rows);
            my_block = bn;
        }
    }
    if (lane < top) { sel[3 * lane] = my_block; sel[3 * lane + 1] = 1; sel[3 * lane + 2] = my_rows; }
    const uint32_t bytes = static_cast<uint32_t>(my_rows * key_row);
    const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
    // The destination may have been read (never written) through the generic proxy before: those
    // reads were ordered before this point by the block-wide barrier, as in any ring of bulk-copy
    // stages released by its consumers, so no proxy fence is needed.
    if (lane == 0) mbar_expect_tx(bar, total);
    __syncwarp();
    if (my_rows > 0)
        bulk_g2s(smem_u32(dst) + static_cast<uint32_t>(lane * bs * key_row),
                 keys + seq_keys + static_cast<size_t>(my_block) * bs * key_row, bytes, bar);
}

__device__ __forceinline__ void issue_remote(const unsigned char* keys, unsigned char* dst,
                                             const int* sel, int top, int bs, size_t key_row,
                                             size_t seq_keys, uint32_t bar) {
    uint32_t total = 0;
    for (int r = 0; r < top; ++r) total += static_cast<uint32_t>(sel[3 * r + 2] * key_row);
    mbar_expect_tx(bar, total);
    for (int r = 0; r < top; ++r)
        if (sel[3 * r + 2] > 0)
            bulk_g2s(smem_u32(dst) + static_cast<uint32_t>(r * bs * key_row),
                     keys + seq_keys + static_cast<size_t>(sel[3 * r]) * bs * key_row,
                     static_cast<uint32_t>(sel[3 * r + 2] * key_row), bar);
}

// The selection of one query row by the whole CTA.  kMulti: called in a loop by the multi-anchor
// kernel (one call per slot and phase): the caller has already ordered itself after earlier
// kernels, hands in the four mbarriers of this call, and in partner-only mode the partner queries
// are completed here with the anchor's row of the partner-anchor cache.
// kResident (decode form): the sequence's whole key caches up to the position are requested at entry
// in place of the local windows, so the remote blocks need no second round of copies once they
// are picked — two dependent memory round trips fewer per row, for contexts whose caches fit the
// shared memory (2 x T x 128 bytes at 16 bits).
template <bool kBf16, bool kDecode, bool kMulti, bool kResident = false>
__device__ __forceinline__ void select_row(const SelectArgs& a, const int row, unsigned char* smem,
                                           const uint32_t bars) {
    __shared__ uint32_t warp_key[2 * kWarps];
    __shared__ int warp_pos[2 * kWarps];
    __shared__ int excl_s[kMaxExclude];
    __shared__ float softplus_s[8];
    // kDecode: the packed operator in its decode form (a row per sequence, one position for all, no
    // exclusion list): the other forms' branches fold away
    const int mode = kDecode ? static_cast<int>(kPacked) : a.mode;
    const int32_t* row_batch = kDecode ? nullptr : a.row_batch;
    const int32_t* row_position = kDecode ? nullptr : a.row_position;
    const int32_t* exclude_list = kDecode ? nullptr : a.exclude_list;
    const int key_dtype = kBf16 ? RLM_BF16 : a.key_dtype, stats_dtype = kBf16 ? RLM_BF16 : a.stats_dtype,
              query_dtype = kBf16 ? RLM_BF16 : a.query_dtype;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool do_anchor = mode != kPartnerOnly, do_partner = mode != kAnchorOnly;
    const int buckets4 = 4 * a.buckets;

    // Decode form: the caches, statistics and the position were written before the previous
    // kernel of the stream started, so everything up to the bulk-copy requests may run while
    // that kernel (the query projection) is still executing; only the queries wait for it.
    // The per-row form and exclusion lists take indices from arbitrary producers: wait first.
    const bool early = row_position == nullptr && row_batch == nullptr && exclude_list == nullptr &&
                       mode != kPartnerOnly;
    if (!early && !kMulti) griddep_sync();
    // threads 32..35 / 36..39 evaluate softplus(gamma) of the anchor / partner heads for everybody
    const bool sp_thread = tid >= 32 && tid < 40 && (tid < 36 ? do_anchor : do_partner);
    float gamma = 0.0f, ba = 0.0f, bp_ = 0.0f;
    if (sp_thread) gamma = load_scalar(tid < 36 ? a.anchor_gamma : a.partner_gamma, tid & 3, a.param_dtype);
    if (tid < buckets4) {
        if (do_anchor) ba = load_scalar(a.anchor_bias, tid, a.param_dtype);
        if (do_partner) bp_ = load_scalar(a.partner_bias, tid, a.param_dtype);
    }
    const int b = row_batch ? row_batch[row] : row;
    const int t = row_position ? row_position[row] : static_cast<int>(*a.position);
    if (b < 0 || b >= a.n_seq || t < 0 || t >= a.max_t) {
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
        // keep the stream's ordering chain intact on this path too: a kernel launched after this
        // one relies on "my predecessor has waited for its own predecessor"
        if (early && !kMulti) griddep_sync();
        return;
    }
    const int nb = a.n_blocks, bs = a.block_size, L = a.local_window, top = a.top_blocks;
    const int bs_shift = (bs & (bs - 1)) == 0 ? 31 - __clz(bs) : -1;
    const int ks = key_dtype == RLM_F32 ? 4 : 2, ss = stats_dtype == RLM_F32 ? 4 : 2;
    const Plan& p = a.plan;

    float* queries = reinterpret_cast<float*>(smem + p.queries);
    float* aq = queries, *arq = queries + kD, *pq = queries + 2 * kD, *prq = queries + 3 * kD;
    float* params = reinterpret_cast<float*>(smem + p.params);
    float* bias_a = params, *bias_p = params + buckets4;
    float* bscore = reinterpret_cast<float*>(smem + p.block_scores);
    float* cand = reinterpret_cast<float*>(smem + p.cand);
    int* sel = reinterpret_cast<int*>(smem + p.sel);
    const uint32_t bar_a = bars, bar_p = bars + 8, bar_ra = bars + 16, bar_rp = bars + 24;

    const int ls = max(t - L + 1, 0);
    const int first_local = ls - (t - L + 1);       // first valid slot of the local window
    const int n_local = t - ls + 1;
    const int n_complete = min((t + 1) / bs, nb);
    const size_t key_row = static_cast<size_t>(kD) * ks, stat_row = static_cast<size_t>(kD) * ss;
    const size_t seq_keys = static_cast<size_t>(b) * a.max_t * key_row;
    const size_t seq_stats = static_cast<size_t>(b) * nb * stat_row;
    const int cap = L + top * bs, cap4 = (cap + 3) & ~3;
    // resident form: row r of the window is position t - L + 1 + r of the resident cache (rows before
    // position 0 are never valid, hence never read)
    const ptrdiff_t window_offset = kResident ? static_cast<ptrdiff_t>(t - L + 1) * static_cast<ptrdiff_t>(key_row) : 0;

    if (tid == 0) {
        // the issuing thread initialises the barriers itself; the others first touch them
        // after the block-wide barrier below
        for (int i = 0; i < 4; ++i) mbar_init(bars + 8 * i, 1);
        fence_barrier_init();
        const uint32_t sbytes = top > 0 ? static_cast<uint32_t>(n_complete * stat_row) : 0u;
        // resident form: positions 0 .. t at rows 0 .. t; otherwise the local window at its slots
        const uint32_t lbytes = static_cast<uint32_t>((kResident ? t + 1 : n_local) * key_row);
        const size_t loff = seq_keys + (kResident ? 0 : static_cast<size_t>(ls) * key_row);
        const uint32_t ldst = kResident ? 0u : static_cast<uint32_t>(first_local * key_row);
        if (do_anchor) {
            mbar_expect_tx(bar_a, 2 * sbytes + lbytes);
            if (sbytes) {
                bulk_g2s(smem_u32(smem + p.a_mean), static_cast<const char*>(a.anchor_mean) + seq_stats, sbytes, bar_a);
                bulk_g2s(smem_u32(smem + p.a_std), static_cast<const char*>(a.anchor_std) + seq_stats, sbytes, bar_a);
            }
            bulk_g2s(smem_u32(smem + p.a_local) + ldst, static_cast<const char*>(a.anchor_keys) + loff, lbytes, bar_a);
        }
        if (do_partner && !a.shared_streams) {
            mbar_expect_tx(bar_p, 2 * sbytes + lbytes);
            if (sbytes) {
                bulk_g2s(smem_u32(smem + p.p_mean), static_cast<const char*>(a.partner_mean) + seq_stats, sbytes, bar_p);
                bulk_g2s(smem_u32(smem + p.p_std), static_cast<const char*>(a.partner_std) + seq_stats, sbytes, bar_p);
            }
            bulk_g2s(smem_u32(smem + p.p_local) + ldst, static_cast<const char*>(a.partner_keys) + loff, lbytes, bar_p);
        }
    }
    if (early && !kMulti) griddep_sync();
    // this thread's query element
    float qv = 0.0f;
    if (mode == kPacked) {
        if (tid < kD) qv = load_scalar(a.anchor_query, row * a.aq_stride + tid, query_dtype);
        else if (tid < 2 * kD) qv = load_scalar(a.anchor_router_query, row * a.arq_stride + tid - kD, query_dtype);
        else qv = load_scalar(a.partner_base, row * a.pbase_stride + tid - 2 * kD, query_dtype);
    } else if (mode == kAnchorOnly) {
        if (tid < kD) qv = load_scalar(a.anchor_query, row * a.aq_stride + tid, query_dtype);
        else if (tid < 2 * kD) qv = load_scalar(a.anchor_router_query, row * a.arq_stride + tid - kD, query_dtype);
    } else {
        if (tid < kD) qv = load_scalar(a.partner_base, row * a.pbase_stride + tid, query_dtype);
        else if (tid < 2 * kD) qv = load_scalar(a.partner_router_query, row * a.prq_stride + tid - kD, query_dtype);
    }
    // queries[0..255]: packed = aq | arq | partner base (exact 64 | router 64);
    // partner-only = (unused 128) | pq | prq; anchor-only = aq | arq
    if (mode == kPartnerOnly) { if (tid < 2 * kD) queries[2 * kD + tid] = qv; }
    else if (mode == kPacked || tid < 2 * kD) queries[tid] = qv;
    if (tid < buckets4) { bias_a[tid] = ba; bias_p[tid] = bp_; }
    for (int i = tid + kThreads; i < buckets4; i += kThreads) {      // bias tables wider than the CTA
        if (do_anchor) bias_a[i] = load_scalar(a.anchor_bias, i, a.param_dtype);
        if (do_partner) bias_p[i] = load_scalar(a.partner_bias, i, a.param_dtype);
    }
    if (tid < cap4 - cap) cand[cap + tid] = kNegInf;   // padding slots never win a comparison
    const int n_excl = exclude_list ? a.exclude_count : 0;
    if (tid < n_excl) excl_s[tid] = exclude_list[static_cast<size_t>(row) * n_excl + tid];
    // softplus of the heads' gammas, evaluated while the bulk copies fly
    if (sp_thread) softplus_s[tid - 32] = canon_log(__fadd_rn(1.0f, canon_exp(gamma)));
    const float* sp_a = softplus_s, *sp_p = softplus_s + 4;
    __syncthreads();

    // With remote blocks, half of the warps score blocks (eight lanes per block) while the other
    // half scores the local window (a lane per row); without, everybody scores rows.
    const bool split = top > 0;
    const int block_warps = split ? kWarps / 2 : 0;
    const int row_wi = warp - block_warps, row_nw = kWarps - block_warps;

    int anchor_pos = 0;
    if (do_anchor) {
        bool ok = mbar_wait(bar_a, 0);
        if (__syncthreads_or(!ok)) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
            return;
        }
        uint32_t bk = 0;
        int bp = 0x7fffffff;
        if (warp < block_warps)
            score_blocks_any<kBf16>(smem + p.a_mean, smem + p.a_std, stats_dtype, nb, n_complete, bs, t, ls,
                                    a.strict_valid, a.buckets, arq, sp_a, bias_a, bscore, warp, block_warps);
        else
            score_rows<kBf16>(smem + p.a_local + window_offset, key_dtype, L, nullptr, bs, first_local, t - L + 1, -1,
                       excl_s, n_excl, aq, nullptr, 0, row_wi, row_nw, bk, bp, 0u, ok, a.sm_count);
        if (lane == 0) { warp_key[warp] = bk; warp_pos[warp] = bp; }
        __syncthreads();
        if (a.shared_streams && tid == kThreads - 1) {
            // every warp has read the anchor's statistics and local window: the partner's take
            // their place while the anchor's remote blocks are fetched and scored
            const uint32_t sbytes = top > 0 ? static_cast<uint32_t>(n_complete * stat_row) : 0u;
            const uint32_t lbytes = static_cast<uint32_t>(n_local * key_row);
            const size_t loff = seq_keys + static_cast<size_t>(ls) * key_row;
            fence_proxy_async();
            mbar_expect_tx(bar_p, 2 * sbytes + lbytes);
            if (sbytes) {
                bulk_g2s(smem_u32(smem + p.p_mean), static_cast<const char*>(a.partner_mean) + seq_stats, sbytes, bar_p);
                bulk_g2s(smem_u32(smem + p.p_std), static_cast<const char*>(a.partner_std) + seq_stats, sbytes, bar_p);
            }
            bulk_g2s(smem_u32(smem + p.p_local) + static_cast<uint32_t>(first_local * key_row),
                     static_cast<const char*>(a.partner_keys) + loff, lbytes, bar_p);
        }
        if (top > 0) {
            if (warp == 0) {
                if (kResident) {
                    pick_blocks(bscore, nb, top, bs, ls, sel);
                } else if (nb <= 128 && top <= 32) {
                    pick_and_issue(bscore, nb, top, bs, ls, sel, static_cast<const unsigned char*>(a.anchor_keys),
                                   smem + p.remote, key_row, seq_keys, bar_ra);
                } else {
                    pick_blocks(bscore, nb, top, bs, ls, sel);
                    if (lane == 0)
                        issue_remote(static_cast<const unsigned char*>(a.anchor_keys), smem + p.remote, sel,
                                     top, bs, key_row, seq_keys, bar_ra);
                }
            }
            __syncthreads();
            bk = 0;
            bp = 0x7fffffff;
            if (kResident)      // the picked blocks' rows are already here, at their positions
                score_rows<kBf16, true>(smem + p.a_local, key_dtype, top * bs, sel, bs, 0, 0, -1, excl_s, n_excl, aq,
                                        nullptr, 0, warp, kWarps, bk, bp, 0u, ok, a.sm_count);
            else                // each warp works out its rows' positions first and only then waits for the copies
                score_rows<kBf16>(smem + p.remote, key_dtype, top * bs, sel, bs, 0, 0, -1, excl_s, n_excl, aq,
                           nullptr, 0, warp, kWarps, bk, bp, bar_ra, ok, a.sm_count);
            if (lane == 0) { warp_key[kWarps + warp] = bk; warp_pos[kWarps + warp] = bp; }
            if (__syncthreads_or(!ok)) {
                if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
                return;
            }
        }
        // Highest score wins; equal scores go to the lowest position (the reference's
        // left-most local arg-max followed by its "equal and earlier" merge rule).
        const int entries = top > 0 ? 2 * kWarps : kWarps;
        uint32_t best_key = lane < entries ? warp_key[lane] : 0u;
        anchor_pos = lane < entries ? warp_pos[lane] : 0x7fffffff;
        if (anchor_pos == 0x7fffffff) best_key = 0u;
        warp_argmax_key(best_key, anchor_pos);
        if (anchor_pos == 0x7fffffff) {   // every candidate was excluded
            anchor_pos = 0;
            best_key = float_key(kNegInf);
        }
        if (tid == 0) {
            a.out_anchor[row] = anchor_pos;
            a.out_anchor_score[row] = key_float(best_key);
        }
        if (!do_partner) return;
        // The anchor's contribution to the partner queries: one 2 x 64 row of the partner-anchor
        // cache, read straight from global memory by the threads that own the elements (one
        // dependent round trip, no staging).  The block-wide barrier below publishes pq / prq.
        if (tid < 2 * kD) {
            const float add = load_scalar(a.partner_anchor_cache,
                                          (static_cast<size_t>(b) * a.max_t + anchor_pos) * 2 * kD + tid, key_dtype);
            pq[tid] = __fadd_rn(pq[tid], add);   // pq[64..127] is prq
        }
    } else {
        anchor_pos = a.anchor_index_in[row];
        if (kMulti && tid < 2 * kD) {
            // factorised partner queries of a multi-anchor slot: query-side base + the anchor's cached row
            const float add = load_scalar(a.partner_anchor_cache,
                                          (static_cast<size_t>(b) * a.max_t + anchor_pos) * 2 * kD + tid, key_dtype);
            pq[tid] = __fadd_rn(pq[tid], add);   // written by this very thread above; pq[64..127] is prq
        }
    }

    bool okp = mbar_wait(bar_p, 0);
    if (__syncthreads_or(!okp)) {   // also publishes pq / prq
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
        return;
    }
    uint32_t dk = 0;
    int dp = 0x7fffffff;
    if (warp < block_warps)
        score_blocks_any<kBf16>(smem + p.p_mean, smem + p.p_std, stats_dtype, nb, n_complete, bs, t, ls,
                                a.strict_valid, a.buckets, prq, sp_p, bias_p, bscore, warp, block_warps);
    else
        score_rows<kBf16>(smem + p.p_local + window_offset, key_dtype, L, nullptr, bs, first_local, t - L + 1, anchor_pos,
                   excl_s, n_excl, pq, cand, 0, row_wi, row_nw, dk, dp, 0u, okp, a.sm_count);
    __syncthreads();
    if (top > 0) {
        if (warp == 0) {
            if (kResident) {
                pick_blocks(bscore, nb, top, bs, ls, sel);
            } else if (nb <= 128 && top <= 32) {
                pick_and_issue(bscore, nb, top, bs, ls, sel, static_cast<const unsigned char*>(a.partner_keys),
                               smem + p.remote, key_row, seq_keys, bar_rp);
            } else {
                pick_blocks(bscore, nb, top, bs, ls, sel);
                if (lane == 0) {
                    fence_proxy_async();   // the anchor phase read this buffer through the generic proxy
                    issue_remote(static_cast<const unsigned char*>(a.partner_keys), smem + p.remote, sel, top,
                                 bs, key_row, seq_keys, bar_rp);
                }
            }
        }
        __syncthreads();
        bool ok = true;
        if (kResident)
            score_rows<kBf16, true>(smem + p.p_local, key_dtype, top * bs, sel, bs, 0, 0, anchor_pos, excl_s, n_excl, pq,
                                    cand, L, warp, kWarps, dk, dp, 0u, ok, a.sm_count);
        else
            score_rows<kBf16>(smem + p.remote, key_dtype, top * bs, sel, bs, 0, 0, anchor_pos, excl_s, n_excl, pq,
                       cand, L, warp, kWarps, dk, dp, bar_rp, ok, a.sm_count);
        if (__syncthreads_or(!ok)) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
            return;
        }
    }
    // Exact top-K of the candidate table: output slot k holds the k-th best candidate (higher
    // score first, equal scores by the earlier slot); results without a finite score report
    // score -inf and the position of candidate slot 0.
    const int K = a.k_out;
    if (cap4 <= 256) {
        // Up to 256 candidate slots: warp 0 holds them all in registers (see topk_tournament)
        if (warp == 0) {
            if (cap4 <= 128)
                topk_tournament<4>(cand, cap4, K, L, t, bs, bs_shift, sel, a.out_partner + static_cast<size_t>(row) * K,
                                   a.out_partner_score + static_cast<size_t>(row) * K);
            else
                topk_tournament<8>(cand, cap4, K, L, t, bs, bs_shift, sel, a.out_partner + static_cast<size_t>(row) * K,
                                   a.out_partner_score + static_cast<size_t>(row) * K);
        }
        return;
    }
    topk_large(cand, cap, K, L, t, bs, sel, a.out_partner + static_cast<size_t>(row) * K,
               a.out_partner_score + static_cast<size_t>(row) * K);
}

// Validation and shared-memory plan of a selector launch: everything but the launch itself.
int prepare(SelectArgs& a, bool& many_rows, bool allow_resident = false) {
    if (a.n_rows < 0 || a.n_seq < 1 || a.max_t < 1 || a.n_blocks < 1 || a.buckets < 1 ||
        a.local_window < 1 || a.top_blocks < 0 || a.max_t % a.n_blocks != 0) {
        set_error("relation_select: sizes must be positive and T a multiple of the block count");
        return RLM_ERR_SHAPE;
    }
    if (a.mode != kAnchorOnly && (a.k_out < 1 || a.k_out > kMaxKOut)) {
        set_error("relation_select: k_out must be between 1 and 32");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(a.query_dtype) || !valid_dtype(a.key_dtype) || !valid_dtype(a.stats_dtype) ||
        !valid_dtype(a.param_dtype)) {
        set_error("relation_select: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    if (a.exclude_list && (a.exclude_count < 0 || a.exclude_count > kMaxExclude)) {
        set_error("relation_select: at most 8 excluded positions per query");
        return RLM_ERR_SHAPE;
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
    a.shared_streams = 0;
    a.plan = make_plan(a.n_blocks, a.block_size, a.local_window, a.top_blocks, a.buckets,
                       dtype_size(a.key_dtype), dtype_size(a.stats_dtype), a.mode, false);
    // More rows than the SMs hold at once: rows in flight set the throughput, so the packed
    // selector stages the two streams one after the other in the same buffers and the build
    // with the smaller register budget runs.
    const int kSms = sm_count();
    a.sm_count = kSms;
    const int resident = kSmemPerCta / (a.plan.total + 1024 + 2304);
    many_rows = a.n_rows > kSms * (resident < 3 ? resident : 3);
    if (many_rows && a.mode == kPacked) {
        a.shared_streams = 1;
        a.plan = make_plan(a.n_blocks, a.block_size, a.local_window, a.top_blocks, a.buckets,
                           dtype_size(a.key_dtype), dtype_size(a.stats_dtype), a.mode, true);
    }
    // At most one row per SM, 16-bit bf16 decode form, caches that fit: stage the whole key caches
    // (see select_row, kResident)
    a.resident = 0;
    if (allow_resident && !many_rows && a.n_rows <= kSms && a.mode == kPacked && !a.row_batch && !a.row_position &&
        !a.exclude_list && a.top_blocks > 0 && a.query_dtype == RLM_BF16 && a.key_dtype == RLM_BF16 &&
        a.stats_dtype == RLM_BF16) {
        const Plan whole = make_plan(a.n_blocks, a.block_size, a.local_window, a.top_blocks, a.buckets,
                                     dtype_size(a.key_dtype), dtype_size(a.stats_dtype), a.mode, false, a.max_t);
        if (whole.total <= kSmemDynamicLimit - 4096) {
            a.plan = whole;
            a.resident = 1;
        }
    }
    const Plan& plan = a.plan;
    if (plan.total > kSmemDynamicLimit) {
        set_error("relation_select: block statistics + local window + remote blocks exceed 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    return RLM_OK;
}

}  // namespace
}  // namespace rlm
