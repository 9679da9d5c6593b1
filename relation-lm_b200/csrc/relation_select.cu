// Routed anchor/partner selection for sm_100a.
//
// One CTA per query row.  Everything a row needs is staged in shared memory by
// untiled bulk (TMA) copies that complete on mbarriers: both streams' block
// statistics and local key windows are requested at kernel entry; the chosen
// remote blocks are requested as soon as the block ranks are known, and the one
// partner-anchor cache row is read directly from global memory.  Key rows are
// scored from shared memory a lane per 64-wide row, block statistics with 8
// lanes per block (16-byte reads, bank-conflict free for 16-bit caches), in
// the canonical order documented in rlm_common.cuh, so the selected indices
// do not depend on the launch geometry.
//
// Semantics follow src/relation_lm/kernels/relation_select.py:50-308 and
// src/relation_lm/kernels/triton_select.py:23-252 of the reference project.

#include "relation_layer_tail_body.cuh"

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
    Plan plan;
};

__host__ __device__ inline int align16(int x) { return (x + 15) & ~15; }

// With `shared_streams` (packed mode only) the partner's statistics and local window take the
// anchor's place once the anchor's first scoring pass has read them: a smaller footprint, so
// more rows per SM, for launches of many rows.
__host__ __device__ inline Plan make_plan(int nb, int bs, int local, int top, int buckets,
                                          int key_size, int stats_size, int mode, bool shared_streams) {
    Plan p;
    int off = 0;
    int stats_bytes = nb * kD * stats_size;
    int local_bytes = local * kD * key_size;
    bool anchor = mode != kPartnerOnly, partner = mode != kAnchorOnly;
    p.a_mean = off; off += anchor ? stats_bytes : 0;
    p.a_std = off; off += anchor ? stats_bytes : 0;
    p.p_mean = shared_streams ? p.a_mean : off; off += partner && !shared_streams ? stats_bytes : 0;
    p.p_std = shared_streams ? p.a_std : off; off += partner && !shared_streams ? stats_bytes : 0;
    p.a_local = off; off += anchor ? local_bytes : 0;
    p.p_local = shared_streams ? p.a_local : off; off += partner && !shared_streams ? local_bytes : 0;
    p.remote = off; off += top * bs * kD * key_size;
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
template <bool kBf16>
__device__ __forceinline__ void score_rows(const unsigned char* rows, int key_dtype, int n_rows,
                                           const int* sel, int bs, int first_valid, int pos0,
                                           int exclude, const int* excl, int n_excl, const float* query,
                                           float* cand, int slot0, int wi, int nw, uint32_t& best_key,
                                           int& best_pos, uint32_t bar, bool& arrived, int sm_count_arg) {
    const int lanes = static_cast<int>(gridDim.x) <= sm_count_arg ? 32 * nw : 0;   // a row per lane when CTAs share the SMs: fewer instructions in total
    if (4 * n_rows <= lanes)
        score_rows_split<kBf16, 4>(rows, key_dtype, n_rows, sel, bs, first_valid, pos0, exclude, excl, n_excl,
                                   query, cand, slot0, wi, nw, best_key, best_pos, bar, arrived);
    else if (2 * n_rows <= lanes)
        score_rows_split<kBf16, 2>(rows, key_dtype, n_rows, sel, bs, first_valid, pos0, exclude, excl, n_excl,
                                   query, cand, slot0, wi, nw, best_key, best_pos, bar, arrived);
    else
        score_rows_split<kBf16, 1>(rows, key_dtype, n_rows, sel, bs, first_valid, pos0, exclude, excl, n_excl,
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

// kMinCtas = 3: the latency-oriented build (decode batches: one wave or less).  kMinCtas = 4:
// launches of many rows, where rows in flight per SM set the throughput.  kBf16: queries, key
// caches and block statistics are all bf16 (the decode configuration); the dtype branches
// fold away, which matters because a row's time is largely instruction fetch.
// The selection of one query row by the whole CTA.  kMulti: called in a loop by the multi-anchor
// kernel (one call per slot and phase): the caller has already ordered itself after earlier
// kernels, hands in the four mbarriers of this call, and in partner-only mode the partner queries
// are completed here with the anchor's row of the partner-anchor cache.
template <bool kBf16, bool kDecode, bool kMulti>
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

    if (tid == 0) {
        // the issuing thread initialises the barriers itself; the others first touch them
        // after the block-wide barrier below
        for (int i = 0; i < 4; ++i) mbar_init(bars + 8 * i, 1);
        fence_barrier_init();
        const uint32_t sbytes = top > 0 ? static_cast<uint32_t>(n_complete * stat_row) : 0u;
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
            score_rows<kBf16>(smem + p.a_local, key_dtype, L, nullptr, bs, first_local, t - L + 1, -1, excl_s,
                       n_excl, aq, nullptr, 0, row_wi, row_nw, bk, bp, 0u, ok, a.sm_count);
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
                if (nb <= 128 && top <= 32) {
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
            // each warp works out its rows' positions first and only then waits for the copies
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
        score_rows<kBf16>(smem + p.p_local, key_dtype, L, nullptr, bs, first_local, t - L + 1, anchor_pos,
                   excl_s, n_excl, pq, cand, 0, row_wi, row_nw, dk, dp, 0u, okp, a.sm_count);
    __syncthreads();
    if (top > 0) {
        if (warp == 0) {
            if (nb <= 128 && top <= 32) {
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

template <int kMinCtas, bool kBf16, bool kDecode>
__global__ void __launch_bounds__(kThreads, kMinCtas) relation_select_kernel(const SelectArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    select_row<kBf16, kDecode, false>(a, blockIdx.x, smem, smem_u32(smem + a.plan.bars));
}

// ---- routed multi-anchor selection: S anchor slots per query row, one launch
//
// Rules of the reference's dense multi-anchor layer (src/relation_lm/models/multi_relation_blocks.py)
// applied inside each slot's routed candidate set: slot s is active for a query at position t iff
// s <= t (:82-84); slots choose their anchors one after another and a position taken by an earlier
// slot is barred (:86-93); an inactive slot reports anchor 0 (:94); the partner selection of every
// slot bars the anchors of all active slots (:133-139); an inactive slot has no partners
// (:140-142); a partner slot is active iff its score is finite (:144-147).  Every slot has its own
// key caches, block statistics and router parameters (leading slot dimension).
constexpr int kMaxSlots = kMaxExclude;

struct MultiSelectArgs {
    SelectArgs base;               // slot 0's pointers; per-slot strides below (bytes)
    Plan plan_anchor, plan_partner;
    int slots;
    size_t keys_slot, pac_slot, stats_slot, gamma_slot, bias_slot;   // bytes between slots
    int32_t* out_anchor;           // [N, S]
    float* out_anchor_score;       // [N, S]
    uint8_t* out_anchor_active;    // [N, S]
    int32_t* out_partner;          // [N, S, K]
    float* out_partner_score;      // [N, S, K]
};

__device__ __forceinline__ const void* slot_ptr(const void* p, size_t bytes) {
    return static_cast<const char*>(p) + bytes;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 3) relation_select_multi_kernel(const MultiSelectArgs m) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long call_bars[4 * 2 * kMaxSlots];
    __shared__ int taken_s[kMaxSlots];
    const int row = blockIdx.x, tid = threadIdx.x;
    const int S = m.slots, K = m.base.k_out;
    griddep_sync();
    const int b = m.base.row_batch[row], t = m.base.row_position[row];
    if (b < 0 || b >= m.base.n_seq || t < 0 || t >= m.base.max_t) {
        if (tid == 0 && m.base.status) atomicOr(m.base.status, RLM_DEV_POSITION);
        return;
    }
    if (tid < kMaxSlots) taken_s[tid] = -1;
    __syncthreads();
    const int esz = m.base.query_dtype == RLM_F32 ? 4 : 2;
    // anchors: slot after slot, each barring the positions taken before it
    for (int s = 0; s < S; ++s) {
        const bool slot_live = s <= t;
        int32_t* out_idx = m.out_anchor + static_cast<size_t>(row) * S + s;
        float* out_sc = m.out_anchor_score + static_cast<size_t>(row) * S + s;
        if (slot_live) {
            SelectArgs a = m.base;
            a.mode = kAnchorOnly;
            a.plan = m.plan_anchor;
            a.anchor_query = slot_ptr(m.base.anchor_query, static_cast<size_t>(s) * kD * esz);
            a.anchor_router_query = slot_ptr(m.base.anchor_router_query, static_cast<size_t>(s) * kD * esz);
            a.anchor_keys = slot_ptr(m.base.anchor_keys, s * m.keys_slot);
            a.anchor_mean = slot_ptr(m.base.anchor_mean, s * m.stats_slot);
            a.anchor_std = slot_ptr(m.base.anchor_std, s * m.stats_slot);
            a.anchor_gamma = slot_ptr(m.base.anchor_gamma, s * m.gamma_slot);
            a.anchor_bias = slot_ptr(m.base.anchor_bias, s * m.bias_slot);
            a.exclude_list = s > 0 ? taken_s - static_cast<ptrdiff_t>(row) * s : nullptr;   // [row * s + i] == taken_s[i]
            a.exclude_count = s;
            a.out_anchor = out_idx - row;                    // [row] lands on (row, s)
            a.out_anchor_score = out_sc - row;
            select_row<kBf16, false, true>(a, row, smem, smem_u32(&call_bars[4 * s]));
        }
        __syncthreads();
        if (tid == 0) {                                      // the thread that stored the slot's result
            const bool live = slot_live && *out_sc > kNegInf;
            if (!live) { *out_idx = 0; *out_sc = kNegInf; }
            taken_s[s] = live ? *out_idx : -1;
            m.out_anchor_active[static_cast<size_t>(row) * S + s] = live ? 1 : 0;
        }
        __syncthreads();
    }
    // partners: every live slot bars the anchors of all slots
    for (int s = 0; s < S; ++s) {
        int32_t* out_idx = m.out_partner + (static_cast<size_t>(row) * S + s) * K;
        float* out_sc = m.out_partner_score + (static_cast<size_t>(row) * S + s) * K;
        const bool live = taken_s[s] >= 0;
        if (live) {
            SelectArgs a = m.base;
            a.mode = kPartnerOnly;
            a.plan = m.plan_partner;
            a.partner_base = slot_ptr(m.base.partner_base, static_cast<size_t>(s) * 2 * kD * esz);
            a.partner_router_query = slot_ptr(m.base.partner_base, (static_cast<size_t>(s) * 2 * kD + kD) * esz);
            a.prq_stride = m.base.pbase_stride;
            a.partner_anchor_cache = slot_ptr(m.base.partner_anchor_cache, s * m.pac_slot);
            a.partner_keys = slot_ptr(m.base.partner_keys, s * m.keys_slot);
            a.partner_mean = slot_ptr(m.base.partner_mean, s * m.stats_slot);
            a.partner_std = slot_ptr(m.base.partner_std, s * m.stats_slot);
            a.partner_gamma = slot_ptr(m.base.partner_gamma, s * m.gamma_slot);
            a.partner_bias = slot_ptr(m.base.partner_bias, s * m.bias_slot);
            a.anchor_index_in = taken_s + s - row;           // [row] == taken_s[s]
            a.exclude_list = taken_s - static_cast<ptrdiff_t>(row) * S;
            a.exclude_count = S;
            a.out_partner = out_idx - static_cast<ptrdiff_t>(row) * K;
            a.out_partner_score = out_sc - static_cast<ptrdiff_t>(row) * K;
            select_row<kBf16, false, true>(a, row, smem, smem_u32(&call_bars[4 * (S + s)]));
        }
        __syncthreads();
        if (tid < K) {                                       // the threads that stored the slot's results
            if (!live || !(out_sc[tid] > kNegInf)) { out_idx[tid] = 0; out_sc[tid] = kNegInf; }
        }
        __syncthreads();
    }
}

// ---- whole-sequence (prefill) selection: a tile of consecutive positions per CTA
//
// Query row (b, t) of a whole-sequence pass sees the same block statistics as its neighbours (the
// complete blocks at t) and a local window that overlaps theirs in all but one row.  One CTA
// therefore serves a tile of consecutive positions of one sequence: the statistics of both
// streams and the union of the tile's local windows are staged in shared memory once, then every
// warp takes the tile's queries one at a time and walks the whole chain for its query on its own
// — block scores, local scores, block picking, remote scores (read where the blocks lie, from
// L2), anchor, partner queries, partner scores, top-K — with warp-level synchronisation only.
// The arithmetic is the per-row kernel's own (the same device functions), so indices and scores
// are bit-identical to relation_select_kernel's.
// CTAs of kTileWarps warps serve 4 kTileWarps positions (16 warps when the shared memory allows, else 8).

// ---- warp-per-query primitives (16-bit bf16 caches).  The arithmetic is the canonical one: every
// sum below is a sum of the per-row kernel with its operands possibly swapped, so scores are
// bit-identical.  A lane owns a whole key row (or block) and keeps the 64-wide query in
// registers, paired for the two-wide fma: v[c][j] = (q[16 c + j], q[16 c + 8 + j]), element j of
// chunks 2c and 2c + 1.  Staged rows are kPadRow bytes apart, so the eight lanes of a quarter
// warp read eight different 16-byte chunk indices without rotating their chunk order.
constexpr uint32_t kPadRow = 2 * kD + 16;

struct QueryRegs { float2 v[4][8]; };

// Shared-memory copies of a query keep the same pairing (element e at paired_index(e)), so that
// a 16-byte load fills two register pairs as they are used.
__device__ __forceinline__ int paired_index(int e) { return (e & ~15) | ((e & 7) << 1) | ((e >> 3) & 1); }

__device__ __forceinline__ void load_query_regs(const float* paired, QueryRegs& r) {
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const float4 v = *reinterpret_cast<const float4*>(paired + 16 * c + 4 * m);
            r.v[c][2 * m] = make_float2(v.x, v.y);
            r.v[c][2 * m + 1] = make_float2(v.z, v.w);
        }
}

// seg8(chunk 2c, q) + seg8(chunk 2c + 1, q): the two chains advance together in one two-wide fma
__device__ __forceinline__ float pair_dot_bf16(const uint4 w0, const uint4 w1, const float2 (&q)[8]) {
    const uint32_t a[4] = {w0.x, w0.y, w0.z, w0.w}, b[4] = {w1.x, w1.y, w1.z, w1.w};
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc = __ffma2_rn(make_float2(__uint_as_float(a[i] << 16), __uint_as_float(b[i] << 16)), q[2 * i], acc);
        acc = __ffma2_rn(make_float2(__uint_as_float(a[i] & 0xffff0000u), __uint_as_float(b[i] & 0xffff0000u)),
                         q[2 * i + 1], acc);
    }
    return __fadd_rn(acc.x, acc.y);
}

// the same with |q| (the deviation term of the block scores)
__device__ __forceinline__ float pair_dot_abs_bf16(const uint4 w0, const uint4 w1, const float2 (&q)[8]) {
    const uint32_t a[4] = {w0.x, w0.y, w0.z, w0.w}, b[4] = {w1.x, w1.y, w1.z, w1.w};
    float x = 0.0f, y = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x = __fmaf_rn(__uint_as_float(a[i] << 16), fabsf(q[2 * i].x), x);
        y = __fmaf_rn(__uint_as_float(b[i] << 16), fabsf(q[2 * i].y), y);
        x = __fmaf_rn(__uint_as_float(a[i] & 0xffff0000u), fabsf(q[2 * i + 1].x), x);
        y = __fmaf_rn(__uint_as_float(b[i] & 0xffff0000u), fabsf(q[2 * i + 1].y), y);
    }
    return __fadd_rn(x, y);
}

// score_rows_split<true, 1> for one warp with the query in registers (same arguments otherwise;
// no exclusion list, rows already in place).  `stride`: bytes between rows.
template <bool kAtPosition>
__device__ __forceinline__ void score_rows_warp(const unsigned char* rows, uint32_t stride, int n_rows, const int* sel,
                                                int bs, int bs_shift, int first_valid, int pos0, int exclude,
                                                const QueryRegs& q, float* cand, int slot0, uint32_t& best_key,
                                                int& best_pos) {
    const int lane = threadIdx.x & 31;
    uint32_t my_key = 0;
    int my_pos = 0x7fffffff;
    for (int base = 0; base < n_rows; base += 32) {
        const int r = base + lane;
        int pos;
        bool valid;
        if (sel) {
            const int rank = bs_shift >= 0 ? r >> bs_shift : r / bs, o = r - rank * bs;
            const bool in = r < n_rows;
            pos = in ? sel[3 * rank] * bs + o : -1;
            valid = in && o < sel[3 * rank + 2];
        } else {
            pos = pos0 + r;
            valid = r < n_rows && r >= first_valid;
        }
        valid = valid && pos != exclude;
        float sc = kNegInf;
        if (valid) {
            const uint4* row = reinterpret_cast<const uint4*>(rows + static_cast<size_t>(kAtPosition ? pos : r) * stride);
            uint4 w[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) w[c] = row[c];
            const float s01 = __fadd_rn(pair_dot_bf16(w[0], w[1], q.v[0]), pair_dot_bf16(w[2], w[3], q.v[1]));
            const float s23 = __fadd_rn(pair_dot_bf16(w[4], w[5], q.v[2]), pair_dot_bf16(w[6], w[7], q.v[3]));
            sc = __fmul_rn(__fadd_rn(s01, s23), 0.125f);
        }
        if (cand) {
            if (r < n_rows) cand[slot0 + r] = sc;
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

// Rows scored where they lie in the key cache (the picked remote blocks), one warp.  A lane that
// reads its own 128-byte row makes every load instruction of the warp touch 32 cache lines, and
// the L1 tag rate then bounds the whole selector; so a pass of 32 rows is fetched coalesced (a
// load instruction covers four whole rows: lane = 8 (row % 4) + chunk), parked in the warp's
// padded staging buffer (32 rows of kPadRow bytes) and scored from there a row per lane, exactly
// like the local window.  Arguments as score_rows_warp with sel != nullptr.
__device__ __forceinline__ void score_remote_warp(const unsigned char* keys, int n_rows, const int* sel, int bs,
                                                  int bs_shift, int exclude, const QueryRegs& q, unsigned char* stage,
                                                  float* cand, int slot0, uint32_t& best_key, int& best_pos) {
    const int lane = threadIdx.x & 31, chunk = lane & 7, rq = lane >> 3;
    uint32_t my_key = 0;
    int my_pos = 0x7fffffff;
    unsigned char* park = stage + rq * kPadRow + 16 * chunk;        // this lane's cell of rows rq, rq + 4, ...
    for (int base = 0; base < n_rows; base += 32) {
        int pos;                                         // position of row base + lane, or -1
        uint4 v[8];
        if (bs_shift >= 5) {
            // the pass lies in one picked block: rows base + 4 i + rq are 512 bytes apart
            const int rank = base >> bs_shift, o0 = base - (rank << bs_shift);
            const int first = sel[3 * rank] * bs, lim = sel[3 * rank + 2];
            const unsigned char* src = keys + static_cast<size_t>(first + o0 + rq) * (2 * kD) + 16 * chunk;
            // rows past `lim` are read too (they lie inside the block, hence inside the cache) and ignored
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = *reinterpret_cast<const uint4*>(src + i * (8 * kD));
            pos = o0 + lane < lim ? first + o0 + lane : -1;
        } else {
            auto row_pos = [&](int r) -> int {
                if (r >= n_rows) return -1;
                const int rank = bs_shift >= 0 ? r >> bs_shift : r / bs, o = r - rank * bs;
                return o < sel[3 * rank + 2] ? sel[3 * rank] * bs + o : -1;
            };
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int p = row_pos(base + 4 * i + rq);
                v[i] = make_uint4(0, 0, 0, 0);
                if (p >= 0) v[i] = *reinterpret_cast<const uint4*>(keys + static_cast<size_t>(p) * (2 * kD) + 16 * chunk);
            }
            pos = row_pos(base + lane);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(park + i * (4 * kPadRow)) = v[i];
        __syncwarp();
        const int r = base + lane;
        const bool valid = pos >= 0 && pos != exclude;
        float sc = kNegInf;
        if (valid) {
            const uint4* row = reinterpret_cast<const uint4*>(stage + lane * kPadRow);
            uint4 w[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) w[c] = row[c];
            const float s01 = __fadd_rn(pair_dot_bf16(w[0], w[1], q.v[0]), pair_dot_bf16(w[2], w[3], q.v[1]));
            const float s23 = __fadd_rn(pair_dot_bf16(w[4], w[5], q.v[2]), pair_dot_bf16(w[6], w[7], q.v[3]));
            sc = __fmul_rn(__fadd_rn(s01, s23), 0.125f);
        }
        __syncwarp();                                   // the staging buffer is free again
        if (cand) {
            if (r < n_rows) cand[slot0 + r] = sc;
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

// score_blocks for one warp, a block per lane with all four heads (no shuffles): out[n] for the
// first n_complete blocks, -inf up to the next multiple of four of nb.
__device__ __forceinline__ void score_blocks_warp(const unsigned char* mean, const unsigned char* stdv, uint32_t stride,
                                                  int nb, int n_complete, int bs, int t, int ls, int strict,
                                                  int buckets, const QueryRegs& rq, const float* sp4, const float* bias,
                                                  float* out) {
    const int lane = threadIdx.x & 31;
    for (int n = n_complete + lane; n < ((nb + 3) & ~3); n += 32) out[n] = kNegInf;
    for (int n = lane; n < n_complete; n += 32) {
        const int end = (n + 1) * bs - 1;
        int dist = t - end;
        if (dist < 0) dist = 0;
        int bucket = 31 - __clz(dist + 1);
        if (bucket > buckets - 1) bucket = buckets - 1;
        const uint4* m = reinterpret_cast<const uint4*>(mean + static_cast<size_t>(n) * stride);
        const uint4* sd4 = reinterpret_cast<const uint4*>(stdv + static_cast<size_t>(n) * stride);
        float sh[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const float md = pair_dot_bf16(m[2 * h], m[2 * h + 1], rq.v[h]);
            const float sd = pair_dot_abs_bf16(sd4[2 * h], sd4[2 * h + 1], rq.v[h]);
            sh[h] = __fadd_rn(__fmul_rn(__fadd_rn(md, __fmul_rn(sp4[h], sd)), 0.25f), bias[h * buckets + bucket]);
        }
        const float mx = fmaxf(fmaxf(sh[0], sh[1]), fmaxf(sh[2], sh[3]));
        const float e01 = __fadd_rn(canon_exp(__fsub_rn(sh[0], mx)), canon_exp(__fsub_rn(sh[1], mx)));
        const float e23 = __fadd_rn(canon_exp(__fsub_rn(sh[2], mx)), canon_exp(__fsub_rn(sh[3], mx)));
        const float acc = __fadd_rn(mx, canon_log(__fadd_rn(e01, e23)));
        out[n] = (!strict || end < ls) ? acc : kNegInf;
    }
}

// pick_blocks for one warp and up to 128 blocks: `top` rounds of (largest score, lowest block on
// ties) through two redux instructions each, instead of ranking every block against all others.
__device__ __forceinline__ void pick_blocks_warp(const float* scores, int nb, int top, int bs, int ls, int* sel) {
    const int lane = threadIdx.x & 31;
    uint32_t key[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = lane + 32 * i;
        const float v = n < nb ? scores[n] : kNegInf;
        key[i] = v > -1.0e30f ? float_key(v + 0.0f) : 0u;
    }
    for (int r = lane; r < top; r += 32) { sel[3 * r] = 0; sel[3 * r + 1] = 0; sel[3 * r + 2] = 0; }
    __syncwarp();
    for (int r = 0; r < top; ++r) {
        uint32_t mk = key[0];
        int mi = 0;
#pragma unroll
        for (int i = 1; i < 4; ++i)
            if (key[i] > mk) { mk = key[i]; mi = i; }
        const uint32_t best = __reduce_max_sync(0xffffffffu, mk);
        if (best == 0u) break;
        const int mine = mk == best ? lane + 32 * mi : 0x7fffffff;
        const int n = __reduce_min_sync(0xffffffffu, mine);
        if (mine == n) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i == mi) key[i] = 0u;
            int rows = ls - n * bs;
            rows = rows < 0 ? 0 : (rows > bs ? bs : rows);
            sel[3 * r] = n;
            sel[3 * r + 1] = 1;
            sel[3 * r + 2] = rows;
        }
    }
    __syncwarp();
}

// Exact top-K by one warp through a threshold: the K-th largest of the 32 lane maxima is a lower
// bound of the K-th largest score, so only candidates at or above it can be selected; they are
// compacted (64 words of `scratch`) and ranked exactly, higher score first and equal scores by the
// earlier slot, as topk_tournament orders them.  Returns false, with nothing written, when fewer
// than K lanes hold a finite score or more than 32 candidates pass (many equal scores): the
// caller then runs the tournament.
template <int kN>
__device__ __forceinline__ bool topk_filter(const float* cand, int cap4, int K, int L, int t, int bs, int bs_shift,
                                            const int* sel, uint32_t* scratch, int32_t* out_pos, float* out_score) {
    const int lane = threadIdx.x & 31;
    uint32_t k[kN], active = 0;
#pragma unroll
    for (int i = 0; i < kN; ++i) {
        const int slot = 32 * i + lane;
        k[i] = slot < cap4 ? float_key(cand[slot] + 0.0f) : 0u;
        active = max(active, k[i]);
    }
    uint32_t tau = 0;
    for (int r = 0; r < K; ++r) {
        tau = __reduce_max_sync(0xffffffffu, active);
        const int w = __ffs(__ballot_sync(0xffffffffu, active == tau)) - 1;
        if (lane == w) active = 0u;
    }
    if (tau <= float_key(kNegInf)) return false;
    int count = 0;
#pragma unroll
    for (int i = 0; i < kN; ++i) {
        const bool pass = k[i] >= tau;
        const unsigned b = __ballot_sync(0xffffffffu, pass);
        const int at = count + __popc(b & ((1u << lane) - 1u));
        if (pass && at < 32) {
            scratch[2 * at] = k[i];
            scratch[2 * at + 1] = static_cast<uint32_t>(32 * i + lane);
        }
        count += __popc(b);
    }
    if (count > 32) return false;
    __syncwarp();
    if (lane < count) {
        const uint32_t key = scratch[2 * lane], slot = scratch[2 * lane + 1];
        int rank = 0;
        for (int j = 0; j < count; ++j) {
            const uint32_t kj = scratch[2 * j], sj = scratch[2 * j + 1];
            rank += (kj > key) || (kj == key && sj < slot);
        }
        if (rank < K) {
            const float sc = cand[slot];
            const int cs = static_cast<int>(slot);
            int pos;
            if (!(sc > kNegInf)) pos = t - L + 1;
            else if (cs < L) pos = t - L + 1 + cs;
            else { const int rr = bs_shift >= 0 ? (cs - L) >> bs_shift : (cs - L) / bs; pos = sel[3 * rr] * bs + (cs - L - rr * bs); }
            out_pos[rank] = pos;
            out_score[rank] = sc;
        }
    }
    __syncwarp();
    return true;
}

struct TileArgs {
    SelectArgs base;          // packed mode; queries [n_seq * q_len, ...]; row = b * q_len + t
    int q_len;                // query positions 0 .. q_len - 1 of every sequence
    int warp_bytes, stats_bytes, window_rows, param_bytes;
};

template <bool kBf16, int kTileWarps>
__global__ void __launch_bounds__(32 * kTileWarps, 16 / kTileWarps) relation_select_tile_kernel(const TileArgs m) {
    constexpr int kTileQ = 4 * kTileWarps, kTileThreads = 32 * kTileWarps;
    extern __shared__ __align__(128) unsigned char smem[];
    const SelectArgs& a = m.base;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int key_dtype = kBf16 ? RLM_BF16 : a.key_dtype, stats_dtype = kBf16 ? RLM_BF16 : a.stats_dtype,
              query_dtype = kBf16 ? RLM_BF16 : a.query_dtype;
    const int tiles_per_seq = (m.q_len + kTileQ - 1) / kTileQ;
    const int b = blockIdx.x / tiles_per_seq, t0 = (blockIdx.x - b * tiles_per_seq) * kTileQ;
    const int t_end = min(t0 + kTileQ, m.q_len);               // exclusive
    const int nb = a.n_blocks, bs = a.block_size, L = a.local_window, top = a.top_blocks, K = a.k_out;
    const int bs_shift = (bs & (bs - 1)) == 0 ? 31 - __clz(bs) : -1;
    const int ks = key_dtype == RLM_F32 ? 4 : 2, ss = stats_dtype == RLM_F32 ? 4 : 2;
    const size_t key_row = static_cast<size_t>(kD) * ks, stat_row = static_cast<size_t>(kD) * ss;
    // bf16 rows are staged with 16 bytes of padding (see kPadRow); the other dtypes keep the
    // per-row kernel's scoring functions and their dense rows
    const uint32_t key_stride = kBf16 ? kPadRow : static_cast<uint32_t>(key_row);
    const uint32_t stat_stride = kBf16 ? kPadRow : static_cast<uint32_t>(stat_row);
    const int buckets4 = 4 * a.buckets;
    griddep_sync();

    // ---- shared staging: statistics of the blocks complete at the tile's last position, and the
    // union of the local windows: positions [w_lo, t_end)
    unsigned char* st[4] = {smem, smem + m.stats_bytes, smem + 2 * m.stats_bytes, smem + 3 * m.stats_bytes};
    unsigned char* win_a = smem + 4 * m.stats_bytes;
    unsigned char* win_p = win_a + static_cast<size_t>(m.window_rows) * key_stride;
    float* params = reinterpret_cast<float*>(win_p + static_cast<size_t>(m.window_rows) * key_stride);
    unsigned char* warp_base = reinterpret_cast<unsigned char*>(params) + m.param_bytes + static_cast<size_t>(warp) * m.warp_bytes;
    const int n_stage = top > 0 ? min(t_end / bs, nb) : 0;
    const int w_lo = max(t0 - L + 1, 0);
    const size_t seq_stats = static_cast<size_t>(b) * nb * stat_row, seq_keys = static_cast<size_t>(b) * a.max_t * key_row;
    {
        const char* src[4] = {static_cast<const char*>(a.anchor_mean) + seq_stats, static_cast<const char*>(a.anchor_std) + seq_stats,
                              static_cast<const char*>(a.partner_mean) + seq_stats, static_cast<const char*>(a.partner_std) + seq_stats};
        const int stat_cpr = static_cast<int>(stat_row / 16), key_cpr = static_cast<int>(key_row / 16);   // 16-byte chunks per row
        const int stat_chunks = n_stage * stat_cpr;
        for (int i = tid; i < 4 * stat_chunks; i += kTileThreads) {
            const int which = i / stat_chunks, c = i - which * stat_chunks;
            const int r = c / stat_cpr, cc = c - r * stat_cpr;
            cp_async16(smem_u32(st[which]) + r * stat_stride + 16 * cc, src[which] + 16 * c);
        }
        const int win_chunks = (t_end - w_lo) * key_cpr;
        const char* ka = static_cast<const char*>(a.anchor_keys) + seq_keys + w_lo * key_row;
        const char* kp = static_cast<const char*>(a.partner_keys) + seq_keys + w_lo * key_row;
        for (int i = tid; i < win_chunks; i += kTileThreads) {
            const int r = i / key_cpr, cc = i - r * key_cpr;
            cp_async16(smem_u32(win_a) + r * key_stride + 16 * cc, ka + 16 * i);
            cp_async16(smem_u32(win_p) + r * key_stride + 16 * cc, kp + 16 * i);
        }
        cp_async_commit();
    }
    // router parameters, shared by the warps: softplus a[4] p[4], bias a, bias p
    float* sp_a = params, *sp_p = params + 4, *bias_a = params + 8, *bias_p = bias_a + buckets4;
    for (int i = tid; i < buckets4; i += kTileThreads) {
        bias_a[i] = load_scalar(a.anchor_bias, i, a.param_dtype);
        bias_p[i] = load_scalar(a.partner_bias, i, a.param_dtype);
    }
    if (tid < 8) {
        const float gamma = load_scalar(tid < 4 ? a.anchor_gamma : a.partner_gamma, tid & 3, a.param_dtype);
        params[tid] = canon_log(__fadd_rn(1.0f, canon_exp(gamma)));
    }
    // per-warp scratch
    float* queries = reinterpret_cast<float*>(warp_base);                     // aq | arq | pq | prq
    uint32_t* short_list = reinterpret_cast<uint32_t*>(queries + 4 * kD);     // 64 words of the top-K filter
    float* bscore = reinterpret_cast<float*>(short_list + 64);
    float* cand = bscore + ((nb + 3) & ~3);
    const int cap = L + top * bs, cap4 = (cap + 3) & ~3;
    int* sel = reinterpret_cast<int*>(cand + cap4);
    unsigned char* stage = warp_base + m.warp_bytes - 32 * kPadRow;          // remote rows of a pass (bf16 caches)
    for (int i = cap + lane; i < cap4; i += 32) cand[i] = kNegInf;
    cp_async_wait_all();
    __syncthreads();

    for (int t = t0 + warp; t < t_end; t += kTileWarps) {
        const int row = b * m.q_len + t;
        const int ls = max(t - L + 1, 0), first_local = ls - (t - L + 1);
        const int n_complete = min((t + 1) / bs, nb);
        // this query's rows of the projections
        for (int i = lane; i < 4 * kD; i += 32) {
            float v;
            if (i < kD) v = load_scalar(a.anchor_query, row * a.aq_stride + i, query_dtype);
            else if (i < 2 * kD) v = load_scalar(a.anchor_router_query, row * a.arq_stride + i - kD, query_dtype);
            else v = load_scalar(a.partner_base, row * a.pbase_stride + i - 2 * kD, query_dtype);
            queries[kBf16 ? (i & ~(kD - 1)) | paired_index(i & (kD - 1)) : i] = v;
        }
        __syncwarp();
        const float* aq = queries, *arq = queries + kD;
        float* pq = queries + 2 * kD, *prq = queries + 3 * kD;
        // the query's window starts (t - L + 1 - w_lo) rows into the staged union (negative rows are never valid)
        const ptrdiff_t win_off = static_cast<ptrdiff_t>(t - L + 1 - w_lo) * static_cast<ptrdiff_t>(key_stride);
        const unsigned char* local_a = win_a + win_off;
        const unsigned char* local_p = win_p + win_off;
        const unsigned char* seq_a = static_cast<const unsigned char*>(a.anchor_keys) + seq_keys;
        const unsigned char* seq_p = static_cast<const unsigned char*>(a.partner_keys) + seq_keys;
        bool ok = true;
        // ---- anchor
        uint32_t bk = 0;
        int bp = 0x7fffffff;
        if constexpr (kBf16) {
            QueryRegs q;
            if (top > 0) {
                load_query_regs(arq, q);
                score_blocks_warp(st[0], st[1], stat_stride, nb, n_complete, bs, t, ls, a.strict_valid, a.buckets, q,
                                  sp_a, bias_a, bscore);
            }
            load_query_regs(aq, q);
            score_rows_warp<false>(local_a, key_stride, L, nullptr, bs, bs_shift, first_local, t - L + 1, -1, q, nullptr,
                                   0, bk, bp);
            if (top > 0) {
                __syncwarp();
                if (nb <= 128) pick_blocks_warp(bscore, nb, top, bs, ls, sel);
                else pick_blocks(bscore, nb, top, bs, ls, sel);
                score_remote_warp(seq_a, top * bs, sel, bs, bs_shift, -1, q, stage, nullptr, 0, bk, bp);
            }
        } else {
            if (top > 0)
                score_blocks_any<kBf16>(st[0], st[1], stats_dtype, nb, n_complete, bs, t, ls, a.strict_valid, a.buckets,
                                        arq, sp_a, bias_a, bscore, 0, 1);
            score_rows_split<kBf16, 1>(local_a, key_dtype, L, nullptr, bs, first_local, t - L + 1, -1, nullptr, 0, aq,
                                       nullptr, 0, 0, 1, bk, bp, 0u, ok);
            if (top > 0) {
                __syncwarp();
                pick_blocks(bscore, nb, top, bs, ls, sel);
                uint32_t rk = 0;
                int rp = 0x7fffffff;
                score_rows_split<kBf16, 1, true>(seq_a, key_dtype, top * bs, sel, bs, 0, 0, -1, nullptr, 0, aq, nullptr, 0,
                                                 0, 1, rk, rp, 0u, ok);
                if (rp != 0x7fffffff && (rk > bk || bp == 0x7fffffff || (rk == bk && rp < bp))) { bk = rk; bp = rp; }
            }
        }
        int anchor_pos = bp;
        if (anchor_pos == 0x7fffffff) { anchor_pos = 0; bk = float_key(kNegInf); }
        if (lane == 0) {
            a.out_anchor[row] = anchor_pos;
            a.out_anchor_score[row] = key_float(bk);
        }
        // ---- partner queries: query-side base + the anchor's cached row
        for (int i = lane; i < 2 * kD; i += 32) {
            const float add = load_scalar(a.partner_anchor_cache,
                                          (static_cast<size_t>(b) * a.max_t + anchor_pos) * 2 * kD + i, key_dtype);
            const int at = kBf16 ? (i & ~(kD - 1)) | paired_index(i & (kD - 1)) : i;
            pq[at] = __fadd_rn(pq[at], add);
        }
        __syncwarp();
        // ---- partners
        uint32_t dk = 0;
        int dp = 0x7fffffff;
        if constexpr (kBf16) {
            QueryRegs q;
            if (top > 0) {
                load_query_regs(prq, q);
                score_blocks_warp(st[2], st[3], stat_stride, nb, n_complete, bs, t, ls, a.strict_valid, a.buckets, q,
                                  sp_p, bias_p, bscore);
            }
            load_query_regs(pq, q);
            score_rows_warp<false>(local_p, key_stride, L, nullptr, bs, bs_shift, first_local, t - L + 1, anchor_pos, q,
                                   cand, 0, dk, dp);
            if (top > 0) {
                __syncwarp();
                if (nb <= 128) pick_blocks_warp(bscore, nb, top, bs, ls, sel);
                else pick_blocks(bscore, nb, top, bs, ls, sel);
                score_remote_warp(seq_p, top * bs, sel, bs, bs_shift, anchor_pos, q, stage, cand, L, dk, dp);
            }
        } else {
            if (top > 0)
                score_blocks_any<kBf16>(st[2], st[3], stats_dtype, nb, n_complete, bs, t, ls, a.strict_valid, a.buckets,
                                        prq, sp_p, bias_p, bscore, 0, 1);
            score_rows_split<kBf16, 1>(local_p, key_dtype, L, nullptr, bs, first_local, t - L + 1, anchor_pos, nullptr, 0,
                                       pq, cand, 0, 0, 1, dk, dp, 0u, ok);
            if (top > 0) {
                __syncwarp();
                pick_blocks(bscore, nb, top, bs, ls, sel);
                score_rows_split<kBf16, 1, true>(seq_p, key_dtype, top * bs, sel, bs, 0, 0, anchor_pos, nullptr, 0, pq, cand,
                                                 L, 0, 1, dk, dp, 0u, ok);
            }
        }
        __syncwarp();
        int32_t* out_pos = a.out_partner + static_cast<size_t>(row) * K;
        float* out_sc = a.out_partner_score + static_cast<size_t>(row) * K;
        if (cap4 <= 128) {
            if (!topk_filter<4>(cand, cap4, K, L, t, bs, bs_shift, sel, short_list, out_pos, out_sc))
                topk_tournament<4>(cand, cap4, K, L, t, bs, bs_shift, sel, out_pos, out_sc);
        } else if (cap4 <= 256) {
            if (!topk_filter<8>(cand, cap4, K, L, t, bs, bs_shift, sel, short_list, out_pos, out_sc))
                topk_tournament<8>(cand, cap4, K, L, t, bs, bs_shift, sel, out_pos, out_sc);
        } else {
            if (!topk_filter<16>(cand, cap4, K, L, t, bs, bs_shift, sel, short_list, out_pos, out_sc))
                topk_tournament<16>(cand, cap4, K, L, t, bs, bs_shift, sel, out_pos, out_sc);
        }
        __syncwarp();
    }
}

int tile_warp_bytes(const SelectArgs& a) {
    const int cap4 = (a.local_window + a.top_blocks * a.block_size + 3) & ~3;
    const int floats = 4 * kD + 64 + ((a.n_blocks + 3) & ~3) + cap4;
    return align16(floats * 4 + 3 * (a.top_blocks > 0 ? a.top_blocks : 1) * 4) + 16 + 32 * static_cast<int>(kPadRow);
}

int launch_tile(TileArgs& m, void* stream) {
    SelectArgs& a = m.base;
    if (a.n_seq < 1 || m.q_len < 1 || m.q_len > a.max_t || a.max_t < 1 || a.n_blocks < 1 || a.buckets < 1 ||
        a.local_window < 1 || a.top_blocks < 0 || a.max_t % a.n_blocks != 0 || a.k_out < 1 || a.k_out > kMaxKOut) {
        set_error("relation_select_packed_prefill: sizes must be positive, T a multiple of the block count, K <= 32, "
                  "query length <= T");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(a.query_dtype) || !valid_dtype(a.key_dtype) || !valid_dtype(a.stats_dtype) || !valid_dtype(a.param_dtype)) {
        set_error("relation_select_packed_prefill: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    const void* need[] = {a.anchor_query, a.anchor_keys, a.anchor_router_query, a.anchor_mean, a.anchor_std, a.anchor_gamma,
                          a.anchor_bias, a.partner_base, a.partner_anchor_cache, a.partner_keys, a.partner_mean,
                          a.partner_std, a.partner_gamma, a.partner_bias, a.out_anchor, a.out_anchor_score, a.out_partner,
                          a.out_partner_score};
    for (const void* q : need) if (!q) { set_error("relation_select_packed_prefill: NULL pointer"); return RLM_ERR_NULL; }
    const void* bulk[] = {a.anchor_keys, a.anchor_mean, a.anchor_std, a.partner_keys, a.partner_mean, a.partner_std,
                          a.partner_anchor_cache};
    for (const void* q : bulk)
        if (!aligned16(q)) {
            set_error("relation_select_packed_prefill: key caches, block statistics and the partner-anchor cache must be 16-byte aligned");
            return RLM_ERR_ALIGN;
        }
    a.block_size = a.max_t / a.n_blocks;
    a.mode = kPacked;
    const int cap = a.local_window + a.top_blocks * a.block_size;
    if (cap > 512) {
        set_error("relation_select_packed_prefill: at most 512 candidates per query (window + remote blocks)");
        return RLM_ERR_UNSUPPORTED;
    }
    const bool bf16 = a.query_dtype == RLM_BF16 && a.key_dtype == RLM_BF16 && a.stats_dtype == RLM_BF16;
    const int key_stride = bf16 ? static_cast<int>(kPadRow) : kD * dtype_size(a.key_dtype);
    const int stat_stride = bf16 ? static_cast<int>(kPadRow) : kD * dtype_size(a.stats_dtype);
    m.warp_bytes = tile_warp_bytes(a);
    m.stats_bytes = align16(a.n_blocks * stat_stride);
    m.param_bytes = align16((8 + 8 * a.buckets) * 4);
    int warps = 16, total = 0;
    for (;; warps = 8) {
        m.window_rows = a.local_window + 4 * warps;
        total = 4 * m.stats_bytes + 2 * m.window_rows * key_stride + m.param_bytes + warps * m.warp_bytes;
        if (total <= kSmemDynamicLimit || warps == 8) break;
    }
    if (total > kSmemDynamicLimit) {
        set_error("relation_select_packed_prefill: block statistics + window union exceed 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    auto kernel = bf16 ? (warps == 16 ? relation_select_tile_kernel<true, 16> : relation_select_tile_kernel<true, 8>)
                       : (warps == 16 ? relation_select_tile_kernel<false, 16> : relation_select_tile_kernel<false, 8>);
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    const int tiles = a.n_seq * ((m.q_len + 4 * warps - 1) / (4 * warps));
    launch_kernel(kernel, dim3(tiles), dim3(32 * warps), total, stream, m);
    count_launch();
    return check_launch("relation_select_tile_kernel");
}

// Validation and shared-memory plan of a selector launch: everything but the launch itself.
int prepare(SelectArgs& a, bool& many_rows) {
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
    const Plan& plan = a.plan;
    if (plan.total > kSmemDynamicLimit) {
        set_error("relation_select: block statistics + local window + remote blocks exceed 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    return RLM_OK;
}

int launch(SelectArgs& a, void* stream) {
    if (a.n_rows == 0) return RLM_OK;
    bool many_rows = false;
    const int ready = prepare(a, many_rows);
    if (ready != RLM_OK) return ready;
    const Plan& plan = a.plan;
    const bool bf16 = a.query_dtype == RLM_BF16 && a.key_dtype == RLM_BF16 && a.stats_dtype == RLM_BF16;
    const bool decode = bf16 && a.mode == kPacked && !a.row_batch && !a.row_position && !a.exclude_list;
    auto kernel = many_rows ? (decode ? relation_select_kernel<4, true, true>
                                      : bf16 ? relation_select_kernel<4, true, false> : relation_select_kernel<4, false, false>)
                            : (decode ? relation_select_kernel<3, true, true>
                                      : bf16 ? relation_select_kernel<3, true, false> : relation_select_kernel<3, false, false>);
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    launch_kernel(kernel, dim3(a.n_rows), dim3(kThreads), plan.total, stream, a);
    count_launch();
    return check_launch("relation_select_kernel");
}

// ---- a whole relation layer of a decode step in one launch: the selector in front of the tail
//
// The tail's cluster (relation_layer_tail_body.cuh) has one CTA per 128 hidden columns; the first
// CTAs of the cluster each run the packed selector for one of the cluster's sequences, in the
// shared memory the tail uses from its gathers on (product tile, hidden tile, term rows), while the
// weight slices stream in.  The indices travel through global memory (they are outputs anyway) and
// the cluster barrier.
template <bool kBf16>
struct SelectInFront {
    static constexpr bool kActive = true;
    const SelectArgs* args;
    uint32_t bars;
    __device__ __forceinline__ bool operator()(unsigned char* scratch, uint32_t rank, int s0, int nseq) const {
        if (static_cast<int>(rank) >= nseq) return false;
        // the selector waits for the previous launch itself, as late as its queries allow
        select_row<kBf16, true, false>(*args, s0 + static_cast<int>(rank), scratch, bars);
        return true;
    }
};

template <bool kBf16>
__global__ void __launch_bounds__(kLtThreads, 1) relation_layer_kernel(
    const __grid_constant__ CUtensorMap map_wm, const __grid_constant__ CUtensorMap map_w2,
    const LayerTailArgs tail, const SelectArgs sel) {
    extern __shared__ __align__(1024) unsigned char layer_smem_raw[];
    __shared__ __align__(8) unsigned long long select_bars[4];
    layer_tail_body<kBf16>(map_wm, map_w2, tail, layer_smem_raw, SelectInFront<kBf16>{&sel, smem_u32(select_bars)});
}

int launch_layer(SelectArgs& sel, LayerTailArgs& tail, const void* product_weight, const void* second_weight,
                 void* stream) {
    static_assert(kLtThreads == kThreads, "selector and tail share one CTA shape");
    bool many_rows = false;
    int rc = prepare(sel, many_rows);
    if (rc != RLM_OK) return rc;
    rc = lt_validate(tail);
    if (rc != RLM_OK) return rc;
    if (sel.mode != kPacked || sel.row_batch || sel.row_position || sel.exclude_list || many_rows ||
        sel.n_rows != tail.n_seq || sel.k_out != tail.k_out || sel.max_t != tail.max_t) {
        set_error("relation_layer: the selector must be the decode form over the tail's sequences");
        return RLM_ERR_SHAPE;
    }
    if (sel.query_dtype != tail.dtype || sel.key_dtype != tail.dtype || sel.stats_dtype != tail.dtype) {
        set_error("relation_layer: queries, caches and statistics must share the tail's 16-bit dtype");
        return RLM_ERR_UNSUPPORTED;
    }
    tail.cluster = tail.hdim / kLtHC;
    const int most = kLtMaxPairs / tail.k_out < kLtMaxSeq ? kLtMaxPairs / tail.k_out : kLtMaxSeq;
    tail.seqs_per_cluster = (tail.n_seq + 3) / 4 < most ? (tail.n_seq + 3) / 4 : most;
    if (tail.seqs_per_cluster > tail.cluster) tail.seqs_per_cluster = tail.cluster;   // a selecting CTA per sequence
    const LtPlan whole = lt_plan(tail.rdim, tail.d, kLtMaxPairs);
    if (sel.plan.total > static_cast<int>(whole.total - whole.p)) {
        set_error("relation_layer: the selector's working set does not fit the tail's tile memory (use the two launches)");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(tail.expanded_cache) || !aligned16(tail.operand_cache) || !aligned16(product_weight) ||
        !aligned16(second_weight) || (tail.query_weight && !aligned16(tail.query_weight))) {
        set_error("relation_layer: caches and weights must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    CUtensorMap mwm, mw2;
    if (!make_map(&mwm, product_weight, tail.hdim, tail.rdim, tail.rdim, kBM, tail.dtype) ||
        !make_map(&mw2, second_weight, tail.d, tail.hdim, tail.hdim, kBM, tail.dtype)) {
        set_error("relation_layer: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    auto kernel = tail.dtype == RLM_BF16 ? relation_layer_kernel<true> : relation_layer_kernel<false>;
    rc = lt_prepare(reinterpret_cast<const void*>(kernel), tail.cluster);
    if (rc != RLM_OK) return rc;
    const int clusters = (tail.n_seq + tail.seqs_per_cluster - 1) / tail.seqs_per_cluster;
    const size_t smem_bytes = lt_plan(tail.rdim, tail.d, kLtMaxPairs).total + 1024;
    launch_kernel_cluster(kernel, dim3(tail.cluster, clusters), dim3(kLtThreads), static_cast<unsigned>(tail.cluster),
                          smem_bytes, stream, mwm, mw2, tail, sel);
    count_launch();
    return check_launch("relation_layer_kernel");
}

int launch_multi(MultiSelectArgs& m, void* stream) {
    SelectArgs& a = m.base;
    if (a.n_rows == 0) return RLM_OK;
    if (a.n_rows < 0 || a.n_seq < 1 || a.max_t < 1 || a.n_blocks < 1 || a.buckets < 1 || a.local_window < 1 ||
        a.top_blocks < 0 || a.max_t % a.n_blocks != 0 || m.slots < 1 || m.slots > kMaxSlots || a.k_out < 1 ||
        a.k_out > kMaxKOut) {
        set_error("relation_select_multi_rows: sizes must be positive, T a multiple of the block count, 1..8 slots, K <= 32");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(a.query_dtype) || !valid_dtype(a.key_dtype) || !valid_dtype(a.stats_dtype) || !valid_dtype(a.param_dtype)) {
        set_error("relation_select_multi_rows: unknown dtype code");
        return RLM_ERR_DTYPE;
    }
    const void* need[] = {a.anchor_query, a.anchor_keys, a.anchor_router_query, a.anchor_mean, a.anchor_std, a.anchor_gamma,
                          a.anchor_bias, a.partner_base, a.partner_anchor_cache, a.partner_keys, a.partner_mean,
                          a.partner_std, a.partner_gamma, a.partner_bias, a.row_batch, a.row_position, m.out_anchor,
                          m.out_anchor_score, m.out_anchor_active, m.out_partner, m.out_partner_score};
    for (const void* q : need) if (!q) { set_error("relation_select_multi_rows: NULL pointer"); return RLM_ERR_NULL; }
    const void* bulk[] = {a.anchor_keys, a.anchor_mean, a.anchor_std, a.partner_keys, a.partner_mean, a.partner_std,
                          a.partner_anchor_cache};
    for (const void* q : bulk)
        if (!aligned16(q)) {
            set_error("relation_select_multi_rows: key caches, block statistics and the partner-anchor cache must be 16-byte aligned");
            return RLM_ERR_ALIGN;
        }
    a.block_size = a.max_t / a.n_blocks;
    a.shared_streams = 0;
    a.sm_count = sm_count();
    const int ks = dtype_size(a.key_dtype), ss = dtype_size(a.stats_dtype), ps = dtype_size(a.param_dtype);
    m.plan_anchor = make_plan(a.n_blocks, a.block_size, a.local_window, a.top_blocks, a.buckets, ks, ss, kAnchorOnly, false);
    m.plan_partner = make_plan(a.n_blocks, a.block_size, a.local_window, a.top_blocks, a.buckets, ks, ss, kPartnerOnly, false);
    const int total = m.plan_anchor.total > m.plan_partner.total ? m.plan_anchor.total : m.plan_partner.total;
    if (total > kSmemDynamicLimit) {
        set_error("relation_select_multi_rows: block statistics + local window + remote blocks exceed 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    m.keys_slot = static_cast<size_t>(a.n_seq) * a.max_t * kD * ks;
    m.pac_slot = static_cast<size_t>(a.n_seq) * a.max_t * 2 * kD * ks;
    m.stats_slot = static_cast<size_t>(a.n_seq) * a.n_blocks * kD * ss;
    m.gamma_slot = static_cast<size_t>(4) * ps;
    m.bias_slot = static_cast<size_t>(4) * a.buckets * ps;
    if (a.aq_stride < static_cast<int64_t>(m.slots) * kD || a.arq_stride < static_cast<int64_t>(m.slots) * kD ||
        a.pbase_stride < static_cast<int64_t>(m.slots) * 2 * kD) {
        set_error("relation_select_multi_rows: a query row stride is shorter than the slots it holds");
        return RLM_ERR_SHAPE;
    }
    const bool bf16 = a.query_dtype == RLM_BF16 && a.key_dtype == RLM_BF16 && a.stats_dtype == RLM_BF16;
    auto kernel = bf16 ? relation_select_multi_kernel<true> : relation_select_multi_kernel<false>;
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    launch_kernel(kernel, dim3(a.n_rows), dim3(kThreads), total, stream, m);
    count_launch();
    return check_launch("relation_select_multi_kernel");
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_relation_layer_supported(int n_seq, int k_out, int relation_dim, int hidden_dim, int d_model,
                                           int n_query, int dtype, int max_t, int n_blocks, int buckets,
                                           int local_window, int top_blocks) {
    using namespace rlm;
    LayerTailArgs t{};
    t.n_seq = n_seq; t.k_out = k_out; t.max_t = max_t; t.rdim = relation_dim; t.hdim = hidden_dim; t.d = d_model;
    t.n_query = n_query; t.dtype = dtype;
    t.query_weight = n_query > 0 ? &t : nullptr;      // only tested for NULL
    t.query = n_query > 0 ? &t : nullptr;
    if (lt_validate(t) != RLM_OK) return 0;
    if (n_seq < 1 || max_t < 1 || n_blocks < 1 || buckets < 1 || local_window < 1 || top_blocks < 0 ||
        max_t % n_blocks != 0 || k_out > kMaxKOut)
        return 0;
    const int cluster = hidden_dim / kLtHC;
    const Plan plan = make_plan(n_blocks, max_t / n_blocks, local_window, top_blocks, buckets, dtype_size(dtype),
                                dtype_size(dtype), kPacked, false);
    const LtPlan whole = lt_plan(relation_dim, d_model, kLtMaxPairs);
    if (plan.total > static_cast<int>(whole.total - whole.p)) return 0;
    auto kernel = dtype == RLM_BF16 ? relation_layer_kernel<true> : relation_layer_kernel<false>;
    if (lt_prepare(reinterpret_cast<const void*>(kernel), cluster) != RLM_OK) return 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(cluster, 1, 1);
    config.blockDim = dim3(kLtThreads, 1, 1);
    config.dynamicSmemBytes = lt_plan(relation_dim, d_model, kLtMaxPairs).total + 1024;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return clusters > 0 ? 1 : 0;
}

extern "C" int rlm_relation_layer(
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
    int hidden_dim, int d_model, int n_query, int dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (n_seq == 0) return RLM_OK;
    if (!expanded_cache || !operand_cache || !product_weight || !second_weight || !second_bias || !norm_weight ||
        !norm_bias || !position || !residual || !mix || !next_norm_weight || !next_norm_bias || !normalized) {
        set_error("relation_layer: NULL pointer");
        return RLM_ERR_NULL;
    }
    SelectArgs a{};
    a.aq_stride = anchor_query_stride; a.arq_stride = anchor_router_query_stride; a.pbase_stride = partner_base_stride;
    a.anchor_query = anchor_query; a.anchor_keys = anchor_keys; a.anchor_router_query = anchor_router_query;
    a.anchor_mean = anchor_mean; a.anchor_std = anchor_std; a.anchor_gamma = anchor_gamma; a.anchor_bias = anchor_bias;
    a.partner_base = partner_base; a.partner_anchor_cache = partner_anchor_cache; a.partner_keys = partner_keys;
    a.partner_mean = partner_mean; a.partner_std = partner_std; a.partner_gamma = partner_gamma; a.partner_bias = partner_bias;
    a.position = position; a.out_anchor = out_anchor; a.out_anchor_score = out_anchor_score;
    a.out_partner = out_partner; a.out_partner_score = out_partner_score; a.status = status;
    a.n_rows = n_seq; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks; a.buckets = buckets;
    a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = k_out; a.strict_valid = strict_valid != 0;
    a.query_dtype = dtype; a.key_dtype = dtype; a.stats_dtype = dtype; a.param_dtype = param_dtype;
    a.mode = kPacked;
    LayerTailArgs t{};
    t.expanded_cache = expanded_cache; t.operand_cache = operand_cache; t.anchor_index = out_anchor;
    t.partner_index = out_partner; t.partner_scores = out_partner_score; t.second_bias = second_bias;
    t.norm_w = norm_weight; t.norm_b = norm_bias; t.position = position; t.residual = residual; t.mix = mix;
    t.next_w = next_norm_weight; t.next_b = next_norm_bias; t.normalized = normalized;
    t.query_weight = query_weight; t.query = query; t.status = status; t.eps = norm_eps; t.next_eps = next_norm_eps;
    t.n_seq = n_seq; t.k_out = k_out; t.max_t = max_t; t.rdim = relation_dim; t.hdim = hidden_dim; t.d = d_model;
    t.n_query = query_weight ? n_query : 0; t.dtype = dtype;
    return launch_layer(a, t, product_weight, second_weight, stream);
}

extern "C" int rlm_relation_select_packed_prefill(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    int32_t* out_anchor, float* out_anchor_score, int32_t* out_partner, float* out_partner_score,
    int64_t anchor_query_stride, int64_t anchor_router_query_stride, int64_t partner_base_stride,
    int n_seq, int query_length, int max_t, int n_blocks, int buckets, int local_window, int top_blocks, int k_out,
    int strict_valid, int query_dtype, int key_dtype, int stats_dtype, int param_dtype, int32_t* status,
    void* stream) {
    rlm::TileArgs m{};
    rlm::SelectArgs& a = m.base;
    a.aq_stride = anchor_query_stride; a.arq_stride = anchor_router_query_stride; a.pbase_stride = partner_base_stride;
    a.anchor_query = anchor_query; a.anchor_keys = anchor_keys; a.anchor_router_query = anchor_router_query;
    a.anchor_mean = anchor_mean; a.anchor_std = anchor_std; a.anchor_gamma = anchor_gamma; a.anchor_bias = anchor_bias;
    a.partner_base = partner_base; a.partner_anchor_cache = partner_anchor_cache; a.partner_keys = partner_keys;
    a.partner_mean = partner_mean; a.partner_std = partner_std; a.partner_gamma = partner_gamma; a.partner_bias = partner_bias;
    a.out_anchor = out_anchor; a.out_anchor_score = out_anchor_score; a.out_partner = out_partner;
    a.out_partner_score = out_partner_score; a.status = status;
    a.n_rows = n_seq * query_length; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks; a.buckets = buckets;
    a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = k_out; a.strict_valid = strict_valid != 0;
    a.query_dtype = query_dtype; a.key_dtype = key_dtype; a.stats_dtype = stats_dtype; a.param_dtype = param_dtype;
    m.q_len = query_length;
    return rlm::launch_tile(m, stream);
}

extern "C" int rlm_relation_select_multi_rows(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    const int32_t* row_batch, const int32_t* row_position, int32_t* out_anchor, float* out_anchor_score,
    uint8_t* out_anchor_active, int32_t* out_partner, float* out_partner_score,
    int64_t anchor_query_stride, int64_t anchor_router_query_stride, int64_t partner_base_stride,
    int n_rows, int n_seq, int slots,
    int max_t, int n_blocks, int buckets, int local_window, int top_blocks, int k_out, int strict_valid,
    int query_dtype, int key_dtype, int stats_dtype, int param_dtype, int32_t* status, void* stream) {
    rlm::MultiSelectArgs m{};
    rlm::SelectArgs& a = m.base;
    a.anchor_query = anchor_query; a.anchor_keys = anchor_keys; a.anchor_router_query = anchor_router_query;
    a.anchor_mean = anchor_mean; a.anchor_std = anchor_std; a.anchor_gamma = anchor_gamma; a.anchor_bias = anchor_bias;
    a.partner_base = partner_base; a.partner_anchor_cache = partner_anchor_cache; a.partner_keys = partner_keys;
    a.partner_mean = partner_mean; a.partner_std = partner_std; a.partner_gamma = partner_gamma; a.partner_bias = partner_bias;
    a.row_batch = row_batch; a.row_position = row_position; a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks; a.buckets = buckets;
    a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = k_out; a.strict_valid = strict_valid != 0;
    a.query_dtype = query_dtype; a.key_dtype = key_dtype; a.stats_dtype = stats_dtype; a.param_dtype = param_dtype;
    a.aq_stride = anchor_query_stride; a.arq_stride = anchor_router_query_stride; a.pbase_stride = partner_base_stride;
    m.slots = slots; m.out_anchor = out_anchor; m.out_anchor_score = out_anchor_score;
    m.out_anchor_active = out_anchor_active; m.out_partner = out_partner; m.out_partner_score = out_partner_score;
    return rlm::launch_multi(m, stream);
}

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
    const int32_t* exclude_index, int exclude_count,
    int32_t* out_index, float* out_score, int n_rows, int n_seq, int max_t, int n_blocks,
    int buckets, int local_window, int top_blocks, int strict_valid, int query_dtype,
    int key_dtype, int stats_dtype, int param_dtype, int32_t* status, void* stream) {
    rlm::SelectArgs a{};
    a.exclude_list = exclude_index; a.exclude_count = exclude_count;
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
    const int32_t* anchor_index, const int32_t* exclude_index, int exclude_count,
    int32_t* out_index, float* out_score, int n_rows, int n_seq,
    int max_t, int n_blocks, int buckets, int local_window, int top_blocks, int k_out,
    int strict_valid, int query_dtype, int key_dtype, int stats_dtype, int param_dtype,
    int32_t* status, void* stream) {
    rlm::SelectArgs a{};
    a.exclude_list = exclude_index; a.exclude_count = exclude_count;
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

