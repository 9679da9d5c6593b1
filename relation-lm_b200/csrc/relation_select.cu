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

#include "relation_select_body.cuh"

namespace rlm {
namespace {

// kMinCtas = 3: the latency-oriented build (decode batches: one wave or less).  kMinCtas = 4:
// launches of many rows, where rows in flight per SM set the throughput.  kBf16: queries, key
// caches and block statistics are all bf16 (the decode configuration); the dtype branches
// fold away, which matters because a row's time is largely instruction fetch.
template <int kMinCtas, bool kBf16, bool kDecode, bool kResident = false>
__global__ void __launch_bounds__(kThreads, kMinCtas) relation_select_kernel(const SelectArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    select_row<kBf16, kDecode, false, kResident>(a, blockIdx.x, smem, smem_u32(smem + a.plan.bars));
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
// Further excluded positions of a query (the anchors of a multi-anchor row's slots; -1 = none).
struct ExclRegs { int v[kMaxExclude]; int n; };

template <bool kExcl>
__device__ __forceinline__ bool not_excluded(int pos, const ExclRegs* ex) {
    bool keep = true;
    if (kExcl) {
#pragma unroll
        for (int x = 0; x < kMaxExclude; ++x) keep = keep && (x >= ex->n || pos != ex->v[x]);
    }
    return keep;
}

template <bool kAtPosition, bool kExcl = false>
__device__ __forceinline__ void score_rows_warp(const unsigned char* rows, uint32_t stride, int n_rows, const int* sel,
                                                int bs, int bs_shift, int first_valid, int pos0, int exclude,
                                                const QueryRegs& q, float* cand, int slot0, uint32_t& best_key,
                                                int& best_pos, const ExclRegs* ex = nullptr) {
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
        valid = valid && pos != exclude && not_excluded<kExcl>(pos, ex);
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
template <bool kExcl = false>
__device__ __forceinline__ void score_remote_warp(const unsigned char* keys, int n_rows, const int* sel, int bs,
                                                  int bs_shift, int exclude, const QueryRegs& q, unsigned char* stage,
                                                  float* cand, int slot0, uint32_t& best_key, int& best_pos,
                                                  const ExclRegs* ex = nullptr) {
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
        const bool valid = pos >= 0 && pos != exclude && not_excluded<kExcl>(pos, ex);
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

// ---- whole-sequence multi-anchor selection: the tiled form of relation_select_multi_kernel (bf16)
//
// A CTA of kTileWarps warps serves 4 kTileWarps consecutive positions of one sequence; every warp
// keeps its queries and walks them through 2 S phases — the anchors of slot 0 .. S - 1 (each barring
// the positions taken before it), then the partners of slot 0 .. S - 1 (each barring all anchors).
// A phase's block statistics and window union (one slot, one stream) are staged for the whole CTA
// in one of two buffers while the previous phase is being computed.  Rules and arithmetic are
// relation_select_multi_kernel's (same results bit for bit).
struct MultiTileArgs {
    MultiSelectArgs m;
    int q_len;
    int warp_bytes, stats_bytes, window_rows, param_bytes, stage_bytes;
};

template <int kTileWarps>
__global__ void __launch_bounds__(32 * kTileWarps, 16 / kTileWarps) relation_select_multi_tile_kernel(const MultiTileArgs ta) {
    constexpr int kTileQ = 4 * kTileWarps, kTileThreads = 32 * kTileWarps;
    extern __shared__ __align__(128) unsigned char smem[];
    const MultiSelectArgs& m = ta.m;
    const SelectArgs& a = m.base;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int S = m.slots, K = a.k_out;
    const int tiles_per_seq = (ta.q_len + kTileQ - 1) / kTileQ;
    const int b = blockIdx.x / tiles_per_seq, t0 = (blockIdx.x - b * tiles_per_seq) * kTileQ;
    const int t_end = min(t0 + kTileQ, ta.q_len);
    const int nb = a.n_blocks, bs = a.block_size, L = a.local_window, top = a.top_blocks;
    const int bs_shift = (bs & (bs - 1)) == 0 ? 31 - __clz(bs) : -1;
    constexpr size_t key_row = 2 * kD, stat_row = 2 * kD;
    const int buckets4 = 4 * a.buckets;
    griddep_sync();

    // two staging buffers: mean | std | window union of one slot and stream
    unsigned char* stage_buf[2] = {smem, smem + ta.stage_bytes};
    float* params = reinterpret_cast<float*>(smem + 2 * ta.stage_bytes);      // per slot: softplus a[4] p[4], bias a, bias p
    const int slot_params = 8 + 2 * buckets4;
    unsigned char* warp_base = reinterpret_cast<unsigned char*>(params) + ta.param_bytes + static_cast<size_t>(warp) * ta.warp_bytes;
    const int n_stage = top > 0 ? min(t_end / bs, nb) : 0;
    const int w_lo = max(t0 - L + 1, 0);
    auto request_phase = [&](int ph) {
        if (ph < 2 * S) {
            const int s = ph < S ? ph : ph - S;
            const bool partner = ph >= S;
            unsigned char* dst = stage_buf[ph & 1];
            const size_t seq_stats = s * m.stats_slot + static_cast<size_t>(b) * nb * stat_row;
            const size_t seq_keys = s * m.keys_slot + static_cast<size_t>(b) * a.max_t * key_row;
            const char* mean = static_cast<const char*>(partner ? a.partner_mean : a.anchor_mean) + seq_stats;
            const char* stdv = static_cast<const char*>(partner ? a.partner_std : a.anchor_std) + seq_stats;
            const char* keys = static_cast<const char*>(partner ? a.partner_keys : a.anchor_keys) + seq_keys + w_lo * key_row;
            const int stat_chunks = n_stage * 8;
            for (int i = tid; i < 2 * stat_chunks; i += kTileThreads) {
                const int which = i >= stat_chunks, c = i - which * stat_chunks;
                cp_async16(smem_u32(dst) + which * ta.stats_bytes + (c >> 3) * kPadRow + 16 * (c & 7),
                           (which ? stdv : mean) + 16 * c);
            }
            const int win_chunks = (t_end - w_lo) * 8;
            for (int i = tid; i < win_chunks; i += kTileThreads)
                cp_async16(smem_u32(dst) + 2 * ta.stats_bytes + (i >> 3) * kPadRow + 16 * (i & 7), keys + 16 * i);
        }
        cp_async_commit();
    };
    request_phase(0);
    for (int i = tid; i < S * slot_params; i += kTileThreads) {
        const int s = i / slot_params, j = i - s * slot_params;
        float v;
        if (j < 8) {
            const float gamma = load_scalar(slot_ptr(j < 4 ? a.anchor_gamma : a.partner_gamma, s * m.gamma_slot), j & 3, a.param_dtype);
            v = canon_log(__fadd_rn(1.0f, canon_exp(gamma)));
        } else if (j < 8 + buckets4) {
            v = load_scalar(slot_ptr(a.anchor_bias, s * m.bias_slot), j - 8, a.param_dtype);
        } else {
            v = load_scalar(slot_ptr(a.partner_bias, s * m.bias_slot), j - 8 - buckets4, a.param_dtype);
        }
        params[i] = v;
    }
    // per-warp scratch
    float* queries = reinterpret_cast<float*>(warp_base);                     // exact query | router query (paired layout)
    uint32_t* short_list = reinterpret_cast<uint32_t*>(queries + 2 * kD);     // 64 words of the top-K filter
    int* taken = reinterpret_cast<int*>(short_list + 64);                     // [4 queries][kMaxSlots]
    float* bscore = reinterpret_cast<float*>(taken + 4 * kMaxSlots);
    float* cand = bscore + ((nb + 3) & ~3);
    const int cap = L + top * bs, cap4 = (cap + 3) & ~3;
    int* sel = reinterpret_cast<int*>(cand + cap4);
    unsigned char* park = warp_base + ta.warp_bytes - 32 * kPadRow;           // remote rows of a pass
    for (int i = cap + lane; i < cap4; i += 32) cand[i] = kNegInf;
    for (int i = lane; i < 4 * kMaxSlots; i += 32) taken[i] = -1;
    const size_t esz = 2;

    for (int ph = 0; ph < 2 * S; ++ph) {
        request_phase(ph + 1);                       // into the buffer phase ph - 1 has left
        cp_async_wait_group1();
        __syncthreads();                             // phase ph is staged (and, first time, the parameters are written)
        const int s = ph < S ? ph : ph - S;
        const bool partner = ph >= S;
        const unsigned char* st_mean = stage_buf[ph & 1];
        const unsigned char* st_std = st_mean + ta.stats_bytes;
        const unsigned char* win = st_mean + 2 * ta.stats_bytes;
        const float* sp = params + s * slot_params + (partner ? 4 : 0);
        const float* bias = params + s * slot_params + 8 + (partner ? buckets4 : 0);
        const unsigned char* seq_keys = static_cast<const unsigned char*>(partner ? a.partner_keys : a.anchor_keys) +
                                        s * m.keys_slot + static_cast<size_t>(b) * a.max_t * key_row;
        int qi = 0;
        for (int t = t0 + warp; t < t_end; t += kTileWarps, ++qi) {
            const int row = b * ta.q_len + t;
            const int ls = max(t - L + 1, 0), first_local = ls - (t - L + 1);
            const int n_complete = min((t + 1) / bs, nb);
            int* mine = taken + qi * kMaxSlots;
            const unsigned char* local = win + static_cast<ptrdiff_t>(t - L + 1 - w_lo) * static_cast<ptrdiff_t>(kPadRow);
            ExclRegs ex;
            if (!partner) {
                // ---- anchor of slot s: active iff s <= t; the positions taken by slots 0 .. s - 1 are barred
                int32_t* out_idx = m.out_anchor + static_cast<size_t>(row) * S + s;
                float* out_sc = m.out_anchor_score + static_cast<size_t>(row) * S + s;
                uint8_t* out_live = m.out_anchor_active + static_cast<size_t>(row) * S + s;
                if (s > t) {
                    if (lane == 0) { *out_idx = 0; *out_sc = kNegInf; *out_live = 0; }
                    continue;                        // taken[s] stays -1
                }
                for (int i = lane; i < 2 * kD; i += 32) {
                    const float v = i < kD ? load_scalar(a.anchor_query, row * a.aq_stride + s * kD + i, RLM_BF16)
                                           : load_scalar(a.anchor_router_query, row * a.arq_stride + s * kD + i - kD, RLM_BF16);
                    queries[(i & ~(kD - 1)) | paired_index(i & (kD - 1))] = v;
                }
                ex.n = s;
#pragma unroll
                for (int x = 0; x < kMaxExclude; ++x) ex.v[x] = x < s ? mine[x] : -1;
                __syncwarp();
                QueryRegs q;
                if (top > 0) {
                    load_query_regs(queries + kD, q);
                    score_blocks_warp(st_mean, st_std, kPadRow, nb, n_complete, bs, t, ls, a.strict_valid, a.buckets, q, sp,
                                      bias, bscore);
                }
                load_query_regs(queries, q);
                uint32_t bk = 0;
                int bp = 0x7fffffff;
                score_rows_warp<false, true>(local, kPadRow, L, nullptr, bs, bs_shift, first_local, t - L + 1, -1, q, nullptr,
                                             0, bk, bp, &ex);
                if (top > 0) {
                    __syncwarp();
                    if (nb <= 128) pick_blocks_warp(bscore, nb, top, bs, ls, sel);
                    else pick_blocks(bscore, nb, top, bs, ls, sel);
                    score_remote_warp<true>(seq_keys, top * bs, sel, bs, bs_shift, -1, q, park, nullptr, 0, bk, bp, &ex);
                }
                const float score = bp == 0x7fffffff ? kNegInf : key_float(bk);
                const bool live = score > kNegInf;
                if (lane == 0) {
                    *out_idx = live ? bp : 0;
                    *out_sc = live ? score : kNegInf;
                    *out_live = live ? 1 : 0;
                    mine[s] = live ? bp : -1;
                }
                __syncwarp();
            } else {
                // ---- partners of slot s: none without an anchor; the anchors of all slots are barred
                int32_t* out_idx = m.out_partner + (static_cast<size_t>(row) * S + s) * K;
                float* out_sc = m.out_partner_score + (static_cast<size_t>(row) * S + s) * K;
                const int anchor_pos = mine[s];
                if (anchor_pos < 0) {
                    if (lane < K) { out_idx[lane] = 0; out_sc[lane] = kNegInf; }
                    continue;
                }
                const unsigned char* pac = static_cast<const unsigned char*>(a.partner_anchor_cache) + s * m.pac_slot;
                for (int i = lane; i < 2 * kD; i += 32) {
                    const float base = load_scalar(a.partner_base, row * a.pbase_stride + s * 2 * kD + i, RLM_BF16);
                    const float add = load_scalar(pac, (static_cast<size_t>(b) * a.max_t + anchor_pos) * 2 * kD + i, RLM_BF16);
                    queries[(i & ~(kD - 1)) | paired_index(i & (kD - 1))] = __fadd_rn(base, add);
                }
                ex.n = S;
#pragma unroll
                for (int x = 0; x < kMaxExclude; ++x) ex.v[x] = x < S ? mine[x] : -1;
                __syncwarp();
                QueryRegs q;
                if (top > 0) {
                    load_query_regs(queries + kD, q);
                    score_blocks_warp(st_mean, st_std, kPadRow, nb, n_complete, bs, t, ls, a.strict_valid, a.buckets, q, sp,
                                      bias, bscore);
                }
                load_query_regs(queries, q);
                uint32_t dk = 0;
                int dp = 0x7fffffff;
                score_rows_warp<false, true>(local, kPadRow, L, nullptr, bs, bs_shift, first_local, t - L + 1, anchor_pos, q,
                                             cand, 0, dk, dp, &ex);
                if (top > 0) {
                    __syncwarp();
                    if (nb <= 128) pick_blocks_warp(bscore, nb, top, bs, ls, sel);
                    else pick_blocks(bscore, nb, top, bs, ls, sel);
                    score_remote_warp<true>(seq_keys, top * bs, sel, bs, bs_shift, anchor_pos, q, park, cand, L, dk, dp, &ex);
                }
                __syncwarp();
                bool exact = false;
                if (cap4 <= 128) exact = topk_filter<4>(cand, cap4, K, L, t, bs, bs_shift, sel, short_list, out_idx, out_sc);
                else if (cap4 <= 256) exact = topk_filter<8>(cand, cap4, K, L, t, bs, bs_shift, sel, short_list, out_idx, out_sc);
                else exact = topk_filter<16>(cand, cap4, K, L, t, bs, bs_shift, sel, short_list, out_idx, out_sc);
                if (!exact) {
                    if (cap4 <= 128) topk_tournament<4>(cand, cap4, K, L, t, bs, bs_shift, sel, out_idx, out_sc);
                    else if (cap4 <= 256) topk_tournament<8>(cand, cap4, K, L, t, bs, bs_shift, sel, out_idx, out_sc);
                    else topk_tournament<16>(cand, cap4, K, L, t, bs, bs_shift, sel, out_idx, out_sc);
                    // slots without a finite score report index 0 (written by this very lane just above)
                    if (lane < K && !(out_sc[lane] > kNegInf)) { out_idx[lane] = 0; out_sc[lane] = kNegInf; }
                }
                __syncwarp();
            }
        }
        __syncthreads();                             // everybody has left buffer ph & 1
    }
    cp_async_wait_all();
    (void)esz;
}

int launch_multi_tile(MultiTileArgs& ta, void* stream) {
    MultiSelectArgs& m = ta.m;
    SelectArgs& a = m.base;
    if (a.n_seq < 1 || ta.q_len < 1 || ta.q_len > a.max_t || a.max_t < 1 || a.n_blocks < 1 || a.buckets < 1 ||
        a.local_window < 1 || a.top_blocks < 0 || a.max_t % a.n_blocks != 0 || m.slots < 1 || m.slots > kMaxSlots ||
        a.k_out < 1 || a.k_out > kMaxKOut) {
        set_error("relation_select_multi_prefill: sizes must be positive, T a multiple of the block count, 1..8 slots, "
                  "K <= 32, query length <= T");
        return RLM_ERR_SHAPE;
    }
    if (a.query_dtype != RLM_BF16 || a.key_dtype != RLM_BF16 || a.stats_dtype != RLM_BF16 || !valid_dtype(a.param_dtype)) {
        set_error("relation_select_multi_prefill: queries, caches and block statistics must be bfloat16 "
                  "(relation_select_multi_rows serves the other dtypes)");
        return RLM_ERR_UNSUPPORTED;
    }
    const void* need[] = {a.anchor_query, a.anchor_keys, a.anchor_router_query, a.anchor_mean, a.anchor_std, a.anchor_gamma,
                          a.anchor_bias, a.partner_base, a.partner_anchor_cache, a.partner_keys, a.partner_mean,
                          a.partner_std, a.partner_gamma, a.partner_bias, m.out_anchor, m.out_anchor_score,
                          m.out_anchor_active, m.out_partner, m.out_partner_score};
    for (const void* q : need) if (!q) { set_error("relation_select_multi_prefill: NULL pointer"); return RLM_ERR_NULL; }
    const void* bulk[] = {a.anchor_keys, a.anchor_mean, a.anchor_std, a.partner_keys, a.partner_mean, a.partner_std,
                          a.partner_anchor_cache};
    for (const void* q : bulk)
        if (!aligned16(q)) {
            set_error("relation_select_multi_prefill: key caches, block statistics and the partner-anchor cache must be 16-byte aligned");
            return RLM_ERR_ALIGN;
        }
    a.block_size = a.max_t / a.n_blocks;
    const int cap = a.local_window + a.top_blocks * a.block_size;
    if (cap > 512) {
        set_error("relation_select_multi_prefill: at most 512 candidates per query (window + remote blocks)");
        return RLM_ERR_UNSUPPORTED;
    }
    const int ps = dtype_size(a.param_dtype);
    m.keys_slot = static_cast<size_t>(a.n_seq) * a.max_t * kD * 2;
    m.pac_slot = static_cast<size_t>(a.n_seq) * a.max_t * 2 * kD * 2;
    m.stats_slot = static_cast<size_t>(a.n_seq) * a.n_blocks * kD * 2;
    m.gamma_slot = static_cast<size_t>(4) * ps;
    m.bias_slot = static_cast<size_t>(4) * a.buckets * ps;
    if (a.aq_stride < static_cast<int64_t>(m.slots) * kD || a.arq_stride < static_cast<int64_t>(m.slots) * kD ||
        a.pbase_stride < static_cast<int64_t>(m.slots) * 2 * kD) {
        set_error("relation_select_multi_prefill: a query row stride is shorter than the slots it holds");
        return RLM_ERR_SHAPE;
    }
    const int cap4 = (cap + 3) & ~3;
    const int floats = 2 * kD + 64 + 4 * kMaxSlots + ((a.n_blocks + 3) & ~3) + cap4;
    ta.warp_bytes = align16(floats * 4 + 3 * (a.top_blocks > 0 ? a.top_blocks : 1) * 4) + 16 + 32 * static_cast<int>(kPadRow);
    ta.stats_bytes = align16(a.n_blocks * static_cast<int>(kPadRow));
    ta.param_bytes = align16(m.slots * (8 + 8 * a.buckets) * 4);
    int warps = 16, total = 0;
    for (;; warps = 8) {
        ta.window_rows = a.local_window + 4 * warps;
        ta.stage_bytes = (2 * ta.stats_bytes + ta.window_rows * static_cast<int>(kPadRow) + 127) & ~127;
        total = 2 * ta.stage_bytes + ta.param_bytes + warps * ta.warp_bytes;
        if (total <= kSmemDynamicLimit || warps == 8) break;
    }
    if (total > kSmemDynamicLimit) {
        set_error("relation_select_multi_prefill: block statistics + window union exceed 227 KB of shared memory");
        return RLM_ERR_SMEM;
    }
    auto kernel = warps == 16 ? relation_select_multi_tile_kernel<16> : relation_select_multi_tile_kernel<8>;
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    const int tiles = a.n_seq * ((ta.q_len + 4 * warps - 1) / (4 * warps));
    launch_kernel(kernel, dim3(tiles), dim3(32 * warps), total, stream, ta);
    count_launch();
    return check_launch("relation_select_multi_tile_kernel");
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

int launch(SelectArgs& a, void* stream) {
    if (a.n_rows == 0) return RLM_OK;
    bool many_rows = false;
    const int ready = prepare(a, many_rows, true);
    if (ready != RLM_OK) return ready;
    const Plan& plan = a.plan;
    const bool bf16 = a.query_dtype == RLM_BF16 && a.key_dtype == RLM_BF16 && a.stats_dtype == RLM_BF16;
    const bool decode = bf16 && a.mode == kPacked && !a.row_batch && !a.row_position && !a.exclude_list;
    auto kernel = a.resident ? relation_select_kernel<1, true, true, true> : many_rows ? (decode ? relation_select_kernel<4, true, true>
                                      : bf16 ? relation_select_kernel<4, true, false> : relation_select_kernel<4, false, false>)
                            : (decode ? relation_select_kernel<3, true, true>
                                      : bf16 ? relation_select_kernel<3, true, false> : relation_select_kernel<3, false, false>);
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    launch_kernel(kernel, dim3(a.n_rows), dim3(kThreads), plan.total, stream, a);
    count_launch();
    return check_launch("relation_select_kernel");
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

extern "C" int rlm_relation_select_multi_prefill(
    const void* anchor_query, const void* anchor_keys, const void* anchor_router_query,
    const void* anchor_mean, const void* anchor_std, const void* anchor_gamma, const void* anchor_bias,
    const void* partner_base, const void* partner_anchor_cache, const void* partner_keys,
    const void* partner_mean, const void* partner_std, const void* partner_gamma, const void* partner_bias,
    int32_t* out_anchor, float* out_anchor_score, uint8_t* out_anchor_active, int32_t* out_partner,
    float* out_partner_score, int64_t anchor_query_stride, int64_t anchor_router_query_stride,
    int64_t partner_base_stride, int query_length, int n_seq, int slots, int max_t, int n_blocks, int buckets,
    int local_window, int top_blocks, int k_out, int strict_valid, int query_dtype, int key_dtype, int stats_dtype,
    int param_dtype, int32_t* status, void* stream) {
    if (n_seq == 0 || query_length == 0) return RLM_OK;
    rlm::MultiTileArgs ta{};
    rlm::MultiSelectArgs& m = ta.m;
    rlm::SelectArgs& a = m.base;
    a.anchor_query = anchor_query; a.anchor_keys = anchor_keys; a.anchor_router_query = anchor_router_query;
    a.anchor_mean = anchor_mean; a.anchor_std = anchor_std; a.anchor_gamma = anchor_gamma; a.anchor_bias = anchor_bias;
    a.partner_base = partner_base; a.partner_anchor_cache = partner_anchor_cache; a.partner_keys = partner_keys;
    a.partner_mean = partner_mean; a.partner_std = partner_std; a.partner_gamma = partner_gamma; a.partner_bias = partner_bias;
    a.status = status; a.n_rows = n_seq * query_length; a.n_seq = n_seq; a.max_t = max_t; a.n_blocks = n_blocks;
    a.buckets = buckets; a.local_window = local_window; a.top_blocks = top_blocks; a.k_out = k_out;
    a.strict_valid = strict_valid != 0;
    a.query_dtype = query_dtype; a.key_dtype = key_dtype; a.stats_dtype = stats_dtype; a.param_dtype = param_dtype;
    a.aq_stride = anchor_query_stride; a.arq_stride = anchor_router_query_stride; a.pbase_stride = partner_base_stride;
    m.slots = slots; m.out_anchor = out_anchor; m.out_anchor_score = out_anchor_score;
    m.out_anchor_active = out_anchor_active; m.out_partner = out_partner; m.out_partner_score = out_partner_score;
    ta.q_len = query_length;
    return rlm::launch_multi_tile(ta, stream);
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

