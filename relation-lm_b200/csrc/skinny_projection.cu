// Projection of a handful of rows (decode batches: at most 16) without tensor memory (sm_100a):
//   out[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n])
// for 16-bit x [M, d], w [N, d] with fp32 accumulation.  With so few rows the product is a stream
// of the weight matrix, so the kernel is built around that stream: no tensor-memory allocation,
// no tensor map, no shared-memory ring.  A warp owns eight output columns; lane (n = lane / 4,
// part = lane % 4) reads 16 bytes of weight row n per step of 32 k-values — 64 contiguous bytes
// per row and instruction, all of a warp's loads requested up front, before the dependency wait
// (weights depend on no earlier kernel).  The arithmetic is the warp-level tensor instruction
// mma.sync.m16n8k16 (rows of x, padded to 16, as the A operand from shared memory): because a dot
// product does not care in which order k is visited, a lane's eight consecutive k-values feed two
// instructions directly, with the rows of x read at the matching k — no transposition, no
// shuffle reduction, and each lane ends with finished outputs.
//
// Optional greedy head (the `logits.argmax(-1)` and `position += 1` that close a decode step;
// src/relation_lm/models/relation_lm.py:204-207 of the reference project gives the heads): every
// CTA folds its columns below `vocab` into one 64-bit key per row (rounded logit, lowest index on
// ties), one atomicMax per row and CTA; the CTA that finishes last turns the keys into token ids,
// clears keys and counter for the next launch and advances the position.  A maximum does not
// depend on the order of the atomics: the result is deterministic.
//
// Stands where the reference calls F.linear on one position's rows
// (src/relation_lm/inference/packed_cache.py:52-57; the heads of relation_lm.py:121-124).

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kSkThreads = 256;
constexpr int kSkWarps = kSkThreads / 32;
constexpr int kSkMaxRows = 16;

struct SkinnyArgs {
    const void* x;            // [M, d] 16-bit, row stride in elements
    const void* w;            // [N, d] 16-bit
    const float* bias;        // [N] or NULL
    void* out;                // [M, N] 16-bit
    unsigned long long* keys; // [16] arg-max keys (zero between launches), or NULL
    unsigned int* counter;    // CTAs done (zero between launches)
    int64_t* next_token;      // [M]
    int64_t* position;        // optional: += 1
    int64_t x_stride;
    int rows, d, n, vocab, dtype;
    int groups;               // groups of eight output columns
};

// State append in the projection's epilogue (the packed projection of a decode step): every output
// element is stored where the step's state keeps it instead of (or besides) a packed row.  Column
// c of layer l's 384 + R packed columns (src/relation_lm/inference/packed_cache.py:10-17):
// anchor key | partner key | operand | partner-anchor -> row `position` of the four token caches;
// anchor / partner router key, channel ch -> the router update of that channel
// (src/relation_lm/kernels/router_cache.py:33-172): raw key, three-tap causal convolution over the
// raw cache, conv cache row, and mean / biased std of the channel over the current block's conv
// rows in ascending order with the fresh (un-rounded) value at the current row.  Every step of
// that update is per channel, so the lane that holds the channel's output does all of it.
struct SkinnyAppend {
    void* token_cache[4];     // [layers, B, T, w]: anchor keys, partner keys, operand, partner-anchor
    void* raw_cache[2];       // [layers, B, T, 64]
    void* conv_cache[2];
    void* mean[2];            // [layers, B, NB, 64]
    void* stdv[2];
    const float* weight[2];   // [layers, 64, 3] fp32
    const int64_t* position;
    int32_t* status;
    int max_t, n_blocks, block_size, layers, rdim;
};

template <bool kBf16>
__device__ __forceinline__ float from16(uint16_t bits) {
    return kBf16 ? bf16_bits_to_float(bits) : __half2float(*reinterpret_cast<const __half*>(&bits));
}
template <bool kBf16>
__device__ __forceinline__ uint16_t to16(float v) {
    if (kBf16) { __nv_bfloat16 h = __float2bfloat16_rn(v); return *reinterpret_cast<uint16_t*>(&h); }
    __half h = __float2half_rn(v);
    return *reinterpret_cast<uint16_t*>(&h);
}

// One packed output of sequence m, column col (already rounded: `bits`, `value`), at position t.
template <bool kBf16>
__device__ __forceinline__ void append_output(const SkinnyAppend& ap, int batch, int m, int col, int t,
                                              uint16_t bits, float value) {
    const int width = 384 + ap.rdim;
    const int l = col / width, c = col - l * width;
    const int64_t seq = static_cast<int64_t>(l) * batch + m;
    const int R = ap.rdim;
    if (c < 256 + R) {
        int which, w, cc;
        if (c < 64) { which = 0; w = 64; cc = c; }
        else if (c < 128) { which = 1; w = 64; cc = c - 64; }
        else if (c < 128 + R) { which = 2; w = R; cc = c - 128; }
        else { which = 3; w = 128; cc = c - 128 - R; }
        static_cast<uint16_t*>(ap.token_cache[which])[(seq * ap.max_t + t) * w + cc] = bits;
        return;
    }
    const int s = (c - 256 - R) >> 6, ch = (c - 256 - R) & 63;
    const int bs = ap.block_size, blk = t / bs, start = blk * bs;
    uint16_t* raw_cache = static_cast<uint16_t*>(ap.raw_cache[s]);
    uint16_t* conv_cache = static_cast<uint16_t*>(ap.conv_cache[s]);
    const int64_t base = seq * ap.max_t * 64 + ch;
    const float prev1 = from16<kBf16>(raw_cache[base + static_cast<int64_t>(max(t - 1, 0)) * 64]);
    const float prev2 = from16<kBf16>(raw_cache[base + static_cast<int64_t>(max(t - 2, 0)) * 64]);
    const float* w3 = ap.weight[s] + (static_cast<int64_t>(l) * 64 + ch) * 3;
    float conv = __fmul_rn(value, w3[2]);
    conv = __fadd_rn(conv, __fmul_rn(__fmul_rn(prev1, w3[1]), t >= 1 ? 1.0f : 0.0f));
    conv = __fadd_rn(conv, __fmul_rn(__fmul_rn(prev2, w3[0]), t >= 2 ? 1.0f : 0.0f));
    raw_cache[base + static_cast<int64_t>(t) * 64] = bits;
    conv_cache[base + static_cast<int64_t>(t) * 64] = to16<kBf16>(conv);
    // the block's rows are fetched sixteen at a time (independent loads in flight together), then
    // folded in ascending order; the second pass finds them in L1
    const int cur = t - start;
    const uint16_t* column = conv_cache + base + static_cast<int64_t>(start) * 64;
    float sum = 0.0f;
    for (int r0 = 0; r0 < bs; r0 += 16) {
        uint16_t raw16[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) raw16[i] = r0 + i < bs ? column[static_cast<int64_t>(r0 + i) * 64] : 0;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (r0 + i < bs) sum = __fadd_rn(sum, r0 + i == cur ? conv : from16<kBf16>(raw16[i]));
    }
    const float mean = __fdiv_rn(sum, static_cast<float>(bs));
    float acc = 0.0f;
    for (int r0 = 0; r0 < bs; r0 += 16) {
        uint16_t raw16[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) raw16[i] = r0 + i < bs ? column[static_cast<int64_t>(r0 + i) * 64] : 0;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (r0 + i < bs) {
                const float dv = __fsub_rn(r0 + i == cur ? conv : from16<kBf16>(raw16[i]), mean);
                acc = __fmaf_rn(dv, dv, acc);
            }
    }
    const float sd = __fsqrt_rn(__fdiv_rn(acc, static_cast<float>(bs)));
    const int64_t stat = (seq * ap.n_blocks + blk) * 64 + ch;
    static_cast<uint16_t*>(ap.mean[s])[stat] = to16<kBf16>(mean);
    static_cast<uint16_t*>(ap.stdv[s])[stat] = to16<kBf16>(sd);
}

template <bool kBf16>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    if (kBf16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// kSteps = d / 32 steps of 32 k-values; kUpper: rows 8..15 of x exist (more than eight rows).
template <int kSteps, bool kUpper, bool kBf16, bool kAppend>
__global__ void __launch_bounds__(kSkThreads) skinny_projection_kernel(const SkinnyArgs a, const SkinnyAppend ap) {
    // rows of x in the operands' own 16-bit format, each row padded by 64 bytes: the two rows a
    // quarter warp reads (64 bytes of each) lie in different halves of the banks
    extern __shared__ __align__(16) unsigned char xs[];
    __shared__ unsigned long long cta_best[kSkMaxRows];
    __shared__ unsigned int last_flag;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int d = a.d;
    const uint32_t row_bytes = static_cast<uint32_t>(d) * 2u + 64u;
    const int n_row = lane >> 2, part = lane & 3;
    const int warps_total = gridDim.x * kSkWarps;
    int g = blockIdx.x * kSkWarps + warp;

    // this warp's first eight weight rows, requested before anything an earlier kernel produced
    uint4 wreg[kSteps];
    auto load_group = [&](int group) {
        const int col = group * 8 + n_row;
        const uint4* wrow = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.w) +
                                                           static_cast<size_t>(col < a.n ? col : a.n - 1) * d);
#pragma unroll
        for (int s = 0; s < kSteps; ++s) wreg[s] = wrow[4 * s + part];
    };
    if (g < a.groups) load_group(g);
    if (tid < kSkMaxRows) cta_best[tid] = 0ull;
    griddep_sync();
    for (int i = tid; i < (kUpper ? 16 : 8) * (d / 8); i += kSkThreads) {
        const int m = i / (d / 8), c = i - m * (d / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < a.rows)
            v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.x) + static_cast<size_t>(m) * a.x_stride + 8 * c);
        *reinterpret_cast<uint4*>(xs + m * row_bytes + 16 * c) = v;
    }
    __syncthreads();
    int t = 0;
    if (kAppend) {
        t = static_cast<int>(*ap.position);
        const int blk = t / ap.block_size;
        if (t < 0 || t >= ap.max_t || blk >= ap.n_blocks || (blk + 1) * ap.block_size > ap.max_t) {
            if (tid == 0 && ap.status) atomicOr(ap.status, RLM_DEV_POSITION);
            return;
        }
    }

    unsigned long long best_lo = 0ull, best_hi = 0ull;         // arg-max keys of rows n_row and n_row + 8
    for (; g < a.groups; g += warps_total) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const unsigned char* xlo = xs + n_row * row_bytes + 16 * part;
        const unsigned char* xhi = xlo + 8 * row_bytes;
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            // eight consecutive k-values of weight row n_row, and of rows n_row / n_row + 8 of x at the same k
            const uint4 lo = *reinterpret_cast<const uint4*>(xlo + 64 * s);
            uint4 hi = make_uint4(0, 0, 0, 0);
            if (kUpper) hi = *reinterpret_cast<const uint4*>(xhi + 64 * s);
            mma16816<kBf16>(acc, lo.x, hi.x, lo.y, hi.y, wreg[s].x, wreg[s].y);
            mma16816<kBf16>(acc, lo.z, hi.z, lo.w, hi.w, wreg[s].z, wreg[s].w);
        }
        const int group = g;
        const int next = g + warps_total;
        if (next < a.groups) load_group(next);
        // this lane holds out[n_row][2 part, 2 part + 1] and out[n_row + 8][same columns]
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = n_row + (e >> 1) * 8, col = group * 8 + 2 * part + (e & 1);
            if ((e >> 1) && !kUpper) continue;
            if (m >= a.rows || col >= a.n) continue;
            float value = acc[e] + (a.bias ? a.bias[col] : 0.0f);
            uint16_t bits;
            if (kBf16) { __nv_bfloat16 h = __float2bfloat16_rn(value); bits = *reinterpret_cast<uint16_t*>(&h); value = __bfloat162float(h); }
            else { __half h = __float2half_rn(value); bits = *reinterpret_cast<uint16_t*>(&h); value = __half2float(h); }
            if (a.out) static_cast<uint16_t*>(a.out)[static_cast<size_t>(m) * a.n + col] = bits;
            if (kAppend) append_output<kBf16>(ap, a.rows, m, col, t, bits, value);
            if (!kAppend && a.keys && col < a.vocab) {
                const unsigned long long key = (static_cast<unsigned long long>(float_key(value + 0.0f)) << 32) |
                                               (0xffffffffu - static_cast<unsigned int>(col));
                if (e >> 1) best_hi = key > best_hi ? key : best_hi;
                else best_lo = key > best_lo ? key : best_lo;
            }
        }
    }
    if (!kAppend && a.keys) {
        // the four lanes of a row, then the CTA's warps through shared memory, then one atomic per row
#pragma unroll
        for (int off = 1; off < 4; off <<= 1) {
            const unsigned long long o_lo = __shfl_xor_sync(0xffffffffu, best_lo, off);
            const unsigned long long o_hi = __shfl_xor_sync(0xffffffffu, best_hi, off);
            best_lo = o_lo > best_lo ? o_lo : best_lo;
            best_hi = o_hi > best_hi ? o_hi : best_hi;
        }
        if (part == 0) {
            if (best_lo) atomicMax(&cta_best[n_row], best_lo);
            if (kUpper && best_hi) atomicMax(&cta_best[n_row + 8], best_hi);
        }
        __syncthreads();
        if (tid < a.rows && cta_best[tid]) atomicMax(a.keys + tid, cta_best[tid]);
        __threadfence();
        __syncthreads();
        if (tid == 0) last_flag = atomicAdd(a.counter, 1u) == gridDim.x - 1 ? 1u : 0u;
        __syncthreads();
        if (last_flag) {                                        // every CTA's keys are in: finalise
            __threadfence();
            if (tid < a.rows) {
                const unsigned long long key = atomicExch(a.keys + tid, 0ull);
                a.next_token[tid] = key ? static_cast<int64_t>(0xffffffffu - static_cast<unsigned int>(key & 0xffffffffu)) : 0;
            }
            if (tid == 0) {
                *a.counter = 0u;
                if (a.position) *a.position += 1;
            }
        }
    }
}

// ---- the front of a decode step in one launch: embedding + two LayerNorms + two projections
//
//   x[b]   = (token_embedding[tokens[b]] + boundary_embedding[boundaries[b]]) * scale + position_embedding[t]
//   out_first  = LayerNorm_1(x) @ w[:n_first].T        (the packed projection of the memory-normed rows)
//   out_second = LayerNorm_2(x) @ w[n_first:].T        (layer 0's query projection of its input-normed rows)
// (src/relation_lm/models/relation_lm.py:130-131, src/relation_lm/inference/packed_cache.py:52-57 of
// the reference project).  Every CTA builds the at most 16 embedded rows and both normalised copies
// in its own shared memory (a warp per row: a few KB out of L2) instead of reading them from a
// launch of their own, then streams its share of the concatenated weight exactly as
// skinny_projection_kernel does.  CTA 0 also stores x (fp32) and the two normalised rows.
struct FrontArgs {
    SkinnyArgs proj;          // w = concatenated weight [n, d]; out = out_first [M, n_first]; no bias, no head
    void* out_second;         // [M, n - n_first]
    int n_first;              // a multiple of 8
    const int64_t* tokens;
    const int64_t* boundaries;
    const void* token_table;
    const void* boundary_table;
    const float* position_table;
    const int64_t* position;
    float* hidden;            // [M, d] fp32
    int32_t* status;
    float scale, eps;
    int vocab, boundary_vocab, max_t;
    const float* norm_w[2];
    const float* norm_b[2];
    void* norm_out[2];        // [M, d] 16-bit
};

template <int kSteps, bool kUpper, bool kBf16>
__global__ void __launch_bounds__(kSkThreads) skinny_front_kernel(const FrontArgs f) {
    extern __shared__ __align__(16) unsigned char xs[];
    const SkinnyArgs& a = f.proj;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int d = 32 * kSteps, per = kSteps;                // columns per lane of a row: d / 32
    constexpr int kRows = kUpper ? 16 : 8;
    const uint32_t row_bytes = static_cast<uint32_t>(d) * 2u + 64u;
    unsigned char* xs_second = xs + kRows * row_bytes;
    const int n_row = lane >> 2, part = lane & 3;
    const int warps_total = gridDim.x * kSkWarps;
    int g = blockIdx.x * kSkWarps + warp;

    uint4 wreg[kSteps];
    auto load_group = [&](int group) {
        const int col = group * 8 + n_row;
        const uint4* wrow = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.w) +
                                                           static_cast<size_t>(col < a.n ? col : a.n - 1) * d);
#pragma unroll
        for (int s = 0; s < kSteps; ++s) wreg[s] = wrow[4 * s + part];
    };
    if (g < a.groups) load_group(g);
    griddep_sync();
    const int t = static_cast<int>(*f.position);
    if (t < 0 || t >= f.max_t) {
        if (tid == 0 && f.status) atomicOr(f.status, RLM_DEV_POSITION);
        return;
    }
    // a warp per row: this lane's `per` consecutive columns
    for (int m = warp; m < kRows; m += kSkWarps) {
        uint16_t* x1 = reinterpret_cast<uint16_t*>(xs + m * row_bytes) + per * lane;
        uint16_t* x2 = reinterpret_cast<uint16_t*>(xs_second + m * row_bytes) + per * lane;
        if (m >= a.rows) {
#pragma unroll
            for (int i = 0; i < per; ++i) { x1[i] = 0; x2[i] = 0; }
            continue;
        }
        int64_t tok = f.tokens[m], bnd = f.boundaries[m];
        if (tok < 0 || tok >= f.vocab || bnd < 0 || bnd >= f.boundary_vocab) {
            if (lane == 0 && f.status) atomicOr(f.status, RLM_DEV_POSITION);
            tok = 0;
            bnd = 0;
        }
        const int c0 = per * lane;
        float v[per];
        {
            const uint16_t* tr = static_cast<const uint16_t*>(f.token_table) + tok * d + c0;
            const uint16_t* br = static_cast<const uint16_t*>(f.boundary_table) + bnd * d + c0;
            const float* pr = f.position_table + static_cast<int64_t>(t) * d + c0;
#pragma unroll
            for (int i = 0; i < per; i += 8) {
                const uint4 tv = *reinterpret_cast<const uint4*>(tr + i), bv = *reinterpret_cast<const uint4*>(br + i);
                const uint16_t* th = reinterpret_cast<const uint16_t*>(&tv);
                const uint16_t* bh = reinterpret_cast<const uint16_t*>(&bv);
                const float4 p0 = *reinterpret_cast<const float4*>(pr + i), p1 = *reinterpret_cast<const float4*>(pr + i + 4);
                const float pe[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // the sum of the two embeddings is rounded to the table dtype first (an addition of two 16-bit tensors)
                    const float e = from16<kBf16>(to16<kBf16>(from16<kBf16>(th[j]) + from16<kBf16>(bh[j])));
                    v[i + j] = e * f.scale + pe[j];
                }
            }
        }
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < per; ++i) sum += v[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        const float mean = sum / static_cast<float>(d);
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < per; ++i) { const float dv = v[i] - mean; sq = fmaf(dv, dv, sq); }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
        const float inv = rsqrtf(sq / static_cast<float>(d) + f.eps);
        const bool store = blockIdx.x == 0;
        if (store) {
#pragma unroll
            for (int i = 0; i < per; i += 4)
                *reinterpret_cast<float4*>(f.hidden + static_cast<int64_t>(m) * d + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            uint16_t* xk = k ? x2 : x1;
            const float4* gw = reinterpret_cast<const float4*>(f.norm_w[k] + c0);
            const float4* gb = reinterpret_cast<const float4*>(f.norm_b[k] + c0);
#pragma unroll
            for (int i = 0; i < per; i += 8) {
                const float4 w0 = gw[i / 4], w1 = gw[i / 4 + 1], b0 = gb[i / 4], b1 = gb[i / 4 + 1];
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                uint32_t packed[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint16_t lo = to16<kBf16>(fmaf((v[i + 2 * e] - mean) * inv, wv[2 * e], bv[2 * e]));
                    const uint16_t hi = to16<kBf16>(fmaf((v[i + 2 * e + 1] - mean) * inv, wv[2 * e + 1], bv[2 * e + 1]));
                    packed[e] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
                }
                const uint4 chunk = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4*>(xk + i) = chunk;
                if (store && f.norm_out[k])
                    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(f.norm_out[k]) + static_cast<int64_t>(m) * d + c0 + i) = chunk;
            }
        }
    }
    __syncthreads();

    for (; g < a.groups; g += warps_total) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const bool second = g * 8 >= f.n_first;
        const unsigned char* xlo = (second ? xs_second : xs) + n_row * row_bytes + 16 * part;
        const unsigned char* xhi = xlo + 8 * row_bytes;
#pragma unroll
        for (int s = 0; s < kSteps; ++s) {
            const uint4 lo = *reinterpret_cast<const uint4*>(xlo + 64 * s);
            uint4 hi = make_uint4(0, 0, 0, 0);
            if (kUpper) hi = *reinterpret_cast<const uint4*>(xhi + 64 * s);
            mma16816<kBf16>(acc, lo.x, hi.x, lo.y, hi.y, wreg[s].x, wreg[s].y);
            mma16816<kBf16>(acc, lo.z, hi.z, lo.w, hi.w, wreg[s].z, wreg[s].w);
        }
        const int group = g;
        const int next = g + warps_total;
        if (next < a.groups) load_group(next);
        uint16_t* out = static_cast<uint16_t*>(second ? f.out_second : a.out);
        const int width = second ? a.n - f.n_first : f.n_first, first_col = second ? f.n_first : 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = n_row + (e >> 1) * 8, col = group * 8 + 2 * part + (e & 1);
            if ((e >> 1) && !kUpper) continue;
            if (m >= a.rows || col >= a.n) continue;
            out[static_cast<size_t>(m) * width + col - first_col] = to16<kBf16>(acc[e]);
        }
    }
}

template <int kSteps, bool kUpper>
int launch_front(const FrontArgs& f, void* stream) {
    auto kernel = f.proj.dtype == RLM_BF16 ? skinny_front_kernel<kSteps, kUpper, true> : skinny_front_kernel<kSteps, kUpper, false>;
    const int smem = 2 * (kUpper ? 16 : 8) * (f.proj.d * 2 + 64);
    int ctas = (f.proj.groups + kSkWarps - 1) / kSkWarps;
    if (ctas > 4 * sm_count()) ctas = 4 * sm_count();
    launch_kernel(kernel, dim3(ctas), dim3(kSkThreads), smem, stream, f);
    count_launch();
    return check_launch("skinny_front_kernel");
}

template <int kSteps, bool kUpper>
int launch_skinny(const SkinnyArgs& a, const SkinnyAppend* append, void* stream) {
    auto kernel = append ? (a.dtype == RLM_BF16 ? skinny_projection_kernel<kSteps, kUpper, true, true>
                                                : skinny_projection_kernel<kSteps, kUpper, false, true>)
                         : (a.dtype == RLM_BF16 ? skinny_projection_kernel<kSteps, kUpper, true, false>
                                                : skinny_projection_kernel<kSteps, kUpper, false, false>);
    const SkinnyAppend ap = append ? *append : SkinnyAppend{};
    const int smem = (kUpper ? 16 : 8) * (a.d * 2 + 64);
    // a warp per group of eight columns while they last, at most four CTAs per SM
    int ctas = (a.groups + kSkWarps - 1) / kSkWarps;
    if (ctas > 4 * sm_count()) ctas = 4 * sm_count();
    launch_kernel(kernel, dim3(ctas), dim3(kSkThreads), smem, stream, a, ap);
    count_launch();
    return check_launch("skinny_projection_kernel");
}

int dispatch_skinny(SkinnyArgs& a, const SkinnyAppend* append, void* stream) {
    a.groups = (a.n + 7) / 8;
    if (a.rows <= 8)
        return a.d == 256 ? launch_skinny<8, false>(a, append, stream) : launch_skinny<16, false>(a, append, stream);
    return a.d == 256 ? launch_skinny<8, true>(a, append, stream) : launch_skinny<16, true>(a, append, stream);
}

int check_skinny_operands(const void* x, int64_t x_row_stride, const void* weight, int rows, int d_in, int n_out,
                          int dtype) {
    if (!x || !weight) { set_error("skinny_projection: NULL pointer"); return RLM_ERR_NULL; }
    if (rows < 0 || rows > 16 || n_out < 1 || x_row_stride < d_in) {
        set_error("skinny_projection: at most 16 rows");
        return RLM_ERR_SHAPE;
    }
    if (d_in != 256 && d_in != 512) {
        set_error("skinny_projection: built for d = 256 and d = 512 (a warp's weight rows in registers); use rlm_packed_projection otherwise");
        return RLM_ERR_UNSUPPORTED;
    }
    if (dtype != RLM_BF16 && dtype != RLM_F16) {
        set_error("skinny_projection: bfloat16 or float16 operands");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(x) || !aligned16(weight) || (x_row_stride * 2) % 16 != 0) {
        set_error("skinny_projection: rows of x and the weight must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    return RLM_OK;
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_skinny_projection(const void* x, int64_t x_row_stride, const void* weight, const float* bias,
                                     void* out, int rows, int d_in, int n_out, int dtype, int vocab,
                                     void* argmax_scratch, int64_t* next_token, int64_t* position, void* stream) {
    using namespace rlm;
    if (rows == 0 || n_out == 0) return RLM_OK;
    if (!out) { set_error("skinny_projection: NULL pointer"); return RLM_ERR_NULL; }
    int rc = check_skinny_operands(x, x_row_stride, weight, rows, d_in, n_out, dtype);
    if (rc != RLM_OK) return rc;
    if (vocab > 0 && (!argmax_scratch || !next_token || vocab > n_out)) {
        set_error("skinny_projection: the greedy head needs scratch (rlm_skinny_argmax_scratch_bytes), next_token and vocab <= n");
        return RLM_ERR_NULL;
    }
    SkinnyArgs a{};
    a.x = x; a.w = weight; a.bias = bias; a.out = out; a.x_stride = x_row_stride;
    a.rows = rows; a.d = d_in; a.n = n_out; a.vocab = vocab > 0 ? vocab : 0; a.dtype = dtype;
    if (vocab > 0) {
        a.keys = static_cast<unsigned long long*>(argmax_scratch);
        a.counter = reinterpret_cast<unsigned int*>(static_cast<char*>(argmax_scratch) + 16 * 8);
        a.next_token = next_token;
        a.position = position;
    }
    return dispatch_skinny(a, nullptr, stream);
}

extern "C" int rlm_packed_projection_append(
    const void* x, int64_t x_row_stride, const void* weight, void* packed_out, int relation_dim,
    void* anchor_keys, void* partner_keys, void* operand_cache, void* partner_anchor_cache,
    void* anchor_raw_cache, void* partner_raw_cache, void* anchor_conv_cache, void* partner_conv_cache,
    void* anchor_mean, void* anchor_std, void* partner_mean, void* partner_std,
    const float* anchor_conv_weight, const float* partner_conv_weight, const int64_t* position,
    int layers, int batch, int d_in, int max_t, int n_blocks, int block_size, int dtype, int32_t* status,
    void* stream) {
    using namespace rlm;
    if (batch == 0) return RLM_OK;
    const void* need[] = {anchor_keys, partner_keys, operand_cache, partner_anchor_cache, anchor_raw_cache,
                          partner_raw_cache, anchor_conv_cache, partner_conv_cache, anchor_mean, anchor_std,
                          partner_mean, partner_std, anchor_conv_weight, partner_conv_weight, position};
    for (const void* q : need)
        if (!q) { set_error("packed_projection_append: NULL pointer"); return RLM_ERR_NULL; }
    if (layers < 1 || relation_dim < 8 || relation_dim % 8 != 0 || max_t < 1 || n_blocks < 1 || block_size < 1 ||
        n_blocks * block_size != max_t) {
        set_error("packed_projection_append: need layers >= 1, R a multiple of 8, T = blocks x block size");
        return RLM_ERR_SHAPE;
    }
    const int n_out = layers * (384 + relation_dim);
    int rc = check_skinny_operands(x, x_row_stride, weight, batch, d_in, n_out, dtype);
    if (rc != RLM_OK) return rc;
    SkinnyArgs a{};
    a.x = x; a.w = weight; a.out = packed_out; a.x_stride = x_row_stride;
    a.rows = batch; a.d = d_in; a.n = n_out; a.dtype = dtype;
    SkinnyAppend ap{};
    ap.token_cache[0] = anchor_keys; ap.token_cache[1] = partner_keys; ap.token_cache[2] = operand_cache;
    ap.token_cache[3] = partner_anchor_cache;
    ap.raw_cache[0] = anchor_raw_cache; ap.raw_cache[1] = partner_raw_cache;
    ap.conv_cache[0] = anchor_conv_cache; ap.conv_cache[1] = partner_conv_cache;
    ap.mean[0] = anchor_mean; ap.mean[1] = partner_mean; ap.stdv[0] = anchor_std; ap.stdv[1] = partner_std;
    ap.weight[0] = anchor_conv_weight; ap.weight[1] = partner_conv_weight;
    ap.position = position; ap.status = status; ap.max_t = max_t; ap.n_blocks = n_blocks; ap.block_size = block_size;
    ap.layers = layers; ap.rdim = relation_dim;
    return dispatch_skinny(a, &ap, stream);
}

extern "C" int rlm_decode_front(
    const int64_t* tokens, const int64_t* boundaries, const void* token_table, const void* boundary_table,
    const float* position_table, const int64_t* position, float scale, const float* norm1_weight,
    const float* norm1_bias, const float* norm2_weight, const float* norm2_bias, float norm_eps, const void* weight,
    float* hidden, void* norm1_out, void* norm2_out, void* out_first, void* out_second, int batch, int d_model,
    int n_first, int n_second, int vocab, int boundary_vocab, int max_t, int dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (batch == 0) return RLM_OK;
    if (!tokens || !boundaries || !token_table || !boundary_table || !position_table || !position || !norm1_weight ||
        !norm1_bias || !norm2_weight || !norm2_bias || !weight || !hidden || !out_first || !out_second) {
        set_error("decode_front: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (batch < 0 || batch > 16 || n_first < 8 || n_first % 8 != 0 || n_second < 1 || vocab < 1 || boundary_vocab < 1 ||
        max_t < 1) {
        set_error("decode_front: at most 16 rows; the first projection's width must be a multiple of 8");
        return RLM_ERR_SHAPE;
    }
    if (d_model != 256 && d_model != 512) {
        set_error("decode_front: built for d = 256 and d = 512");
        return RLM_ERR_UNSUPPORTED;
    }
    if (dtype != RLM_BF16 && dtype != RLM_F16) {
        set_error("decode_front: bfloat16 or float16 tables and weights");
        return RLM_ERR_UNSUPPORTED;
    }
    const void* vec[] = {token_table, boundary_table, position_table, norm1_weight, norm1_bias, norm2_weight, norm2_bias,
                         weight, hidden, norm1_out, norm2_out};
    for (const void* q : vec)
        if (q && !aligned16(q)) { set_error("decode_front: tensors must be 16-byte aligned"); return RLM_ERR_ALIGN; }
    FrontArgs f{};
    f.proj.w = weight; f.proj.out = out_first; f.proj.rows = batch; f.proj.d = d_model; f.proj.n = n_first + n_second;
    f.proj.dtype = dtype; f.proj.groups = (f.proj.n + 7) / 8;
    f.out_second = out_second; f.n_first = n_first;
    f.tokens = tokens; f.boundaries = boundaries; f.token_table = token_table; f.boundary_table = boundary_table;
    f.position_table = position_table; f.position = position; f.hidden = hidden; f.status = status;
    f.scale = scale; f.eps = norm_eps; f.vocab = vocab; f.boundary_vocab = boundary_vocab; f.max_t = max_t;
    f.norm_w[0] = norm1_weight; f.norm_w[1] = norm2_weight; f.norm_b[0] = norm1_bias; f.norm_b[1] = norm2_bias;
    f.norm_out[0] = norm1_out; f.norm_out[1] = norm2_out;
    if (batch <= 8) return d_model == 256 ? launch_front<8, false>(f, stream) : launch_front<16, false>(f, stream);
    return d_model == 256 ? launch_front<8, true>(f, stream) : launch_front<16, true>(f, stream);
}

// Bytes of the greedy head's scratch: 16 arg-max keys and the CTA counter.  Zero it once; every
// launch leaves it zero.
extern "C" int64_t rlm_skinny_argmax_scratch_bytes(void) { return 16 * 8 + 16; }
