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
template <int kSteps, bool kUpper, bool kBf16>
__global__ void __launch_bounds__(kSkThreads) skinny_projection_kernel(const SkinnyArgs a) {
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
            static_cast<uint16_t*>(a.out)[static_cast<size_t>(m) * a.n + col] = bits;
            if (a.keys && col < a.vocab) {
                const unsigned long long key = (static_cast<unsigned long long>(float_key(value + 0.0f)) << 32) |
                                               (0xffffffffu - static_cast<unsigned int>(col));
                if (e >> 1) best_hi = key > best_hi ? key : best_hi;
                else best_lo = key > best_lo ? key : best_lo;
            }
        }
    }
    if (a.keys) {
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

template <int kSteps, bool kUpper>
int launch_skinny(const SkinnyArgs& a, void* stream) {
    auto kernel = a.dtype == RLM_BF16 ? skinny_projection_kernel<kSteps, kUpper, true> : skinny_projection_kernel<kSteps, kUpper, false>;
    const int smem = (kUpper ? 16 : 8) * (a.d * 2 + 64);
    // a warp per group of eight columns while they last, at most four CTAs per SM
    int ctas = (a.groups + kSkWarps - 1) / kSkWarps;
    if (ctas > 4 * 148) ctas = 4 * 148;
    launch_kernel(kernel, dim3(ctas), dim3(kSkThreads), smem, stream, a);
    count_launch();
    return check_launch("skinny_projection_kernel");
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_skinny_projection(const void* x, int64_t x_row_stride, const void* weight, const float* bias,
                                     void* out, int rows, int d_in, int n_out, int dtype, int vocab,
                                     void* argmax_scratch, int64_t* next_token, int64_t* position, void* stream) {
    using namespace rlm;
    if (rows == 0 || n_out == 0) return RLM_OK;
    if (!x || !weight || !out) { set_error("skinny_projection: NULL pointer"); return RLM_ERR_NULL; }
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
    a.groups = (n_out + 7) / 8;
    if (rows <= 8) return d_in == 256 ? launch_skinny<8, false>(a, stream) : launch_skinny<16, false>(a, stream);
    return d_in == 256 ? launch_skinny<8, true>(a, stream) : launch_skinny<16, true>(a, stream);
}

// Bytes of the greedy head's scratch: 16 arg-max keys and the CTA counter.  Zero it once; every
// launch leaves it zero.
extern "C" int64_t rlm_skinny_argmax_scratch_bytes(void) { return 16 * 8 + 16; }
