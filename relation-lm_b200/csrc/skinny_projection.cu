// Projection of a handful of rows (decode batches: at most 16) on the CUDA cores (sm_100a):
//   out[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n])
// for 16-bit x [M, d], w [N, d] with fp32 accumulation.  With so few rows the product is a stream
// of the weight matrix: no tensor-memory allocation, no tensor map, no shared-memory ring — every
// warp reads whole weight rows with 16-byte loads (requested before the dependency wait, they
// depend on no earlier kernel), multiplies them with the rows of x held as fp32 in shared memory
// and folds the 32 lanes' partial sums of (columns x rows) = 32 values with a halving butterfly
// (31 shuffles for all of them together).
//
// Optional greedy head (the `logits.argmax(-1)` and `position += 1` that close a decode step,
// src/relation_lm/models/relation_lm.py:204-207 of the reference project gives the heads): every
// CTA folds its columns below `vocab` into one 64-bit key per row (rounded logit, lowest index on
// ties) with atomicMax; the CTA that finishes last turns the keys into token ids, clears keys and
// counter for the next launch and advances the position.  The maximum does not depend on the
// order of the atomics, so the result is deterministic.
//
// Stands where the reference calls F.linear on one position's rows
// (src/relation_lm/inference/packed_cache.py:52-57; the heads of relation_lm.py:121-124).

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kSkThreads = 256;
constexpr int kSkWarps = kSkThreads / 32;

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
    int groups;               // column groups of kCols columns in total
};

// kRows: rows of x padded to 8 or 16; kCols = 32 / kRows columns per warp pass; kCpl: 16-byte
// chunks of a weight row per lane (d = 256 * kCpl).
template <int kRows, int kCpl, bool kBf16>
__global__ void __launch_bounds__(kSkThreads) skinny_projection_kernel(const SkinnyArgs a) {
    constexpr int kCols = 32 / kRows;
    extern __shared__ __align__(16) float xs[];               // [kRows][d]
    __shared__ unsigned int last_flag;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int dtype = kBf16 ? static_cast<int>(RLM_BF16) : static_cast<int>(RLM_F16);
    const int d = a.d;
    const int warps_total = gridDim.x * kSkWarps;
    const int first = blockIdx.x * kSkWarps + warp;

    // the first group's weight chunks, requested before anything an earlier kernel produced
    uint4 wreg[kCols][kCpl];
    auto load_group = [&](int g) {
#pragma unroll
        for (int c = 0; c < kCols; ++c) {
            const int col = g * kCols + c;
            const uint4* wrow = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.w) +
                                                               static_cast<size_t>(col < a.n ? col : a.n - 1) * d);
#pragma unroll
            for (int i = 0; i < kCpl; ++i) wreg[c][i] = wrow[lane + 32 * i];
        }
    };
    if (first < a.groups) load_group(first);
    griddep_sync();
    // rows of x as fp32 (rows beyond M: zeros)
    for (int i = tid; i < kRows * (d / 8); i += kSkThreads) {
        const int m = i / (d / 8), c = i - m * (d / 8);
        float f[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (m < a.rows)
            load8(static_cast<const uint16_t*>(a.x) + static_cast<size_t>(m) * a.x_stride, 8 * c, dtype, f);
        float4* dst = reinterpret_cast<float4*>(xs + m * d + 8 * c);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncthreads();

    unsigned long long best = 0ull;                             // this lane's (row, column slot) arg-max key
    for (int g = first; g < a.groups; g += warps_total) {
        float acc[kCols][kRows];
#pragma unroll
        for (int c = 0; c < kCols; ++c)
#pragma unroll
            for (int m = 0; m < kRows; ++m) acc[c][m] = 0.0f;
#pragma unroll
        for (int i = 0; i < kCpl; ++i) {
            float wf[kCols][8];
#pragma unroll
            for (int c = 0; c < kCols; ++c) {
                Raw8 r;
                r.lo = wreg[c][i];
                r.hi = make_uint4(0, 0, 0, 0);
                convert8(r, dtype, wf[c]);
            }
#pragma unroll
            for (int m = 0; m < kRows; ++m) {
                const float4* xp = reinterpret_cast<const float4*>(xs + m * d + 8 * (lane + 32 * i));
                const float4 x0 = xp[0], x1 = xp[1];
#pragma unroll
                for (int c = 0; c < kCols; ++c) {
                    float s = acc[c][m];
                    s = fmaf(wf[c][0], x0.x, s); s = fmaf(wf[c][1], x0.y, s); s = fmaf(wf[c][2], x0.z, s); s = fmaf(wf[c][3], x0.w, s);
                    s = fmaf(wf[c][4], x1.x, s); s = fmaf(wf[c][5], x1.y, s); s = fmaf(wf[c][6], x1.z, s); s = fmaf(wf[c][7], x1.w, s);
                    acc[c][m] = s;
                }
            }
        }
        const int next = g + warps_total;
        if (next < a.groups) load_group(next);                  // the next group's weights fly during the reduction
        // halving butterfly over the 32 (column, row) sums: lane l ends with the total of element l
        float v[32];
#pragma unroll
        for (int c = 0; c < kCols; ++c)
#pragma unroll
            for (int m = 0; m < kRows; ++m) v[c * kRows + m] = acc[c][m];
#pragma unroll
        for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
            const bool upper = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < n / 2; ++i) {
                const float keep = upper ? v[i + n / 2] : v[i];
                const float send = upper ? v[i] : v[i + n / 2];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
        }
        const int c = lane / kRows, m = lane - c * kRows;
        const int col = g * kCols + c;
        if (col < a.n && m < a.rows) {
            float value = v[0] + (a.bias ? a.bias[col] : 0.0f);
            uint16_t bits;
            if (kBf16) { __nv_bfloat16 h = __float2bfloat16_rn(value); bits = *reinterpret_cast<uint16_t*>(&h); value = __bfloat162float(h); }
            else { __half h = __float2half_rn(value); bits = *reinterpret_cast<uint16_t*>(&h); value = __half2float(h); }
            static_cast<uint16_t*>(a.out)[static_cast<size_t>(m) * a.n + col] = bits;
            if (a.keys && col < a.vocab) {
                const unsigned long long key = (static_cast<unsigned long long>(float_key(value + 0.0f)) << 32) |
                                               (0xffffffffu - static_cast<unsigned int>(col));
                best = key > best ? key : best;
            }
        }
    }
    if (a.keys) {
        // the lanes of one row (same m, different column slot) first, then one atomic per row and warp
#pragma unroll
        for (int off = kRows; off < 32; off <<= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, off);
            best = other > best ? other : best;
        }
        if (lane < kRows && lane < a.rows && best) atomicMax(a.keys + lane, best);
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

template <int kRows, int kCpl>
int launch_skinny(const SkinnyArgs& a, void* stream) {
    constexpr int kCols = 32 / kRows;
    auto kernel = a.dtype == RLM_BF16 ? skinny_projection_kernel<kRows, kCpl, true> : skinny_projection_kernel<kRows, kCpl, false>;
    const int smem = kRows * a.d * 4;
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    // enough CTAs to cover the SMs twice, never more warps than column groups
    int ctas = (a.groups + kSkWarps - 1) / kSkWarps;
    if (ctas > 2 * 148) ctas = 2 * 148;
    (void)kCols;
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
        set_error("skinny_projection: built for d = 256 and d = 512 (a weight row in registers); use rlm_packed_projection otherwise");
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
    const int cpl = d_in / 256;
    if (rows <= 8) {
        a.groups = (n_out + 3) / 4;
        return cpl == 1 ? launch_skinny<8, 1>(a, stream) : launch_skinny<8, 2>(a, stream);
    }
    a.groups = (n_out + 1) / 2;
    return cpl == 1 ? launch_skinny<16, 1>(a, stream) : launch_skinny<16, 2>(a, stream);
}

// Bytes of the greedy head's scratch: 16 arg-max keys and the CTA counter.  Zero it once; every
// launch leaves it zero.
extern "C" int64_t rlm_skinny_argmax_scratch_bytes(void) { return 16 * 8 + 16; }
