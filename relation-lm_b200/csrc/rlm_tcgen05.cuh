// tcgen05 / TMA building blocks shared by the tensor-core kernels of this library (sm_100a).
#pragma once

#include <cuda.h>

#include "rlm_common.cuh"

namespace rlm {

constexpr int kBM = 128;       // rows per tile == TMEM lanes
constexpr int kBK = 64;        // K elements per stage: 128 bytes, one swizzle atom

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle: 8-row groups 1024 bytes apart (stride byte offset), leading byte offset
// unused (1), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(addr));
}

__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(addr));
}

// ---- device helpers shared by the relation-MLP kernels

// GELU(x) = x * Phi(x) with Phi(x) = 1 - erfc(|x| / sqrt 2) / 2 mirrored for x < 0, erfc from the
// Abramowitz & Stegun 7.1.26 polynomial (absolute error below 1.5e-7) on the hardware
// reciprocal and exponential: about a third of the instructions of erff, enough for 16-bit
// outputs.  The polynomial coefficients carry the factor 1/2.
__device__ __forceinline__ float gelu_tc(float x) {
    const float z = fabsf(x) * 0.70710678118654752f;
    float t, e;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.0f)));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * z * -1.4426950408889634f));
    float p = 0.5307027145f;
    p = fmaf(p, t, -0.7265760135f);
    p = fmaf(p, t, 0.7107068705f);
    p = fmaf(p, t, -0.142248368f);
    p = fmaf(p, t, 0.127414796f);
    const float h = p * t * e;                 // erfc(z) / 2
    return x * (x >= 0.0f ? 1.0f - h : h);
}

// gelu_tc of two values at once on the two-wide fp32 instructions (the same operations in the same
// order, so each half equals gelu_tc of its input bit for bit): the epilogues that apply GELU to
// millions of values are bound by instruction issue, not by the arithmetic pipes.
__device__ __forceinline__ float2 gelu_tc2(float2 x) {
    const float2 z = __fmul2_rn(make_float2(fabsf(x.x), fabsf(x.y)), make_float2(0.70710678118654752f, 0.70710678118654752f));
    const float2 den = __ffma2_rn(make_float2(0.3275911f, 0.3275911f), z, make_float2(1.0f, 1.0f));
    const float2 arg = __fmul2_rn(__fmul2_rn(z, z), make_float2(-1.4426950408889634f, -1.4426950408889634f));
    float2 t, e;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.x) : "f"(den.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t.y) : "f"(den.y));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(arg.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(arg.y));
    float2 p = make_float2(0.5307027145f, 0.5307027145f);
    p = __ffma2_rn(p, t, make_float2(-0.7265760135f, -0.7265760135f));
    p = __ffma2_rn(p, t, make_float2(0.7107068705f, 0.7107068705f));
    p = __ffma2_rn(p, t, make_float2(-0.142248368f, -0.142248368f));
    p = __ffma2_rn(p, t, make_float2(0.127414796f, 0.127414796f));
    const float2 h = __fmul2_rn(__fmul2_rn(p, t), e);                                   // erfc(z) / 2
    const float2 c = __ffma2_rn(h, make_float2(-1.0f, -1.0f), make_float2(1.0f, 1.0f));  // 1 - h
    return __fmul2_rn(x, make_float2(x.x >= 0.0f ? c.x : h.x, x.y >= 0.0f ? c.y : h.y));
}

// Eight consecutive 16-bit values as four pairs (elements 2i, 2i + 1), for the two-wide instructions.
__device__ __forceinline__ void unpack8_pairs(const uint4& raw, int dtype, float2 (&f)[4]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (dtype == RLM_BF16) {
            f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
        } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            f[i] = __half22float2(h);
        }
    }
}

__device__ __forceinline__ void unpack8(const uint4& raw, int dtype, float (&f)[8]) {
    Raw8 r;
    r.lo = raw;
    r.hi = make_uint4(0, 0, 0, 0);
    convert8(r, dtype, f);
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int dtype) {
    if (dtype == RLM_BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Byte offset of 16-byte chunk c (0 .. R/8) of row r inside a K-major tile stored as
// K-blocks of `rows` x 128 bytes with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swizzled(int r, int c, uint32_t kblock_bytes) {
    return static_cast<uint32_t>(c >> 3) * kblock_bytes + static_cast<uint32_t>(r >> 3) * 1024u +
           static_cast<uint32_t>(r & 7) * 128u + static_cast<uint32_t>(((c & 7) ^ (r & 7)) << 4);
}

// ---- host side: tensor maps

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_fn() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

// [rows, cols] row-major 16-bit matrix, box = box_rows x 64 columns, 128-byte swizzle, zero fill.
inline bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int64_t row_stride_elems,
              int box_rows, int dtype) {
    EncodeTiled fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride_elems) * 2};
    cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(box_rows)};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMapDataType dt = dtype == RLM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


}  // namespace rlm
