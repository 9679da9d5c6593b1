// Shared device/host helpers for the relation_lm_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/relation_lm_b200.h"

namespace rlm {

// ------------------------------------------------------------------ host side

void set_error(const char* message);          // remembered per thread for rlm_last_error()
void count_launch();                          // bumps rlm_launch_count()
int check_launch(const char* kernel_name);    // cudaGetLastError -> rlm_status
// Opts a kernel into `bytes` of dynamic shared memory, once per device.
int allow_large_smem(const void* kernel, int bytes);

// Streaming multiprocessors of the current device (queried once per device; 148 on a B200).
int sm_count();

// Whether kernels are launched with programmatic stream serialisation (rlm_set_programmatic_launch).
bool programmatic_launch_enabled();

// Launches `kernel`; with programmatic launch enabled the grid may start while the kernel before
// it in the stream is still running, and every kernel here orders itself with griddep_wait()
// before it touches anything an earlier kernel may have produced.
template <typename... Params, typename... Args>
inline void launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem_bytes, void* stream,
                          Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem_bytes;
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attribute[1];
    if (programmatic_launch_enabled()) {
        attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[0].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
    }
    cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// The same for a kernel whose CTAs form clusters of `cluster_x` along x.
template <typename... Params, typename... Args>
inline void launch_kernel_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, unsigned cluster_x,
                                  size_t smem_bytes, void* stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem_bytes;
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster_x;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.numAttrs = 1;
    if (programmatic_launch_enabled()) {
        attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[1].val.programmaticStreamSerializationAllowed = 1;
        config.numAttrs = 2;
    }
    config.attrs = attribute;
    cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// Shared memory one CTA may use on sm_100 (227 KB) and the part of it the kernels here
// request dynamically (the rest covers their small static allocations).
constexpr int kSmemPerCta = 232448;
constexpr int kSmemDynamicLimit = kSmemPerCta - 1024;

inline bool valid_dtype(int d) { return d == RLM_F32 || d == RLM_BF16 || d == RLM_F16; }
inline int dtype_size(int d) { return d == RLM_F32 ? 4 : 2; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------ device side

constexpr float kNegInf = -__builtin_huge_valf();

// Programmatic dependent launch: wait until every kernel earlier in the stream has completed and
// its writes are visible (a no-op for an ordinary launch), then let the next kernel's CTAs start
// their own preamble.  Before the wait a kernel may only touch what no earlier kernel of the
// same stream can still be writing: its parameters (weights, tables) and its own shared memory.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_sync() { griddep_wait(); griddep_launch_dependents(); }

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

// One element of a tensor whose dtype is only known at run time (small tensors).
__device__ __forceinline__ float load_scalar(const void* base, int64_t index, int dtype) {
    if (dtype == RLM_F32) return static_cast<const float*>(base)[index];
    if (dtype == RLM_BF16)
        return bf16_bits_to_float(static_cast<const uint16_t*>(base)[index]);
    return __half2float(static_cast<const __half*>(base)[index]);
}

__device__ __forceinline__ void store_scalar(void* base, int64_t index, int dtype, float v) {
    if (dtype == RLM_F32) static_cast<float*>(base)[index] = v;
    else if (dtype == RLM_BF16) static_cast<__nv_bfloat16*>(base)[index] = __float2bfloat16_rn(v);
    else static_cast<__half*>(base)[index] = __float2half_rn(v);
}

// Eight consecutive elements starting at element index `first` (a multiple of
// 8) of a row that starts at `row` (16-byte aligned; shared or global).
__device__ __forceinline__ void load8(const void* row, int first, int dtype, float (&f)[8]) {
    if (dtype == RLM_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(row) + first);
        float4 a = p[0], b = p[1];
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
        f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        uint4 v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(row) + first);
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
        if (dtype == RLM_BF16) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                f[2 * i] = __uint_as_float(w[i] << 16);
                f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __half2 h = *reinterpret_cast<__half2*>(&w[i]);
                float2 p = __half22float2(h);
                f[2 * i] = p.x;
                f[2 * i + 1] = p.y;
            }
        }
    }
}

// Split form of load8 for software pipelining: fetch the raw bytes of eight elements now,
// convert them later (after more loads have been issued).
struct Raw8 { uint4 lo, hi; };

__device__ __forceinline__ Raw8 load8_raw(const void* row, int first, int dtype) {
    Raw8 r;
    if (dtype == RLM_F32) {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const float*>(row) + first);
        r.lo = p[0];
        r.hi = p[1];
    } else {
        r.lo = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(row) + first);
        r.hi = make_uint4(0, 0, 0, 0);
    }
    return r;
}

__device__ __forceinline__ void convert8(const Raw8& r, int dtype, float (&f)[8]) {
    if (dtype == RLM_F32) {
        f[0] = __uint_as_float(r.lo.x); f[1] = __uint_as_float(r.lo.y);
        f[2] = __uint_as_float(r.lo.z); f[3] = __uint_as_float(r.lo.w);
        f[4] = __uint_as_float(r.hi.x); f[5] = __uint_as_float(r.hi.y);
        f[6] = __uint_as_float(r.hi.z); f[7] = __uint_as_float(r.hi.w);
    } else {
        uint32_t w[4] = {r.lo.x, r.lo.y, r.lo.z, r.lo.w};
        if (dtype == RLM_BF16) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                f[2 * i] = __uint_as_float(w[i] << 16);
                f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __half2 h = *reinterpret_cast<__half2*>(&w[i]);
                float2 p = __half22float2(h);
                f[2 * i] = p.x;
                f[2 * i + 1] = p.y;
            }
        }
    }
}

// ---- canonical fp32 arithmetic: every operation that can move a selected
// index is spelled with an explicit rounding so that no contraction or
// reassociation can differ between builds.  exp/log are plain-fp32
// Cody-Waite/polynomial evaluations (not the hardware approximations), which
// makes block scores reproducible bit for bit by a CPU following the same steps.

__device__ __forceinline__ float canon_exp(float x) {
    if (x != x) return x;
    if (x < -86.0f) return 0.0f;
    if (x > 88.0f) return __int_as_float(0x7f800000);
    const float magic = 12582912.0f;  // 1.5 * 2^23
    float kf = __fsub_rn(__fmaf_rn(x, 1.44269502f, magic), magic);
    float r = __fmaf_rn(kf, -0.693145752f, x);
    r = __fmaf_rn(kf, -1.42860677e-06f, r);
    float p = 1.98412701e-04f;
    p = __fmaf_rn(p, r, 1.38888892e-03f);
    p = __fmaf_rn(p, r, 8.33333377e-03f);
    p = __fmaf_rn(p, r, 4.16666679e-02f);
    p = __fmaf_rn(p, r, 1.66666672e-01f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    int k = static_cast<int>(kf);
    return __int_as_float(__float_as_int(p) + k * (1 << 23));
}

__device__ __forceinline__ float canon_log(float y) {
    if (y != y || y < 0.0f) return __int_as_float(0x7fc00000);
    if (y == 0.0f) return kNegInf;
    if (y == __int_as_float(0x7f800000)) return y;
    int bits = __float_as_int(y);
    int e = (bits - 0x3f3504f3) >> 23;
    float m = __int_as_float(bits - e * (1 << 23));
    float f = __fsub_rn(m, 1.0f);
    float z = __fdiv_rn(f, __fadd_rn(2.0f, f));
    float w = __fmul_rn(z, z);
    float p = 9.09090936e-02f;
    p = __fmaf_rn(p, w, 1.11111112e-01f);
    p = __fmaf_rn(p, w, 1.42857149e-01f);
    p = __fmaf_rn(p, w, 0.2f);
    p = __fmaf_rn(p, w, 3.33333343e-01f);
    p = __fmul_rn(p, w);
    float z2 = __fadd_rn(z, z);
    float lm = __fmaf_rn(z2, p, z2);
    float ef = static_cast<float>(e);
    float r = __fmaf_rn(ef, 1.42860677e-06f, lm);
    return __fmaf_rn(ef, 0.693145752f, r);
}

// acc = 0; acc = fma(a[i], b[i], acc) for ascending i.
__device__ __forceinline__ float seg8(const float (&a)[8], const float (&b)[8]) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = __fmaf_rn(a[i], b[i], acc);
    return acc;
}

// ---- mbarrier + bulk (TMA, untiled) copies

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders earlier generic-proxy accesses to shared memory before later
// async-proxy (bulk copy) accesses to the same locations.
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after `limit` SM cycles and reports false.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - start > limit) return false;
    }
}

// The wait every kernel uses: about 2^31 SM cycles (roughly a second).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    return mbar_wait_limit(bar, parity, 1ll << 31);
}

// Global -> shared bulk copy; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// Shared -> global bulk copy (same alignment rules), tracked by the thread's bulk group.
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst), "r"(src), "r"(bytes)
                 : "memory");
}

// Closes the thread's bulk group and waits until its copies have read their shared-memory source.
__device__ __forceinline__ void bulk_commit_and_wait_read() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// 16-byte asynchronous global -> shared copy of this thread (L2 only), and its completion.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_group1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- warp helpers

// Order-preserving map of a float onto an unsigned key (larger float <=> larger key).
__device__ __forceinline__ uint32_t float_key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Arg-max over the warp of (key, slot) pairs with two redux instructions: the largest key
// wins, ties go to the lowest slot.  Lanes without a candidate pass slot = 0x7fffffff and
// key = 0.  All lanes receive the result.
__device__ __forceinline__ void warp_argmax_key(uint32_t& key, int& slot) {
    const uint32_t best = __reduce_max_sync(0xffffffffu, key);
    const uint32_t mine = key == best ? static_cast<uint32_t>(slot) : 0x7fffffffu;
    slot = static_cast<int>(__reduce_min_sync(0xffffffffu, mine));
    key = best;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

// LayerNorm of one row spread over a 256-thread CTA as four consecutive columns per thread
// (column c = 4 * threadIdx.x; `live` = c < dim), written as 16-bit values to up to two
// outputs that share the statistics but have their own affine parameters.  `scratch` holds 18
// floats of shared memory.  Two-pass statistics (mean, then biased variance) as layer_norm does.
struct NormTarget {
    const float* gamma;
    const float* beta;
    void* out_row;       // NULL: target unused
};

__device__ __forceinline__ float block_sum256(float v, float* scratch) {
    v = warp_sum(v);
    __syncthreads();                       // the previous use of scratch is over
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += scratch[w];
    return total;
}

__device__ __forceinline__ void block_layer_norm4(const float (&v)[4], bool live, int c, int dim, float eps,
                                                  const NormTarget& t0, const NormTarget& t1,
                                                  int out_dtype, float* scratch,
                                                  const float4* loaded_gamma = nullptr,
                                                  const float4* loaded_beta = nullptr) {
    const float mean = block_sum256(live ? (v[0] + v[1]) + (v[2] + v[3]) : 0.0f, scratch) / static_cast<float>(dim);
    float d[4], sq = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { d[i] = live ? v[i] - mean : 0.0f; sq = fmaf(d[i], d[i], sq); }
    const float inv = rsqrtf(block_sum256(sq, scratch) / static_cast<float>(dim) + eps);
    if (!live) return;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const NormTarget& t = k ? t1 : t0;
        if (!t.out_row) continue;
        // both targets of a caller that hands in loaded parameters share them
        const float4 g = loaded_gamma ? *loaded_gamma : *reinterpret_cast<const float4*>(t.gamma + c);
        const float4 b = loaded_beta ? *loaded_beta : *reinterpret_cast<const float4*>(t.beta + c);
        const float y0 = fmaf(d[0] * inv, g.x, b.x), y1 = fmaf(d[1] * inv, g.y, b.y);
        const float y2 = fmaf(d[2] * inv, g.z, b.z), y3 = fmaf(d[3] * inv, g.w, b.w);
        uint2 packed;
        if (out_dtype == RLM_BF16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
        } else {
            __half2 lo = __floats2half2_rn(y0, y1), hi = __floats2half2_rn(y2, y3);
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
        }
        *reinterpret_cast<uint2*>(static_cast<uint16_t*>(t.out_row) + c) = packed;
    }
}

}  // namespace rlm
