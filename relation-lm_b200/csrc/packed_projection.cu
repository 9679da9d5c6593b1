// Packed sparse-cache / router projection on the 5th-generation tensor cores (sm_100a):
//   out[M, N] = x[M, K] . w[N, K]^T      bf16 or fp16 operands, fp32 accumulation in TMEM.
//
// One CTA per 128 x BN output tile.  A single producer thread streams 128 x 64 tiles of x
// and BN x 64 tiles of w into a 3- or 8-stage shared-memory ring with tiled TMA loads
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast); a single thread issues
// tcgen05.mma (UMMA 128 x BN x 16, both operands K-major from shared memory) and releases
// ring stages with tcgen05.commit; the four warps then read the accumulator with
// tcgen05.ld, convert and store.  Rows past M are zero-filled by TMA and not stored.
// Every wait is bounded; on expiry the kernel sets RLM_DEV_TIMEOUT, frees its TMEM and returns.
//
// Replaces the F.linear of src/relation_lm/inference/packed_cache.py:52-57 of the reference
// project (and serves the query-side router projections, which have the same shape).

#include "rlm_tcgen05.cuh"

namespace rlm {
namespace {

constexpr int kGemmThreads = 128;

// Ring depth: wide tiles use three stages (96 KB) so that two CTAs share an SM and one CTA's
// epilogue overlaps the other's main loop; narrow tiles (few rows, latency-bound) use eight so
// that a whole K = 512 reduction is requested at once.
__host__ __device__ constexpr int stages_for(int bn) { return bn >= 128 ? 3 : 8; }

struct GemmArgs {
    void* out;
    const float* bias;     // optional [n]: added to every row before the output is rounded
    int32_t* status;
    int m, n, k;
    int out_dtype;
    uint32_t idesc;
    uint32_t a_bytes;      // bytes one x tile load delivers (box rows x 128)
    int issuers;           // MMA-issuing warps (1 or 2)
    int k_blocks_per_split;  // K-blocks of 64 one CTA contracts (all of them without split K)
    int k_splits;
};

template <int BN>
__global__ void __launch_bounds__(kGemmThreads) packed_projection_kernel(
    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
    const GemmArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    constexpr int kStages = stages_for(BN);
    // one or two warps issue MMAs (K-blocks dealt round-robin into accumulators of their own, summed by
    // the epilogue): a single thread issues a tcgen05.mma every ~60 cycles, which bounds short
    // K loops; tensor-memory columns = issuers * BN, at least 32
    const int issuers = a.issuers;
    uint32_t tmem_cols = 32;
    while (tmem_cols < static_cast<uint32_t>(issuers * BN)) tmem_cols *= 2;
    constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = BN * kBK * 2;
    // the ring must start on a 1024-byte boundary for the 128-byte swizzle
    unsigned char* ring = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t ring_addr = smem_u32(ring);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * kBM;
    // split K: grid.z CTAs share an output tile, each contracts k_blocks_per_split K-blocks and
    // writes its own fp32 slice out[z] (summed by the consumer)
    const int k_first = blockIdx.z * a.k_blocks_per_split;
    const int k_iters = min((a.k + kBK - 1) / kBK - k_first, a.k_blocks_per_split);
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * kStages);

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int i = 0; i < 2 * kStages; ++i) mbar_init(bar0 + 8u * i, 1);
        mbar_init(acc_full, static_cast<uint32_t>(issuers));
        fence_barrier_init();
        failed = 0;
    }
    if (warp == 1) {   // one warp owns the TMEM allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    // Producer (warp 0): the first round of the ring is requested by one lane per stage at once
    // (the stages are free), later rounds by lane 0 as stages are released.  The weight tiles do
    // not depend on earlier kernels: they are requested before the dependency wait, x after it.
    if (warp == 0 && lane < kStages && lane < k_iters) {
        mbar_expect_tx(full(lane), a.a_bytes + kBBytes);
        tma_load_2d(ring_addr + lane * (kABytes + kBBytes) + kABytes, &map_w, (k_first + lane) * kBK, n0, full(lane));
    }
    griddep_sync();
    // barriers and tensor memory are set up; x may come from the previous kernel

    if (warp == 0) {
        if (lane < kStages && lane < k_iters)
            tma_load_2d(ring_addr + lane * (kABytes + kBBytes), &map_x, (k_first + lane) * kBK, m0, full(lane));
        __syncwarp();
        if (lane == 0) {
            for (int it = kStages; it < k_iters; ++it) {
                const int s = it % kStages;
                if (!mbar_wait(empty(s), ((it / kStages) - 1) & 1)) { failed = 1; break; }
                mbar_expect_tx(full(s), a.a_bytes + kBBytes);
                tma_load_2d(ring_addr + s * (kABytes + kBBytes), &map_x, (k_first + it) * kBK, m0, full(s));
                tma_load_2d(ring_addr + s * (kABytes + kBBytes) + kABytes, &map_w, (k_first + it) * kBK, n0, full(s));
            }
        }
        __syncwarp();
    } else if (warp <= issuers) {
        const int me = warp - 1;                              // issuer index: K-blocks me, me + issuers, ...
        const uint32_t my_acc = tmem_base + static_cast<uint32_t>(me * BN);
        // tensor-core issue: four UMMA K-steps of 16 per stage.  The whole warp walks the loop so
        // that addresses and descriptors stay warp-uniform; one lane issues the instructions.
        bool ok = true;
        for (int it = me; it < k_iters && ok; it += issuers) {
            const int s = it % kStages;
            ok = mbar_wait(full(s), (it / kStages) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = smem_desc_sw128(ring_addr + s * (kABytes + kBBytes));
            const uint64_t db = smem_desc_sw128(ring_addr + s * (kABytes + kBBytes) + kABytes);
            if (lane == 0) {
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)      // +32 bytes along K inside the swizzle atom
                    umma_f16(my_acc, da + 2 * kk, db + 2 * kk, a.idesc, (it >= issuers || kk > 0) ? 1u : 0u);
                umma_commit(empty(s));                       // stage reusable once these MMAs retire
            }
            __syncwarp();
        }
        if (lane == 0) {
            if (!ok) failed = 1;
            umma_commit(acc_full);                           // accumulator complete (or abandoned)
        }
    }
    __syncwarp();

    // epilogue: warp w reads TMEM lanes 32w .. 32w+31 (one output row per thread)
    bool ready = mbar_wait(acc_full, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ready = ready && (*reinterpret_cast<volatile int*>(&failed) == 0);
    if (!__syncthreads_or(!ready)) {
        const int row = m0 + warp * 32 + lane;
#pragma unroll 1                 // executed once per CTA: compact code beats unrolling
        for (int c = 0; c < BN; c += 16) {
            uint32_t v[16];
            tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            for (int extra = 1; extra < issuers; ++extra) {
                uint32_t v2[16];
                tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + extra * BN + c, v2);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(v2[i]));
            }
            if (a.bias) {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + a.bias[n0 + c + i]);
            }
            if (row < a.m) {
                const size_t at = (static_cast<size_t>(blockIdx.z) * a.m + row) * a.n + n0 + c;
                if (a.out_dtype == RLM_F32) {
                    float4* o = reinterpret_cast<float4*>(static_cast<float*>(a.out) + at);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        o[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                           __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                } else {
                    uint32_t packed[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float lo = __uint_as_float(v[2 * i]), hi = __uint_as_float(v[2 * i + 1]);
                        if (a.out_dtype == RLM_BF16) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                            packed[i] = *reinterpret_cast<uint32_t*>(&h);
                        } else {
                            __half2 h = __floats2half2_rn(lo, hi);
                            packed[i] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    }
                    uint4* o = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + at);
                    o[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    o[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        }
    } else if (tid == 0 && a.status) {
        atomicOr(a.status, RLM_DEV_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(tmem_cols) : "memory");
}

// ------------------------------------------------------------------ many rows: persistent CTAs
//
// Products with thousands of rows (whole-sequence passes).  One CTA per SM walks output tiles
// (n-tiles fastest, so that the CTAs running at the same time share their x rows in L2); three
// roles, each on bounded waits:
//   warp 0, one lane: TMA producer, a ring of stages (x rows x 64 | w 256 x 64);
//   warp 1, one lane: tcgen05.mma 128 x 256 x 16;
//   warps 2-9: epilogue (tcgen05.ld, bias, convert, store; two warps per quarter of the TMEM lanes,
//   128 columns each).
// kRowTiles = 1: tiles of 128 x 256, two accumulators (2 x 256 TMEM columns) used by alternate
// tiles, so that a tile's epilogue runs behind the next tile's main loop.
// kRowTiles = 2: tiles of 256 x 256 — two row tiles share every w tile, which halves the weight
// traffic per output: without a two-SM MMA every CTA fetches its operands through its own
// 64-byte-per-clock L2 port, and at 85 flop per byte (128 x 256) that port, not the tensor pipe,
// sets the pace.  Both accumulators belong to one tile; the next tile's MMAs into an accumulator
// start as soon as the epilogue has read it out.
constexpr int kPgThreads = 320;
constexpr int kPgBN = 256;

struct PersistentGemmArgs {
    void* out;
    const float* bias;
    int32_t* status;
    int m, n, k, out_dtype;
    uint32_t idesc;
    int tiles_n, tiles;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <int kRowTiles>
__global__ void __launch_bounds__(kPgThreads, 1) packed_projection_persistent_kernel(
    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
    const PersistentGemmArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int kStages = kRowTiles == 2 ? 3 : 4;
    __shared__ __align__(8) unsigned long long bars[2 * kStages + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    constexpr int kTileRows = kBM * kRowTiles;
    constexpr uint32_t kABytes = kTileRows * kBK * 2, kBBytes = kPgBN * kBK * 2, kStageBytes = kABytes + kBBytes;
    unsigned char* ring = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t ring_addr = smem_u32(ring);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int k_blocks = a.k / kBK;
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int i = 0; i < 2 * kStages; ++i) mbar_init(bar0 + 8u * i, 1);
        mbar_init(acc_full(0), 1);
        mbar_init(acc_full(1), 1);
        mbar_init(acc_empty(0), 8);                  // one arrival per epilogue warp
        mbar_init(acc_empty(1), 8);
        fence_barrier_init();
        failed = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(2 * kPgBN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    griddep_sync();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                          // stage uses so far, across tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / a.tiles_n) * kTileRows, n0 = (tile % a.tiles_n) * kPgBN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages && !mbar_wait(empty(s), ((it / kStages) - 1) & 1)) { ok = false; break; }
                    mbar_expect_tx(full(s), kStageBytes);
                    tma_load_2d(ring_addr + s * kStageBytes, &map_x, kb * kBK, m0, full(s));
                    tma_load_2d(ring_addr + s * kStageBytes + kABytes, &map_w, kb * kBK, n0, full(s));
                }
            }
            if (!ok) failed = 1;
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, j = 0;                                   // stage uses / tiles so far
            bool ok = true;
            for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x, ++j) {
                // kRowTiles == 1: accumulator j & 1, free once the epilogue of tile j - 2 has read it out.
                // kRowTiles == 2: both accumulators, each free once the epilogue of tile j - 1 has read it out.
                const int b = kRowTiles == 1 ? (j & 1) : 0;
                if (kRowTiles == 1 && j >= 2 && !mbar_wait(acc_empty(b), ((j >> 1) - 1) & 1)) { ok = false; break; }
                for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(full(s), (it / kStages) & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t db = smem_desc_sw128(ring_addr + s * kStageBytes + kABytes);
#pragma unroll
                    for (int r = 0; r < kRowTiles; ++r) {
                        if (kRowTiles == 2 && kb == 0 && j >= 1) {
                            if (!mbar_wait(acc_empty(r), (j - 1) & 1)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        const uint32_t acc = tmem_base + static_cast<uint32_t>((kRowTiles == 1 ? b : r) * kPgBN);
                        const uint64_t da = smem_desc_sw128(ring_addr + s * kStageBytes + r * (kBM * kBK * 2));
#pragma unroll
                        for (int kk = 0; kk < kBK / 16; ++kk)
                            umma_f16(acc, da + 2 * kk, db + 2 * kk, a.idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(empty(s));
                }
                umma_commit(acc_full(b));                        // tile complete (or abandoned)
            }
            if (!ok) failed = 1;
        }
        __syncwarp();
    } else {
        // epilogue warps 2 .. 9: TMEM lanes 32 (warp % 4) .., one output row and 128 columns per thread
        const int quarter = warp & 3, col_half = (warp - 2) >> 2;
        const uint32_t lane_base = static_cast<uint32_t>(32 * quarter) << 16;
        int j = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < a.tiles && ok; tile += gridDim.x, ++j) {
            const int b = kRowTiles == 1 ? (j & 1) : 0;
            const int m0 = (tile / a.tiles_n) * kTileRows, n0 = (tile % a.tiles_n) * kPgBN;
            ok = mbar_wait(acc_full(b), kRowTiles == 1 ? ((j >> 1) & 1) : (j & 1));
            ok = __all_sync(0xffffffffu, ok) && (*reinterpret_cast<volatile int*>(&failed) == 0);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int r = 0; r < kRowTiles; ++r) {
                const int accn = kRowTiles == 1 ? b : r;
                const int row = m0 + kBM * r + 32 * quarter + lane;
#pragma unroll 1
                for (int c = col_half * (kPgBN / 2); c < (col_half + 1) * (kPgBN / 2); c += 32) {
                    uint32_t v[32];
                    tmem_ld16(tmem_base + lane_base + accn * kPgBN + c, *reinterpret_cast<uint32_t(*)[16]>(&v[0]));
                    tmem_ld16(tmem_base + lane_base + accn * kPgBN + c + 16, *reinterpret_cast<uint32_t(*)[16]>(&v[16]));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c + 32 == (col_half + 1) * (kPgBN / 2)) {
                        // this warp's share of the accumulator is in registers: hand it back to the MMA warp
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty(accn));
                    }
                    if (a.bias) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + a.bias[n0 + c + i]);
                    }
                    if (row >= a.m) continue;
                    const size_t at = static_cast<size_t>(row) * a.n + n0 + c;
                    if (a.out_dtype == RLM_F32) {
                        float4* o = reinterpret_cast<float4*>(static_cast<float*>(a.out) + at);
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            o[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                               __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                    } else {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float lo = __uint_as_float(v[2 * i]), hi = __uint_as_float(v[2 * i + 1]);
                            if (a.out_dtype == RLM_BF16) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                                packed[i] = *reinterpret_cast<uint32_t*>(&h);
                            } else {
                                __half2 h = __floats2half2_rn(lo, hi);
                                packed[i] = *reinterpret_cast<uint32_t*>(&h);
                            }
                        }
                        uint4* o = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + at);
#pragma unroll
                        for (int i = 0; i < 4; ++i) o[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
                    }
                }
            }
        }
        if (!ok && lane == 0) failed = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && a.status && *reinterpret_cast<volatile int*>(&failed)) atomicOr(a.status, RLM_DEV_TIMEOUT);
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(2 * kPgBN) : "memory");
}

template <int kRowTiles>
int launch_persistent_gemm(const CUtensorMap& mx, const CUtensorMap& mw, PersistentGemmArgs& a, void* stream) {
    constexpr int kStages = kRowTiles == 2 ? 3 : 4;
    const int smem_bytes = kStages * (kRowTiles * kBM * kBK * 2 + kPgBN * kBK * 2) + 1024;
    auto kernel = packed_projection_persistent_kernel<kRowTiles>;
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    a.tiles_n = a.n / kPgBN;
    a.tiles = a.tiles_n * ((a.m + kRowTiles * kBM - 1) / (kRowTiles * kBM));
    const int ctas = a.tiles < sm_count() ? a.tiles : sm_count();
    launch_kernel(kernel, dim3(ctas), dim3(kPgThreads), smem_bytes, stream, mx, mw, a);
    count_launch();
    return check_launch("packed_projection_persistent_kernel");
}

// ------------------------------------------------------------------ LayerNorm + projection
//
// out = LayerNorm(x) . w^T for fp32 rows (decode batches): every CTA normalises the (at most
// 128) rows of its tile itself (a few KB), writes them as 16-bit values straight into the swizzled
// K-major layout the tensor core reads, and streams only its BN x K slice of w with TMA.
// The x tile of K-block kb starts kb * a_stride bytes into the A region, a_stride covering
// just the row groups that exist; the MMA reads 128 rows from there, rows that do not exist
// land in accumulator lanes that are never stored.

struct NormGemmArgs {
    const float* x;
    const float* gamma;
    const float* beta;
    void* out;
    int32_t* status;
    int64_t x_stride;
    float eps;
    int m, n, k;
    int w_dtype, out_dtype;
    uint32_t idesc;
    uint32_t a_stride;     // bytes between consecutive K-blocks of the x tile
    uint32_t a_bytes;      // size of the A region (multiple of 1024)
    int tile_rows;         // rows per CTA (multiple of 8, at most 128)
};

constexpr int kNormMaxPerLane = 4;     // 16-byte chunks per lane: d_in <= 1024

template <int BN>
__global__ void __launch_bounds__(kGemmThreads) norm_projection_kernel(
    const __grid_constant__ CUtensorMap map_w, const NormGemmArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * 8 + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    constexpr int kStages = 8;
    constexpr int kTmemCols = BN < 32 ? 32 : BN;
    constexpr uint32_t kBBytes = BN * kBK * 2;
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* a_tile = base;
    const uint32_t a_addr = smem_u32(a_tile);
    const uint32_t ring_addr = a_addr + a.a_bytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * a.tile_rows;
    const int m_here = min(a.m - m0, a.tile_rows);
    const int k_iters = (a.k + kBK - 1) / kBK;
    const uint32_t bar0 = smem_u32(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
    const uint32_t acc_full = bar0 + 8u * (2 * kStages);

    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        for (int i = 0; i < 2 * kStages + 1; ++i) mbar_init(bar0 + 8u * i, 1);
        fence_barrier_init();
        failed = 0;
        // the weight slice does not depend on the normalisation: request it first
        for (int it = 0; it < k_iters && it < kStages; ++it) {
            mbar_expect_tx(full(it), kBBytes);
            tma_load_2d(ring_addr + it * kBBytes, &map_w, it * kBK, n0, full(it));
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // LayerNorm of the rows, one warp per row, lane l owns the 16-byte chunks l, l+32, ...
    griddep_sync();      // the weight slice is on its way; x may come from the previous kernel
    const int chunks = a.k / 8;
    // two rows of a warp are in flight at a time (their loads are issued before either reduction)
    for (int r0 = warp; r0 < m_here; r0 += 2 * (kGemmThreads / 32)) {
        float v[2][kNormMaxPerLane][8];
        float sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int r = r0 + u * (kGemmThreads / 32);
            if (r >= m_here) continue;
            const float* row = a.x + (m0 + r) * a.x_stride;
#pragma unroll
            for (int i = 0; i < kNormMaxPerLane; ++i) {
                const int c = lane + 32 * i;
                if (c < chunks) {
                    const float4 lo = *reinterpret_cast<const float4*>(row + 8 * c);
                    const float4 hi = *reinterpret_cast<const float4*>(row + 8 * c + 4);
                    v[u][i][0] = lo.x; v[u][i][1] = lo.y; v[u][i][2] = lo.z; v[u][i][3] = lo.w;
                    v[u][i][4] = hi.x; v[u][i][5] = hi.y; v[u][i][6] = hi.z; v[u][i][7] = hi.w;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int r = r0 + u * (kGemmThreads / 32);
            if (r >= m_here) continue;
#pragma unroll
            for (int i = 0; i < kNormMaxPerLane; ++i)
                if (lane + 32 * i < chunks)
#pragma unroll
                    for (int e = 0; e < 8; ++e) sum[u] += v[u][i][e];
            float mean = 0.0f, inv = 1.0f;
            if (a.gamma) {
                mean = warp_sum(sum[u]) / static_cast<float>(a.k);
                float sq = 0.0f;
#pragma unroll
                for (int i = 0; i < kNormMaxPerLane; ++i)
                    if (lane + 32 * i < chunks)
#pragma unroll
                        for (int e = 0; e < 8; ++e) { float d = v[u][i][e] - mean; sq = fmaf(d, d, sq); }
                inv = rsqrtf(warp_sum(sq) / static_cast<float>(a.k) + a.eps);
            }
#pragma unroll
            for (int i = 0; i < kNormMaxPerLane; ++i) {
                const int c = lane + 32 * i;
                if (c >= chunks) continue;
                uint32_t packed[4];
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    float y0 = (v[u][i][e] - mean) * inv, y1 = (v[u][i][e + 1] - mean) * inv;
                    if (a.gamma) {
                        y0 = fmaf(y0, a.gamma[8 * c + e], a.beta[8 * c + e]);
                        y1 = fmaf(y1, a.gamma[8 * c + e + 1], a.beta[8 * c + e + 1]);
                    }
                    if (a.w_dtype == RLM_BF16) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
                        packed[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                    } else {
                        __half2 h = __floats2half2_rn(y0, y1);
                        packed[e / 2] = *reinterpret_cast<uint32_t*>(&h);
                    }
                }
                // K-major, 128-byte swizzle: 16-byte chunk index xor (row mod 8)
                const int kb = c >> 3, c16 = c & 7;
                unsigned char* dst = a_tile + kb * a.a_stride + (r >> 3) * 1024 + (r & 7) * 128 +
                                     ((c16 ^ (r & 7)) << 4);
                *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
        }
    }
    fence_proxy_async();     // generic-proxy writes of the x tile -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (tid == 0) {
        for (int it = kStages; it < k_iters; ++it) {
            const int s = it % kStages;
            if (!mbar_wait(empty(s), ((it / kStages) - 1) & 1)) { failed = 1; break; }
            mbar_expect_tx(full(s), kBBytes);
            tma_load_2d(ring_addr + s * kBBytes, &map_w, it * kBK, n0, full(s));
        }
    } else if (tid == 32) {
        bool ok = true;
        for (int it = 0; it < k_iters && ok; ++it) {
            const int s = it % kStages;
            ok = mbar_wait(full(s), (it / kStages) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = smem_desc_sw128(a_addr + it * a.a_stride);
            const uint64_t db = smem_desc_sw128(ring_addr + s * kBBytes);
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk)
                umma_f16(tmem_base, da + 2 * kk, db + 2 * kk, a.idesc, (it > 0 || kk > 0) ? 1u : 0u);
            umma_commit(empty(s));
        }
        if (!ok) failed = 1;
        umma_commit(acc_full);
    }
    __syncwarp();

    bool ready = mbar_wait(acc_full, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ready = ready && (*reinterpret_cast<volatile int*>(&failed) == 0);
    if (!__syncthreads_or(!ready)) {
        const int row = warp * 32 + lane;
        if (warp * 32 < m_here) {   // warps whose 32 rows do not exist skip the read-back
#pragma unroll
            for (int c = 0; c < BN; c += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < m_here) {
                    const size_t at = static_cast<size_t>(m0 + row) * a.n + n0 + c;
                    if (a.out_dtype == RLM_F32) {
                        float4* o = reinterpret_cast<float4*>(static_cast<float*>(a.out) + at);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            o[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                               __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                    } else {
                        uint32_t packed[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float lo = __uint_as_float(v[2 * i]), hi = __uint_as_float(v[2 * i + 1]);
                            if (a.out_dtype == RLM_BF16) {
                                __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                                packed[i] = *reinterpret_cast<uint32_t*>(&h);
                            } else {
                                __half2 h = __floats2half2_rn(lo, hi);
                                packed[i] = *reinterpret_cast<uint32_t*>(&h);
                            }
                        }
                        uint4* o = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + at);
                        o[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        o[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    }
                }
            }
        }
    } else if (tid == 0 && a.status) {
        atomicOr(a.status, RLM_DEV_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// ------------------------------------------------------------------ LayerNorm -> 16-bit rows
//
// For batches beyond one row tile the normalisation is done once (one warp per row) into a
// 16-bit matrix that packed_projection_kernel then streams with TMA, instead of once per
// output-column tile.  Arithmetic identical to the fused kernel above.
constexpr int kCastThreads = 256;

struct NormCastArgs {
    const float* x;
    const float* gamma;
    const float* beta;
    void* out;
    int64_t x_stride;
    float eps;
    int m, k, out_dtype;
};

__global__ void __launch_bounds__(kCastThreads) layer_norm_cast_kernel(const NormCastArgs a) {
    griddep_sync();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (kCastThreads / 32) + (threadIdx.x >> 5);
    if (r >= a.m) return;
    const int chunks = a.k / 8;
    const float* row = a.x + r * a.x_stride;
    float v[kNormMaxPerLane][8];
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
            const float4 lo = *reinterpret_cast<const float4*>(row + 8 * c);
            const float4 hi = *reinterpret_cast<const float4*>(row + 8 * c + 4);
            v[i][0] = lo.x; v[i][1] = lo.y; v[i][2] = lo.z; v[i][3] = lo.w;
            v[i][4] = hi.x; v[i][5] = hi.y; v[i][6] = hi.z; v[i][7] = hi.w;
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += v[i][e];
        }
    }
    float mean = 0.0f, inv = 1.0f;
    if (a.gamma) {
        mean = warp_sum(sum) / static_cast<float>(a.k);
        float sq = 0.0f;
#pragma unroll
        for (int i = 0; i < kNormMaxPerLane; ++i)
            if (lane + 32 * i < chunks)
#pragma unroll
                for (int e = 0; e < 8; ++e) { float d = v[i][e] - mean; sq = fmaf(d, d, sq); }
        inv = rsqrtf(warp_sum(sq) / static_cast<float>(a.k) + a.eps);
    }
#pragma unroll
    for (int i = 0; i < kNormMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c >= chunks) continue;
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            float y0 = (v[i][e] - mean) * inv, y1 = (v[i][e + 1] - mean) * inv;
            if (a.gamma) {
                y0 = fmaf(y0, a.gamma[8 * c + e], a.beta[8 * c + e]);
                y1 = fmaf(y1, a.gamma[8 * c + e + 1], a.beta[8 * c + e + 1]);
            }
            if (a.out_dtype == RLM_BF16) {
                __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
                packed[e / 2] = *reinterpret_cast<uint32_t*>(&h);
            } else {
                __half2 h = __floats2half2_rn(y0, y1);
                packed[e / 2] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
        *reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + static_cast<size_t>(r) * a.k + 8 * c) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

template <int BN>
int launch_gemm(const CUtensorMap& mx, const CUtensorMap& mw, const GemmArgs& a, void* stream) {
    const int smem_bytes = stages_for(BN) * (kBM * kBK * 2 + BN * kBK * 2) + 1024;
    auto kernel = packed_projection_kernel<BN>;
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    dim3 grid(a.n / BN, (a.m + kBM - 1) / kBM, a.k_splits);
    launch_kernel(kernel, dim3(grid), dim3(kGemmThreads), smem_bytes, stream, mx, mw, a);
    count_launch();
    return check_launch("packed_projection_kernel");
}

template <int BN>
int launch_norm_gemm(const CUtensorMap& mw, const NormGemmArgs& a, void* stream) {
    const int smem_bytes = static_cast<int>(a.a_bytes) + 8 * BN * kBK * 2 + 1024;
    if (smem_bytes > kSmemDynamicLimit) {
        set_error("norm_projection: rows x d_in too large for the shared-memory x tile");
        return RLM_ERR_SMEM;
    }
    auto kernel = norm_projection_kernel<BN>;
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    dim3 grid(a.n / BN, (a.m + a.tile_rows - 1) / a.tile_rows);
    launch_kernel(kernel, dim3(grid), dim3(kGemmThreads), smem_bytes, stream, mw, a);
    count_launch();
    return check_launch("norm_projection_kernel");
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_norm_projection(const float* x, int64_t x_row_stride, const float* gamma,
                                   const float* beta, float eps, const void* weight, void* out,
                                   int rows, int d_in, int n_out, int weight_dtype, int out_dtype,
                                   int32_t* status, void* stream) {
    using namespace rlm;
    if (rows == 0) return RLM_OK;
    if (!x || !weight || !out || ((gamma == nullptr) != (beta == nullptr))) {
        set_error("norm_projection: NULL pointer (gamma and beta go together)");
        return RLM_ERR_NULL;
    }
    if (rows < 0 || d_in < 64 || d_in % 64 != 0 || d_in > 256 * kNormMaxPerLane ||
        n_out < 32 || n_out % 32 != 0 || x_row_stride < d_in || x_row_stride % 4 != 0) {
        set_error("norm_projection: need d_in a multiple of 64 up to 1024 and n_out a multiple of 32");
        return RLM_ERR_SHAPE;
    }
    if ((weight_dtype != RLM_BF16 && weight_dtype != RLM_F16) || !valid_dtype(out_dtype)) {
        set_error("norm_projection: weights must be bfloat16 or float16");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || (gamma && (!aligned16(gamma) || !aligned16(beta)))) {
        set_error("norm_projection: tensors must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    const int m_tiles = (rows + kBM - 1) / kBM, tile_rows = rows < kBM ? rows : kBM;
    int bn = 128;
    if (n_out % 128 != 0 || n_out / 128 * m_tiles < 100) bn = 64;
    if (n_out % 64 != 0 || (n_out / 64 * m_tiles < 100 && bn == 64)) bn = 32;
    CUtensorMap mw;
    if (!make_map(&mw, weight, n_out, d_in, d_in, bn, weight_dtype)) {
        set_error("norm_projection: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    NormGemmArgs a{};
    a.x = x; a.gamma = gamma; a.beta = beta; a.out = out; a.status = status; a.x_stride = x_row_stride;
    a.eps = eps; a.m = rows; a.n = n_out; a.k = d_in; a.w_dtype = weight_dtype; a.out_dtype = out_dtype;
    const uint32_t fmt = weight_dtype == RLM_BF16 ? 1u : 0u;
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(bn >> 3) << 17) |
              (static_cast<uint32_t>(kBM >> 4) << 24);
    // rows per CTA: as many as the shared memory left by the weight ring holds
    a.tile_rows = ((tile_rows + 7) / 8) * 8;
    for (;;) {
        a.a_stride = static_cast<uint32_t>(a.tile_rows / 8) * 1024u;
        a.a_bytes = (static_cast<uint32_t>(d_in / kBK) - 1u) * a.a_stride + kBM * kBK * 2;
        if (static_cast<int>(a.a_bytes) + 8 * bn * kBK * 2 + 1024 <= kSmemDynamicLimit || a.tile_rows <= 8)
            break;
        a.tile_rows -= 8;
    }
    if (bn == 32) return launch_norm_gemm<32>(mw, a, stream);
    if (bn == 64) return launch_norm_gemm<64>(mw, a, stream);
    return launch_norm_gemm<128>(mw, a, stream);
}

extern "C" int rlm_layer_norm_cast(const float* x, int64_t x_row_stride, const float* gamma,
                                   const float* beta, float eps, void* out, int rows, int d_in,
                                   int out_dtype, void* stream) {
    using namespace rlm;
    if (rows == 0) return RLM_OK;
    if (!x || !out || ((gamma == nullptr) != (beta == nullptr))) {
        set_error("layer_norm_cast: NULL pointer (gamma and beta go together)");
        return RLM_ERR_NULL;
    }
    if (rows < 0 || d_in < 8 || d_in % 8 != 0 || d_in > 256 * kNormMaxPerLane || x_row_stride < d_in ||
        x_row_stride % 4 != 0) {
        set_error("layer_norm_cast: need d_in a multiple of 8 up to 1024");
        return RLM_ERR_SHAPE;
    }
    if (out_dtype != RLM_BF16 && out_dtype != RLM_F16) {
        set_error("layer_norm_cast: the output must be bfloat16 or float16");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(x) || !aligned16(out) || (gamma && (!aligned16(gamma) || !aligned16(beta)))) {
        set_error("layer_norm_cast: tensors must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    NormCastArgs a{};
    a.x = x; a.gamma = gamma; a.beta = beta; a.out = out; a.x_stride = x_row_stride; a.eps = eps;
    a.m = rows; a.k = d_in; a.out_dtype = out_dtype;
    const int per_cta = kCastThreads / 32;
    launch_kernel(layer_norm_cast_kernel, dim3((rows + per_cta - 1) / per_cta), dim3(kCastThreads), 0, stream, a);
    count_launch();
    return check_launch("layer_norm_cast_kernel");
}

extern "C" int rlm_packed_projection(const void* x, int64_t x_row_stride, const void* weight,
                                     const float* bias, void* out, int rows, int d_in, int n_out,
                                     int in_dtype, int out_dtype, int k_splits, int32_t* status,
                                     void* stream) {
    using namespace rlm;
    if (rows == 0) return RLM_OK;
    if (!x || !weight || !out) { set_error("packed_projection: NULL pointer"); return RLM_ERR_NULL; }
    if (rows < 0 || d_in < 8 || d_in % 8 != 0 || n_out < 32 || n_out % 32 != 0 || x_row_stride < d_in ||
        x_row_stride % 8 != 0) {
        set_error("packed_projection: need d_in and the row stride multiples of 8 and n_out a multiple of 32");
        return RLM_ERR_SHAPE;
    }
    if ((in_dtype != RLM_BF16 && in_dtype != RLM_F16) || !valid_dtype(out_dtype)) {
        set_error("packed_projection: operands must be bfloat16 or float16 (fp32 inputs are not a tensor-core format here)");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(x) || !aligned16(weight) || !aligned16(out)) {
        set_error("packed_projection: tensors must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    if (k_splits < 1 || (k_splits > 1 && (out_dtype != RLM_F32 || bias || ((d_in + kBK - 1) / kBK) % k_splits != 0))) {
        set_error("packed_projection: split K needs fp32 output slices, no bias and a split count that divides d_in / 64");
        return RLM_ERR_SHAPE;
    }
    const int m_tiles = (rows + kBM - 1) / kBM;
    if (k_splits == 1 && n_out % kPgBN == 0 && d_in % kBK == 0 && m_tiles * (n_out / kPgBN) >= 2 * sm_count()) {
        // at least two 128 x 256 tiles per SM: persistent CTAs; 256 x 256 tiles when there are two of those per SM
        // (a 256-row tile's epilogue is not hidden behind the next main loop: it pays only with a long reduction)
        const bool tall = d_in >= 1024 && ((rows + 2 * kBM - 1) / (2 * kBM)) * (n_out / kPgBN) >= 2 * sm_count();
        CUtensorMap px, pw;
        if (!make_map(&px, x, rows, d_in, x_row_stride, tall ? 2 * kBM : kBM, in_dtype) ||
            !make_map(&pw, weight, n_out, d_in, d_in, kPgBN, in_dtype)) {
            set_error("packed_projection: cuTensorMapEncodeTiled failed");
            return RLM_ERR_LAUNCH;
        }
        PersistentGemmArgs p{};
        p.out = out; p.bias = bias; p.status = status; p.m = rows; p.n = n_out; p.k = d_in; p.out_dtype = out_dtype;
        const uint32_t pfmt = in_dtype == RLM_BF16 ? 1u : 0u;
        p.idesc = (1u << 4) | (pfmt << 7) | (pfmt << 10) | (static_cast<uint32_t>(kPgBN >> 3) << 17) |
                  (static_cast<uint32_t>(kBM >> 4) << 24);
        return tall ? launch_persistent_gemm<2>(px, pw, p, stream) : launch_persistent_gemm<1>(px, pw, p, stream);
    }
    // Tile width: with few rows the weight read dominates, so pick the widest tile that still
    // gives about one CTA per SM; with many rows use wide tiles.
    int bn = 128;
    if (n_out % 128 != 0 || n_out / 128 * m_tiles * k_splits < 100) bn = 64;
    if (n_out % 64 != 0 || (n_out / 64 * m_tiles * k_splits < 100 && bn == 64)) bn = 32;
    // x tile: the box holds only the rows that exist (a multiple of 8, at most 128); the MMA
    // reads 128 rows of the stage, the rest is never stored
    const int box_rows = rows >= kBM ? kBM : ((rows + 7) / 8) * 8;
    CUtensorMap mx, mw;
    if (!make_map(&mx, x, rows, d_in, x_row_stride, box_rows, in_dtype) ||
        !make_map(&mw, weight, n_out, d_in, d_in, bn, in_dtype)) {
        set_error("packed_projection: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    GemmArgs a{};
    a.out = out; a.bias = bias; a.status = status; a.m = rows; a.n = n_out; a.k = d_in; a.out_dtype = out_dtype;
    a.a_bytes = static_cast<uint32_t>(box_rows) * kBK * 2;
    // a single thread issues one tcgen05.mma per ~60 cycles, more than a 128-wide MMA runs: two warps issue
    const int k_blocks = ((d_in + kBK - 1) / kBK) / k_splits;
    a.k_blocks_per_split = k_blocks;
    a.k_splits = k_splits;
    // (with an even ring depth each issuer owns its own stages, so every stage barrier is consumed in order)
    a.issuers = (k_blocks >= 2 && stages_for(bn) % 2 == 0) ? 2 : 1;
    const uint32_t fmt = in_dtype == RLM_BF16 ? 1u : 0u;
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(bn >> 3) << 17) |
              (static_cast<uint32_t>(kBM >> 4) << 24);
    if (bn == 32) return launch_gemm<32>(mx, mw, a, stream);
    if (bn == 64) return launch_gemm<64>(mx, mw, a, stream);
    return launch_gemm<128>(mx, mw, a, stream);
}

