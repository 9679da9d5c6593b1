// First relation-MLP layer over gathered rows on the 5th-generation tensor cores (sm_100a),
// for launches with many relation rows (decode batches of hundreds of sequences, prefill):
//
//   out[row, k, h] = gelu( product_weight[h, :] . (operand[a] * operand[p_k])
//                          + expanded[a, h] + expanded[p_k, H + h] )
//
// with a = anchor_index[row], p_k = partner_index[row, k], and, in the update form, the
// expanded row of the current position computed here first
// (expanded[t, :H] = anchor_weight . operand[t] + bias, expanded[t, H:] = partner_weight . operand[t]),
// written to the cache and used un-rounded by the rows that selected position t.
//
// One CTA per tile of 128 (row, partner) pairs x 128 hidden columns:
//   * the three 128 x R weight tiles arrive by tiled TMA loads (128-byte swizzle, no multicast);
//   * all threads gather the operand rows, multiply them in fp32 and write the 16-bit products
//     straight into the swizzled K-major layout the tensor core reads (A tile, 128 x R);
//   * one thread issues tcgen05.mma: pairs x weight^T into 128 TMEM columns and, in the update
//     form, weight x current-operands^T (hidden columns on the TMEM lanes, the tile's sequences
//     on 16..32 columns) for the two fresh half rows;
//   * the epilogue reads TMEM with tcgen05.ld; every thread owns one pair row and 64 hidden
//     columns, adds the two gathered expanded-cache terms (requested before the MMA wait),
//     applies GELU and stores.
// Every wait is bounded; on expiry the kernel sets RLM_DEV_TIMEOUT, frees its TMEM and returns.
//
// Semantics follow src/relation_lm/kernels/relation_reduce.py:72-146 and 186-309 of the
// reference project; the products are rounded to the cache dtype before the tensor-core
// contraction (the reference contracts fp32 products), which the 16-bit tolerance covers.

#include "rlm_tcgen05.cuh"

namespace rlm {
namespace {

constexpr int kTcThreads = 256;
constexpr int kTcBN = 128;          // hidden columns per tile
constexpr int kTcMaxFresh = 32;     // sequences per tile in the update form (128 / K, K >= 4)

struct HiddenTcArgs {
    void* expanded_cache;
    const void* operand_cache;
    const int32_t* anchor_index;
    const int32_t* partner_index;
    const void* first_bias;
    const int64_t* position;
    const int32_t* row_batch;
    void* out;
    int32_t* status;
    int n_rows, n_seq, max_t, rdim, hdim, k_out;
    int dtype, out_dtype;
    int rows_per_tile;      // 128 / K
    int n_fresh;            // rows_per_tile rounded up to 16 (update form)
    int tmem_cols;
    uint32_t idesc_main, idesc_fresh;
};

__device__ __forceinline__ float gelu_erf_tc(float x) {
    return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
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

template <bool kUpdate>
__global__ void __launch_bounds__(kTcThreads) relation_hidden_tc_kernel(
    const __grid_constant__ CUtensorMap map_wm, const __grid_constant__ CUtensorMap map_wa,
    const __grid_constant__ CUtensorMap map_wp, const HiddenTcArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    __shared__ int idx_s[2 * kBM];      // [rows_per_tile][K + 1]
    __shared__ int seq_s[kBM];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int R = a.rdim, H = a.hdim, K = a.k_out, RPT = a.rows_per_tile;
    const int kblocks = R / kBK, chunks = R / 8;
    const int h0 = blockIdx.x * kTcBN, row0 = blockIdx.y * RPT;
    const int tile_pairs = RPT * K;

    int t = -1;
    if (kUpdate) {
        t = static_cast<int>(*a.position);
        if (t < 0 || t >= a.max_t) {
            if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
            return;
        }
    }

    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t tile_bytes = static_cast<uint32_t>(kblocks) * kBM * 128u;   // one 128 x R tile
    unsigned char* a_tile = base;
    unsigned char* wm_tile = a_tile + tile_bytes;
    unsigned char* wa_tile = wm_tile + tile_bytes;                              // kUpdate only
    unsigned char* wp_tile = wa_tile + (kUpdate ? tile_bytes : 0u);
    unsigned char* cur_tile = wp_tile + (kUpdate ? tile_bytes : 0u);            // [kblocks][n_fresh][128 B]
    const uint32_t cur_kblock = static_cast<uint32_t>(a.n_fresh) * 128u;
    float* fresh_s = reinterpret_cast<float*>(cur_tile + (kUpdate ? kblocks * cur_kblock : 0u));  // [2][RPT][128]

    const uint32_t bar_w = smem_u32(&bars[0]), bar_acc = smem_u32(&bars[1]);
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_wm) : "memory");
        if (kUpdate) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_wa) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_wp) : "memory");
        }
        mbar_init(bar_w, 1);
        mbar_init(bar_acc, 1);
        fence_barrier_init();
        failed = 0;
        mbar_expect_tx(bar_w, (kUpdate ? 3u : 1u) * tile_bytes);
        for (int kb = 0; kb < kblocks; ++kb) {
            tma_load_2d(smem_u32(wm_tile) + kb * kBM * 128u, &map_wm, kb * kBK, h0, bar_w);
            if (kUpdate) {
                tma_load_2d(smem_u32(wa_tile) + kb * kBM * 128u, &map_wa, kb * kBK, h0, bar_w);
                tma_load_2d(smem_u32(wp_tile) + kb * kBM * 128u, &map_wp, kb * kBK, h0, bar_w);
            }
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // gathered indices of the tile's sequences
    for (int i = tid; i < RPT * (K + 1); i += kTcThreads) {
        const int rb = i / (K + 1), j = i - rb * (K + 1), row = row0 + rb;
        int v = 0;
        if (row < a.n_rows)
            v = j == 0 ? a.anchor_index[row] : a.partner_index[static_cast<size_t>(row) * K + j - 1];
        idx_s[i] = min(max(v, 0), a.max_t - 1);
        if (j == 0) {
            int b = row < a.n_rows ? (a.row_batch ? a.row_batch[row] : row) : -1;
            if (row < a.n_rows && (b < 0 || b >= a.n_seq)) {
                if (a.status) atomicOr(a.status, RLM_DEV_POSITION);
                b = -1;
            }
            seq_s[rb] = b;
        }
    }
    __syncthreads();

    // A tile: products of the gathered operand rows, four 16-byte chunks per thread in flight
    const size_t op_row = static_cast<size_t>(R) * 2;
    const int items = kBM * chunks;
    for (int i0 = tid; i0 < items; i0 += 4 * kTcThreads) {
        uint4 ra[4], rp[4];
        bool live[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * kTcThreads;
            const int r = i / chunks, c = i - r * chunks;
            const int rb = r / K, k = r - rb * K;
            live[u] = i < items && r < tile_pairs && seq_s[rb < RPT ? rb : 0] >= 0;
            if (live[u]) {
                const char* operand = static_cast<const char*>(a.operand_cache) +
                                      static_cast<size_t>(seq_s[rb]) * a.max_t * op_row;
                ra[u] = *reinterpret_cast<const uint4*>(operand + idx_s[rb * (K + 1)] * op_row + 16 * c);
                rp[u] = *reinterpret_cast<const uint4*>(operand + idx_s[rb * (K + 1) + k + 1] * op_row + 16 * c);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * kTcThreads;
            if (i >= items) continue;
            const int r = i / chunks, c = i - r * chunks;
            uint4 packed = make_uint4(0, 0, 0, 0);
            if (live[u]) {
                float fa[8], fp[8];
                unpack8(ra[u], a.dtype, fa);
                unpack8(rp[u], a.dtype, fp);
                packed.x = pack2(fp[0] * fa[0], fp[1] * fa[1], a.dtype);
                packed.y = pack2(fp[2] * fa[2], fp[3] * fa[3], a.dtype);
                packed.z = pack2(fp[4] * fa[4], fp[5] * fa[5], a.dtype);
                packed.w = pack2(fp[6] * fa[6], fp[7] * fa[7], a.dtype);
            }
            *reinterpret_cast<uint4*>(a_tile + swizzled(r, c, kBM * 128u)) = packed;
        }
    }
    if (kUpdate) {
        // current operand rows of the tile's sequences (zero rows up to n_fresh)
        for (int i = tid; i < a.n_fresh * chunks; i += kTcThreads) {
            const int j = i / chunks, c = i - j * chunks;
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (j < RPT && seq_s[j] >= 0)
                raw = *reinterpret_cast<const uint4*>(
                    static_cast<const char*>(a.operand_cache) +
                    (static_cast<size_t>(seq_s[j]) * a.max_t + t) * op_row + 16 * c);
            *reinterpret_cast<uint4*>(cur_tile + swizzled(j, c, cur_kblock)) = raw;
        }
    }
    fence_proxy_async();     // generic-proxy writes of the tiles -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    const uint32_t tmem_fresh = tmem_base + kTcBN;      // anchor half, then partner half n_fresh further

    if (tid == 0) {
        bool ok = mbar_wait(bar_w, 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = 0; kb < kblocks; ++kb) {
                const uint64_t da = smem_desc_sw128(smem_u32(a_tile) + kb * kBM * 128u);
                const uint64_t db = smem_desc_sw128(smem_u32(wm_tile) + kb * kBM * 128u);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)
                    umma_f16(tmem_base, da + 2 * kk, db + 2 * kk, a.idesc_main, (kb > 0 || kk > 0) ? 1u : 0u);
            }
            if (kUpdate) {
                for (int half = 0; half < 2; ++half)
                    for (int kb = 0; kb < kblocks; ++kb) {
                        const uint64_t dw = smem_desc_sw128(smem_u32(half ? wp_tile : wa_tile) + kb * kBM * 128u);
                        const uint64_t dc = smem_desc_sw128(smem_u32(cur_tile) + kb * cur_kblock);
#pragma unroll
                        for (int kk = 0; kk < kBK / 16; ++kk)
                            umma_f16(tmem_fresh + half * a.n_fresh, dw + 2 * kk, dc + 2 * kk, a.idesc_fresh,
                                     (kb > 0 || kk > 0) ? 1u : 0u);
                    }
            }
        } else {
            failed = 1;
        }
        umma_commit(bar_acc);     // accumulators complete (or abandoned)
    }
    __syncwarp();

    // This thread's epilogue share: pair row `pr`, hidden columns [h0 + 64 ch, h0 + 64 ch + 64).
    // The expanded-cache terms are requested now and consumed after the MMA wait.
    const int pr = 32 * (warp & 3) + lane, ch = warp >> 2;
    const int rb = pr / K, k = pr - rb * K;
    const bool pair_live = pr < tile_pairs && row0 + rb < a.n_rows && seq_s[rb < RPT ? rb : 0] >= 0;
    bool sub_a = false, sub_p = false;
    uint4 ea[8], ep[8];
    if (pair_live) {
        const int ai = idx_s[rb * (K + 1)], pi = idx_s[rb * (K + 1) + k + 1];
        sub_a = kUpdate && ai == t;
        sub_p = kUpdate && pi == t;
        const char* ex = static_cast<const char*>(a.expanded_cache) +
                         static_cast<size_t>(seq_s[rb]) * a.max_t * 2 * H * 2;
        const uint4* pa = reinterpret_cast<const uint4*>(ex + (static_cast<size_t>(ai) * 2 * H + h0 + 64 * ch) * 2);
        const uint4* pp = reinterpret_cast<const uint4*>(ex + (static_cast<size_t>(pi) * 2 * H + H + h0 + 64 * ch) * 2);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            ea[i] = sub_a ? make_uint4(0, 0, 0, 0) : pa[i];
            ep[i] = sub_p ? make_uint4(0, 0, 0, 0) : pp[i];
        }
    }

    bool ready = mbar_wait(bar_acc, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ready = ready && (*reinterpret_cast<volatile int*>(&failed) == 0);
    if (!__syncthreads_or(!ready)) {
        const uint32_t lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        if (kUpdate) {
            // fresh half rows: this thread owns hidden column h0 + hc of half `ch`
            const int hc = 32 * (warp & 3) + lane;
            const float bias = ch == 0 ? load_scalar(a.first_bias, h0 + hc, a.dtype) : 0.0f;
            for (int c = 0; c < a.n_fresh; c += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_fresh + ch * a.n_fresh + lane_base + c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int s = c + j;
                    if (s >= RPT || seq_s[s] < 0) continue;
                    const float val = __uint_as_float(v[j]) + bias;
                    fresh_s[(ch * RPT + s) * kTcBN + hc] = val;
                    store_scalar(a.expanded_cache,
                                 (static_cast<int64_t>(seq_s[s]) * a.max_t + t) * 2 * H + ch * H + h0 + hc,
                                 a.dtype, val);
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t v[16];
            tmem_ld16(tmem_base + lane_base + 64 * ch + 16 * q, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (!pair_live) continue;
            float fa[16], fp[16];
            {
                float lo[8], hi[8];
                unpack8(ea[2 * q], a.dtype, lo);
                unpack8(ea[2 * q + 1], a.dtype, hi);
#pragma unroll
                for (int i = 0; i < 8; ++i) { fa[i] = lo[i]; fa[8 + i] = hi[i]; }
                unpack8(ep[2 * q], a.dtype, lo);
                unpack8(ep[2 * q + 1], a.dtype, hi);
#pragma unroll
                for (int i = 0; i < 8; ++i) { fp[i] = lo[i]; fp[8 + i] = hi[i]; }
            }
            if (kUpdate && (sub_a || sub_p)) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (sub_a) fa[i] = fresh_s[(0 * RPT + rb) * kTcBN + 64 * ch + 16 * q + i];
                    if (sub_p) fp[i] = fresh_s[(1 * RPT + rb) * kTcBN + 64 * ch + 16 * q + i];
                }
            }
            float y[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) y[i] = gelu_erf_tc(__uint_as_float(v[i]) + (fa[i] + fp[i]));
            const size_t at = (static_cast<size_t>(row0) * K + pr) * H + h0 + 64 * ch + 16 * q;
            if (a.out_dtype == RLM_F32) {
                float4* o = reinterpret_cast<float4*>(static_cast<float*>(a.out) + at);
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
            } else {
                uint4* o = reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) + at);
                o[0] = make_uint4(pack2(y[0], y[1], a.out_dtype), pack2(y[2], y[3], a.out_dtype),
                                  pack2(y[4], y[5], a.out_dtype), pack2(y[6], y[7], a.out_dtype));
                o[1] = make_uint4(pack2(y[8], y[9], a.out_dtype), pack2(y[10], y[11], a.out_dtype),
                                  pack2(y[12], y[13], a.out_dtype), pack2(y[14], y[15], a.out_dtype));
            }
        }
    } else if (tid == 0 && a.status) {
        atomicOr(a.status, RLM_DEV_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
}

}  // namespace

// Whether the tensor-core form applies; the callers fall back to the CUDA-core kernel otherwise.
bool hidden_tc_applicable(bool update, int n_rows, int rdim, int hdim, int k_out, int cache_dtype,
                          int weight_dtype, const void* expanded_cache, const void* out, int out_dtype) {
    if (cache_dtype != weight_dtype || (cache_dtype != RLM_BF16 && cache_dtype != RLM_F16)) return false;
    if (rdim % kBK != 0 || hdim % kTcBN != 0 || k_out < 1 || k_out > 16) return false;
    if (static_cast<long long>(n_rows) * k_out < 256) return false;    // small launches: latency-bound form
    if (update && kBM / k_out > kTcMaxFresh) return false;
    if (!aligned16(expanded_cache) || !aligned16(out)) return false;
    (void)out_dtype;
    const int kblocks = rdim / kBK;
    const int rpt = kBM / k_out, n_fresh = (rpt + 15) & ~15;
    size_t bytes = 1024 + static_cast<size_t>(update ? 4 : 2) * kblocks * kBM * 128;
    if (update) bytes += static_cast<size_t>(kblocks) * n_fresh * 128 + static_cast<size_t>(2) * rpt * kTcBN * 4;
    return bytes <= static_cast<size_t>(kSmemDynamicLimit);
}

int launch_hidden_tc(bool update, void* expanded_cache, const void* operand_cache,
                     const int32_t* anchor_index, const int32_t* partner_index,
                     const void* anchor_weight, const void* partner_weight, const void* product_weight,
                     const void* first_bias, const int64_t* position, const int32_t* row_batch, void* out,
                     int n_rows, int n_seq, int max_t, int rdim, int hdim, int k_out, int dtype,
                     int out_dtype, int32_t* status, void* stream) {
    HiddenTcArgs a{};
    a.expanded_cache = expanded_cache; a.operand_cache = operand_cache; a.anchor_index = anchor_index;
    a.partner_index = partner_index; a.first_bias = first_bias; a.position = position;
    a.row_batch = row_batch; a.out = out; a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.rdim = rdim; a.hdim = hdim; a.k_out = k_out;
    a.dtype = dtype; a.out_dtype = out_dtype;
    a.rows_per_tile = kBM / k_out;
    a.n_fresh = update ? (a.rows_per_tile + 15) & ~15 : 0;
    int cols = kTcBN + 2 * a.n_fresh;
    a.tmem_cols = 32;
    while (a.tmem_cols < cols) a.tmem_cols *= 2;
    const uint32_t fmt = dtype == RLM_BF16 ? 1u : 0u;
    a.idesc_main = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kTcBN >> 3) << 17) |
                   (static_cast<uint32_t>(kBM >> 4) << 24);
    a.idesc_fresh = (1u << 4) | (fmt << 7) | (fmt << 10) |
                    (static_cast<uint32_t>((update ? a.n_fresh : 16) >> 3) << 17) |
                    (static_cast<uint32_t>(kBM >> 4) << 24);
    CUtensorMap mm, ma, mp;
    if (!make_map(&mm, product_weight, hdim, rdim, rdim, kTcBN, dtype) ||
        !make_map(&ma, update ? anchor_weight : product_weight, hdim, rdim, rdim, kTcBN, dtype) ||
        !make_map(&mp, update ? partner_weight : product_weight, hdim, rdim, rdim, kTcBN, dtype)) {
        set_error("relation_hidden: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    const int kblocks = rdim / kBK;
    size_t bytes = 1024 + static_cast<size_t>(update ? 4 : 2) * kblocks * kBM * 128;
    if (update)
        bytes += static_cast<size_t>(kblocks) * a.n_fresh * 128 + static_cast<size_t>(2) * a.rows_per_tile * kTcBN * 4;
    dim3 grid(hdim / kTcBN, (n_rows + a.rows_per_tile - 1) / a.rows_per_tile);
    int rc;
    if (update) {
        auto kernel = relation_hidden_tc_kernel<true>;
        rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
        if (rc != RLM_OK) return rc;
        kernel<<<grid, kTcThreads, bytes, static_cast<cudaStream_t>(stream)>>>(mm, ma, mp, a);
    } else {
        auto kernel = relation_hidden_tc_kernel<false>;
        rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
        if (rc != RLM_OK) return rc;
        kernel<<<grid, kTcThreads, bytes, static_cast<cudaStream_t>(stream)>>>(mm, ma, mp, a);
    }
    count_launch();
    return check_launch("relation_hidden_tc_kernel");
}

}  // namespace rlm
