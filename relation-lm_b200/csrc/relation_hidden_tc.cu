// First relation-MLP layer over gathered rows on the 5th-generation tensor cores (sm_100a),
// for launches with many relation rows (decode batches of hundreds of sequences, prefill):
//
//   out[row, k, h] = gelu( product_weight[h, :] . (operand[a] * operand[p_k])
//                          + expanded[a, h] + expanded[p_k, H + h] )
//
// with a = anchor_index[row], p_k = partner_index[row, k].  The update form first writes the
// expanded row of the current position,
//   expanded[t, :H] = anchor_weight . operand[t] + bias,  expanded[t, H:] = partner_weight . operand[t],
// with a kernel of its own (expanded_row_update_kernel) and then runs the gather kernel, which
// therefore reads position t like any other row (rounded to the cache dtype).
//
// relation_hidden_tc_kernel, one CTA per tile of 128 (row, partner) pairs x 128 hidden columns:
//   * the 128 x R product-weight tile arrives by tiled TMA loads (128-byte swizzle, no multicast);
//   * all threads copy the partner operand rows asynchronously (cp.async) straight into the
//     swizzled K-major layout the tensor core reads (A tile, 128 x R) and multiply them there,
//     in fp32, with the anchor operand chunks they hold in registers;
//   * one thread issues tcgen05.mma (pairs x weight^T into 128 TMEM columns);
//   * once the MMA has consumed the tiles, all threads gather the two expanded-cache terms of
//     every pair into the same shared memory as 16-byte asynchronous copies (cp.async), two
//     256-byte tile rows per warp instruction;
//   * the epilogue reads TMEM with tcgen05.ld; every thread owns one pair row and 64 hidden
//     columns, adds the staged terms, applies GELU and writes 16-bit results over the staged
//     partner term; the rows then leave with coalesced 16-byte stores (fp32 results are stored
//     directly).
//     Three CTAs share an SM so that one tile's gathers overlap another's arithmetic.
// expanded_row_update_kernel, one CTA per 128 hidden columns of one half and up to 64 sequences:
//   weight tile (TMA) x current-operand rows^T, hidden columns on the TMEM lanes and sequences on
//   the TMEM columns, so that a warp's stores of one sequence are contiguous in the cache row.
// Every wait is bounded; on expiry a kernel sets RLM_DEV_TIMEOUT, frees its TMEM and returns.
//
// Semantics follow src/relation_lm/kernels/relation_reduce.py:72-146 and 186-309 of the
// reference project; the products are rounded to the cache dtype before the tensor-core
// contraction and GELU uses a 1.5e-7 polynomial erfc on the hardware reciprocal and exponential
// (the reference contracts fp32 products and calls erf), which the 16-bit tolerance of this path covers.

#include "rlm_tcgen05.cuh"

namespace rlm {
namespace {

constexpr int kTcThreads = 256;
constexpr int kTcBN = 128;          // hidden columns per tile
constexpr int kUpdThreads = 128;
constexpr int kUpdMaxSeq = 64;      // sequences per CTA of the update kernel

struct HiddenTcArgs {
    const void* expanded_cache;
    const void* operand_cache;
    const int32_t* anchor_index;
    const int32_t* partner_index;
    const int32_t* row_batch;
    void* out;
    int32_t* status;
    int n_rows, n_seq, max_t, rdim, hdim, k_out;
    int dtype, out_dtype;
    int rows_per_tile;      // 128 / K
    int inv_k16;            // ceil(65536 / K): r / K == (r * inv_k16) >> 16 for r < 256
    uint32_t idesc;
};

struct RowUpdateArgs {
    void* expanded_cache;           // [layers, n_seq, max_t, 2H]
    const void* operand_cache;      // [layers, n_seq, max_t, R]
    // alternative source of the current operand rows: the packed projection rows of this position
    // ([n_seq, packed_stride], layer l's operand at column l * packed_layer + packed_offset), which an
    // EARLIER launch than the immediate predecessor wrote: the kernel then works before its dependency wait
    const void* packed;
    int64_t packed_stride;
    int packed_layer, packed_offset;
    const void* first_bias;         // [layers, H]
    const int64_t* position;
    int32_t* status;
    int n_seq, max_t, rdim, hdim, dtype;
    int seq_groups;                 // grid.z = layers * seq_groups
};

// ------------------------------------------------------------------ gather + product GEMM + GELU

constexpr uint32_t kRowBytes = kTcBN * 2;            // one tile row of a 16-bit matrix
constexpr uint32_t kRowStride = kRowBytes + 16;      // padded: conflict-free 16-byte row accesses

// Shared-memory plan of the gather kernel (bytes past the 1024-aligned base): the A and weight
// tiles first; once the MMA has consumed them the same bytes hold the gathered expanded-cache
// rows (anchor terms, then partner terms), which the epilogue overwrites with its results.
struct GatherPlan { uint32_t partner_rows, total; };

__host__ __device__ inline GatherPlan gather_plan(int rdim, int rows_per_tile) {
    GatherPlan p;
    const uint32_t tile_bytes = static_cast<uint32_t>(rdim / kBK) * kBM * 128u;
    p.partner_rows = static_cast<uint32_t>(rows_per_tile) * kRowStride;
    const uint32_t staged = p.partner_rows + kBM * kRowStride;
    p.total = 2 * tile_bytes > staged ? 2 * tile_bytes : staged;
    return p;
}

// kDt: dtype of the caches and weights, kOut: dtype of the output (compile-time, so that the
// conversions carry no branches).
template <int kDt, int kOut>
__global__ void __launch_bounds__(kTcThreads, 3) relation_hidden_tc_kernel(
    const __grid_constant__ CUtensorMap map_wm, const HiddenTcArgs a) {
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

    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const GatherPlan plan = gather_plan(R, RPT);
    const uint32_t tile_bytes = static_cast<uint32_t>(kblocks) * kBM * 128u;   // one 128 x R tile
    unsigned char* a_tile = base;
    unsigned char* wm_tile = a_tile + tile_bytes;
    unsigned char* g_anchor = base;                        // after the MMA: [RPT][kRowStride] expanded[a, h0 ..]
    unsigned char* g_partner = base + plan.partner_rows;   // [128][kRowStride] expanded[p, H + h0 ..], then results

    const uint32_t bar_w = smem_u32(&bars[0]), bar_acc = smem_u32(&bars[1]);
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_wm) : "memory");
        mbar_init(bar_w, 1);
        mbar_init(bar_acc, 1);
        fence_barrier_init();
        failed = 0;
        mbar_expect_tx(bar_w, tile_bytes);
        for (int kb = 0; kb < kblocks; ++kb)
            tma_load_2d(smem_u32(wm_tile) + kb * kBM * 128u, &map_wm, kb * kBK, h0, bar_w);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(kTcBN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    griddep_sync();      // weight tile requested, tensor memory allocated: now the previous kernel's outputs
    // gathered indices of the tile's sequences
#pragma unroll 1
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
    __syncthreads();      // also publishes the barrier initialisation

    // A tile: the partner operand rows go straight to their swizzled places in the A tile as
    // 16-byte asynchronous copies while the anchor chunks they are multiplied with wait in
    // registers; once this thread's copies have landed it multiplies them in place (fp32).
    // A thread keeps one chunk column and walks the pair rows, eight rows per round.
    const size_t op_row = static_cast<size_t>(R) * 2;
    {
        constexpr int kRound = 8;
        const int rows_per_pass = kTcThreads / chunks;
        const int bc = tid % chunks, r_first = tid / chunks;
        for (int r0 = r_first < rows_per_pass ? r_first : kBM; r0 < kBM; r0 += kRound * rows_per_pass) {
            uint4 anchor_chunk[kRound];
#pragma unroll
            for (int u = 0; u < kRound; ++u) {
                const int r = r0 + u * rows_per_pass;
                anchor_chunk[u] = make_uint4(0, 0, 0, 0);
                if (r >= kBM) continue;
                const int rb = (r * a.inv_k16) >> 16, k = r - rb * K;
                const uint32_t dst = smem_u32(a_tile) + swizzled(r, bc, kBM * 128u);
                if (r < tile_pairs && seq_s[rb < RPT ? rb : 0] >= 0) {
                    const char* operand = static_cast<const char*>(a.operand_cache) +
                                          static_cast<size_t>(seq_s[rb]) * a.max_t * op_row + 16 * bc;
                    cp_async16(dst, operand + idx_s[rb * (K + 1) + k + 1] * op_row);
                    anchor_chunk[u] = *reinterpret_cast<const uint4*>(operand + idx_s[rb * (K + 1)] * op_row);
                } else {
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
                }
            }
            cp_async_commit();
            cp_async_wait_all();
#pragma unroll
            for (int u = 0; u < kRound; ++u) {
                const int r = r0 + u * rows_per_pass;
                if (r >= kBM) continue;
                uint4* cell = reinterpret_cast<uint4*>(a_tile + swizzled(r, bc, kBM * 128u));
                float fa[8], fp[8];
                unpack8(anchor_chunk[u], kDt, fa);
                unpack8(*cell, kDt, fp);
                *cell = make_uint4(pack2(fp[0] * fa[0], fp[1] * fa[1], kDt), pack2(fp[2] * fa[2], fp[3] * fa[3], kDt),
                                   pack2(fp[4] * fa[4], fp[5] * fa[5], kDt), pack2(fp[6] * fa[6], fp[7] * fa[7], kDt));
            }
        }
    }
    fence_proxy_async();     // generic-proxy writes of the tile -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (tid == 0) {
        bool ok = mbar_wait(bar_w, 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = 0; kb < kblocks; ++kb) {
                const uint64_t da = smem_desc_sw128(smem_u32(a_tile) + kb * kBM * 128u);
                const uint64_t db = smem_desc_sw128(smem_u32(wm_tile) + kb * kBM * 128u);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)
                    umma_f16(tmem_base, da + 2 * kk, db + 2 * kk, a.idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
        } else {
            failed = 1;
        }
        umma_commit(bar_acc);     // accumulator complete (or abandoned)
    }
    __syncwarp();

    bool ready = mbar_wait(bar_acc, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ready = ready && (*reinterpret_cast<volatile int*>(&failed) == 0);
    const bool staged = kOut != RLM_F32;
    if (!__syncthreads_or(!ready)) {
    // The operand tiles are consumed: all threads request the expanded-cache segments of the
        // epilogue into the same bytes as 16-byte asynchronous copies (a warp covers two 256-byte
        // tile rows per instruction): row j < RPT of the staging area is the anchor term of
        // sequence j, row RPT + r the partner term of pair r.
            {
            const int c = tid & 15, n_rows_staged = RPT + tile_pairs;
#pragma unroll 1
            for (int g = tid >> 4; g < n_rows_staged; g += kTcThreads / 16) {
                const int r = g - RPT;
                const int rb = g < RPT ? g : (r * a.inv_k16) >> 16;
                if (row0 + rb >= a.n_rows || seq_s[rb] < 0) continue;
                const int at = g < RPT ? idx_s[rb * (K + 1)] : idx_s[rb * (K + 1) + (r - rb * K) + 1];
                const char* src = static_cast<const char*>(a.expanded_cache) +
                                  ((static_cast<size_t>(seq_s[rb]) * a.max_t + at) * 2 * H + (g < RPT ? 0 : H) + h0) * 2;
                // the partner rows follow the anchor rows in shared memory
                cp_async16(smem_u32(g_anchor) + g * kRowStride + 16 * c, src + 16 * c);
            }
            cp_async_commit();
        }
        cp_async_wait_all();
        __syncthreads();
        // This thread's share: pair row `pr`, hidden columns [h0 + 64 ch, h0 + 64 ch + 64).
        const int pr = 32 * (warp & 3) + lane, ch = warp >> 2;
        const int prb = (pr * a.inv_k16) >> 16;
        const bool pair_live = pr < tile_pairs && row0 + prb < a.n_rows && seq_s[prb < RPT ? prb : 0] >= 0;
        const uint32_t lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
        const unsigned char* ga = g_anchor + (prb < RPT ? prb : 0) * kRowStride + 128 * ch;
        const unsigned char* gp = g_partner + pr * kRowStride + 128 * ch;
        unsigned char* so = g_partner + pr * kRowStride + 128 * ch;      // results replace the partner term
#pragma unroll 1      // the body is large and runs once per warp: keep the instruction footprint small
        for (int q = 0; q < 4; ++q) {
            uint32_t v[16];
            tmem_ld16(tmem_base + lane_base + 64 * ch + 16 * q, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (!pair_live) continue;
            float y[16];
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                float2 fa[4], fp[4];
                unpack8_pairs(*reinterpret_cast<const uint4*>(ga + 32 * q + 16 * hlf), kDt, fa);
                unpack8_pairs(*reinterpret_cast<const uint4*>(gp + 32 * q + 16 * hlf), kDt, fp);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 acc = make_float2(__uint_as_float(v[8 * hlf + 2 * i]), __uint_as_float(v[8 * hlf + 2 * i + 1]));
                    const float2 g = gelu_tc2(__fadd2_rn(acc, __fadd2_rn(fa[i], fp[i])));
                    y[8 * hlf + 2 * i] = g.x;
                    y[8 * hlf + 2 * i + 1] = g.y;
                }
            }
            if (!staged) {
                const size_t at = (static_cast<size_t>(row0) * K + pr) * H + h0 + 64 * ch + 16 * q;
                float4* o = reinterpret_cast<float4*>(static_cast<float*>(a.out) + at);
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
            } else {
                uint4* o = reinterpret_cast<uint4*>(so + 32 * q);
                o[0] = make_uint4(pack2(y[0], y[1], kOut), pack2(y[2], y[3], kOut),
                                  pack2(y[4], y[5], kOut), pack2(y[6], y[7], kOut));
                o[1] = make_uint4(pack2(y[8], y[9], kOut), pack2(y[10], y[11], kOut),
                                  pack2(y[12], y[13], kOut), pack2(y[14], y[15], kOut));
            }
        }
        if (staged) {
            // 16-bit outputs leave row by row: a warp stores two 256-byte pair rows per instruction
            __syncthreads();
            const int c = tid & 15;
#pragma unroll 2
            for (int r = tid >> 4; r < tile_pairs; r += kTcThreads / 16) {
                const int rb = (r * a.inv_k16) >> 16;
                if (row0 + rb >= a.n_rows || seq_s[rb] < 0) continue;
                *reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.out) +
                                          (static_cast<size_t>(row0) * K + r) * H + h0 + 8 * c) =
                    *reinterpret_cast<const uint4*>(g_partner + r * kRowStride + 16 * c);
            }
        }
    } else if (tid == 0 && a.status) {
        atomicOr(a.status, RLM_DEV_TIMEOUT);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(kTcBN) : "memory");
}

// ------------------------------------------------------------------ many rows: a CTA per pair tile, all hidden tiles
//
// Launches of thousands of rows (whole-sequence passes) repeat the operand gather and the product
// for every one of the H / 128 hidden tiles in the kernel above, and its three CTAs per SM overlap
// only by chance.  Here a CTA of 16 warps keeps one tile of 128 pairs: the product tile is built
// once, then the hidden tiles stream through a two-stage pipeline — weight tile j + 2 (TMA) and
// the expanded-cache terms of tile j + 1 (cp.async) are in flight and the MMA of tile j + 1 runs
// into the second half of the tensor memory while the warps finish tile j (tcgen05.ld, + terms,
// GELU, 16-bit results stored straight from the registers, 64 contiguous bytes per thread).  16-bit
// outputs only.  (Measured slower: 32 warps with 16 columns per thread, 1.13 ms against 0.99 ms; a
// seventeenth warp that only requests weight tiles and issues the MMAs, 0.95 ms against 0.905 ms.)
constexpr int kRowsThreads = 512;

struct RowsPlan { uint32_t a_tile, w_tile[2], terms[2], partner_rows, total; };

__host__ __device__ inline RowsPlan rows_plan(int rdim, int rows_per_tile) {
    RowsPlan p;
    const uint32_t tile_bytes = static_cast<uint32_t>(rdim / kBK) * kBM * 128u;
    p.a_tile = 0;
    p.w_tile[0] = tile_bytes;
    p.w_tile[1] = 2 * tile_bytes;
    p.partner_rows = static_cast<uint32_t>(rows_per_tile) * kRowStride;
    const uint32_t staged = (p.partner_rows + kBM * kRowStride + 127u) & ~127u;
    p.terms[0] = 3 * tile_bytes;
    p.terms[1] = p.terms[0] + staged;
    p.total = p.terms[1] + staged;
    return p;
}

template <int kDt, int kOut>
__global__ void __launch_bounds__(kRowsThreads, 1) relation_hidden_rows_kernel(
    const __grid_constant__ CUtensorMap map_wm, const HiddenTcArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[4];      // weight tile landed [2], accumulator complete [2]
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;
    __shared__ int idx_s[2 * kBM];      // [rows_per_tile][K + 1]
    __shared__ int seq_s[kBM];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int R = a.rdim, H = a.hdim, K = a.k_out, RPT = a.rows_per_tile;
    const int kblocks = R / kBK, chunks = R / 8, n_tiles = H / kTcBN;
    const int row0 = blockIdx.x * RPT;
    const int tile_pairs = RPT * K;

    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const RowsPlan plan = rows_plan(R, RPT);
    const uint32_t tile_bytes = static_cast<uint32_t>(kblocks) * kBM * 128u;
    unsigned char* a_tile = base + plan.a_tile;

    const uint32_t bar_w[2] = {smem_u32(&bars[0]), smem_u32(&bars[1])};
    const uint32_t bar_acc[2] = {smem_u32(&bars[2]), smem_u32(&bars[3])};
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_wm) : "memory");
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bars[i]), 1);
        fence_barrier_init();
        failed = 0;
        for (int j = 0; j < 2 && j < n_tiles; ++j) {
            mbar_expect_tx(bar_w[j], tile_bytes);
            for (int kb = 0; kb < kblocks; ++kb)
                tma_load_2d(smem_u32(base + plan.w_tile[j]) + kb * kBM * 128u, &map_wm, kb * kBK, j * kTcBN, bar_w[j]);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(2 * kTcBN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    griddep_sync();
#pragma unroll 1
    for (int i = tid; i < RPT * (K + 1); i += kRowsThreads) {
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
    __syncthreads();      // also publishes the barrier initialisation

    // product tile, once: partner operand rows copied to their swizzled places, multiplied in
    // place (fp32) with the anchor chunks held in registers
    const size_t op_row = static_cast<size_t>(R) * 2;
    {
        constexpr int kRound = 4;
        const int rows_per_pass = kRowsThreads / chunks;
        const int bc = tid % chunks, r_first = tid / chunks;
        for (int r0 = r_first < rows_per_pass ? r_first : kBM; r0 < kBM; r0 += kRound * rows_per_pass) {
            uint4 anchor_chunk[kRound];
#pragma unroll
            for (int u = 0; u < kRound; ++u) {
                const int r = r0 + u * rows_per_pass;
                anchor_chunk[u] = make_uint4(0, 0, 0, 0);
                if (r >= kBM) continue;
                const int rb = (r * a.inv_k16) >> 16, k = r - rb * K;
                const uint32_t dst = smem_u32(a_tile) + swizzled(r, bc, kBM * 128u);
                if (r < tile_pairs && seq_s[rb < RPT ? rb : 0] >= 0) {
                    const char* operand = static_cast<const char*>(a.operand_cache) +
                                          static_cast<size_t>(seq_s[rb]) * a.max_t * op_row + 16 * bc;
                    cp_async16(dst, operand + idx_s[rb * (K + 1) + k + 1] * op_row);
                    anchor_chunk[u] = *reinterpret_cast<const uint4*>(operand + idx_s[rb * (K + 1)] * op_row);
                } else {
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
                }
            }
            cp_async_commit();
            cp_async_wait_all();
#pragma unroll
            for (int u = 0; u < kRound; ++u) {
                const int r = r0 + u * rows_per_pass;
                if (r >= kBM) continue;
                uint4* cell = reinterpret_cast<uint4*>(a_tile + swizzled(r, bc, kBM * 128u));
                float fa[8], fp[8];
                unpack8(anchor_chunk[u], kDt, fa);
                unpack8(*cell, kDt, fp);
                *cell = make_uint4(pack2(fp[0] * fa[0], fp[1] * fa[1], kDt), pack2(fp[2] * fa[2], fp[3] * fa[3], kDt),
                                   pack2(fp[4] * fa[4], fp[5] * fa[5], kDt), pack2(fp[6] * fa[6], fp[7] * fa[7], kDt));
            }
        }
    }
    // the expanded-cache terms of hidden tile j: row g < RPT of the staging area is the anchor term
    // of sequence g, row RPT + r the partner term of pair r (16 threads copy a 256-byte row).  The
    // rows a thread copies are the same for every hidden tile: their source addresses are worked
    // out once, a tile then costs one copy instruction per row.
    constexpr int kTermRows = 2 * kBM * 16 / kRowsThreads;     // staged rows per thread, at most (RPT + pairs <= 256)
    const char* term_src[kTermRows];
    {
        const int c = tid & 15, n_rows_staged = RPT + tile_pairs;
#pragma unroll
        for (int k = 0; k < kTermRows; ++k) {
            const int g = (tid >> 4) + k * (kRowsThreads / 16);
            term_src[k] = nullptr;
            if (g >= n_rows_staged) continue;
            const int r = g - RPT;
            const int rb = g < RPT ? g : (r * a.inv_k16) >> 16;
            if (row0 + rb >= a.n_rows || seq_s[rb] < 0) continue;
            const int at = g < RPT ? idx_s[rb * (K + 1)] : idx_s[rb * (K + 1) + (r - rb * K) + 1];
            term_src[k] = static_cast<const char*>(a.expanded_cache) +
                          ((static_cast<size_t>(seq_s[rb]) * a.max_t + at) * 2 * H + (g < RPT ? 0 : H)) * 2 + 16 * c;
        }
    }
    const uint32_t term_dst = static_cast<uint32_t>((tid >> 4) * kRowStride + 16 * (tid & 15));
    auto request_terms = [&](int j) {
        if (j < n_tiles) {
            const uint32_t dst = smem_u32(base + plan.terms[j & 1]) + term_dst;
#pragma unroll
            for (int k = 0; k < kTermRows; ++k)
                if (term_src[k]) cp_async16(dst + k * (kRowsThreads / 16) * kRowStride, term_src[k] + static_cast<size_t>(j) * kTcBN * 2);
        }
        cp_async_commit();
    };
    request_terms(0);
    fence_proxy_async();     // generic-proxy writes of the product tile -> visible to the tensor core
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    // thread 0: MMA of hidden tile j into accumulator j & 1 once its weight tile has landed
    auto issue_mma = [&](int j) {
        const int b = j & 1;
        if (mbar_wait(bar_w[b], (j >> 1) & 1)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = 0; kb < kblocks; ++kb) {
                const uint64_t da = smem_desc_sw128(smem_u32(a_tile) + kb * kBM * 128u);
                const uint64_t db = smem_desc_sw128(smem_u32(base + plan.w_tile[b]) + kb * kBM * 128u);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)
                    umma_f16(tmem_base + b * kTcBN, da + 2 * kk, db + 2 * kk, a.idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
        } else {
            failed = 1;
        }
        umma_commit(bar_acc[b]);     // accumulator complete (or abandoned)
    };
    if (tid == 0) issue_mma(0);

    // this thread's share of a tile: pair row `pr`, hidden columns [32 cg, 32 cg + 32) of the tile
    const int pr = 32 * (warp & 3) + lane, cg = warp >> 2;
    const int prb = (pr * a.inv_k16) >> 16;
    const bool pair_live = pr < tile_pairs && row0 + prb < a.n_rows && seq_s[prb < RPT ? prb : 0] >= 0;
    const uint32_t lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    bool good = true;
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
        const int b = j & 1;
        request_terms(j + 1);                                  // into the buffer tile j - 1 has left
        if (tid == 0) {
            if (j + 1 < n_tiles) issue_mma(j + 1);             // accumulator (j + 1) & 1 was read out in iteration j - 1
        }
        bool ready = mbar_wait(bar_acc[b], (j >> 1) & 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tid == 0 && ready && j + 2 < n_tiles) {            // weight buffer b is consumed: tile j + 2 may land
            mbar_expect_tx(bar_w[b], tile_bytes);
            for (int kb = 0; kb < kblocks; ++kb)
                tma_load_2d(smem_u32(base + plan.w_tile[b]) + kb * kBM * 128u, &map_wm, kb * kBK, (j + 2) * kTcBN, bar_w[b]);
        }
        cp_async_wait_group1();                                // the terms of tile j (tile j + 1's may be in flight)
        ready = ready && (*reinterpret_cast<volatile int*>(&failed) == 0);
        if (__syncthreads_or(!ready)) { good = false; break; }
        unsigned char* g_anchor = base + plan.terms[b];
        unsigned char* g_partner = g_anchor + plan.partner_rows;
        const unsigned char* ga = g_anchor + (prb < RPT ? prb : 0) * kRowStride + 64 * cg;
        const unsigned char* gp = g_partner + pr * kRowStride + 64 * cg;
        // results leave straight from the registers: 64 contiguous bytes of the pair's output row per thread
        uint16_t* orow = static_cast<uint16_t*>(a.out) + (static_cast<size_t>(row0) * K + pr) * H + j * kTcBN + 32 * cg;
        // both halves of this thread's 32 accumulator columns in one round trip to the tensor memory
        uint32_t v2[2][16];
        tmem_ld16(tmem_base + lane_base + b * kTcBN + 32 * cg, v2[0]);
        tmem_ld16(tmem_base + lane_base + b * kTcBN + 32 * cg + 16, v2[1]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const uint32_t (&v)[16] = v2[q];
            if (!pair_live) continue;
            float y[16];
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf) {
                float2 fa[4], fp[4];
                unpack8_pairs(*reinterpret_cast<const uint4*>(ga + 32 * q + 16 * hlf), kDt, fa);
                unpack8_pairs(*reinterpret_cast<const uint4*>(gp + 32 * q + 16 * hlf), kDt, fp);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 acc = make_float2(__uint_as_float(v[8 * hlf + 2 * i]), __uint_as_float(v[8 * hlf + 2 * i + 1]));
                    const float2 g = gelu_tc2(__fadd2_rn(acc, __fadd2_rn(fa[i], fp[i])));
                    y[8 * hlf + 2 * i] = g.x;
                    y[8 * hlf + 2 * i + 1] = g.y;
                }
            }
            uint4* o = reinterpret_cast<uint4*>(orow + 16 * q);
            o[0] = make_uint4(pack2(y[0], y[1], kOut), pack2(y[2], y[3], kOut), pack2(y[4], y[5], kOut), pack2(y[6], y[7], kOut));
            o[1] = make_uint4(pack2(y[8], y[9], kOut), pack2(y[10], y[11], kOut), pack2(y[12], y[13], kOut),
                              pack2(y[14], y[15], kOut));
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();                                       // staging buffer b and accumulator b are free
    }
    if (!good) {
        cp_async_wait_all();
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_TIMEOUT);
    }
    cp_async_wait_all();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem_base), "r"(2 * kTcBN) : "memory");
}

// ------------------------------------------------------------------ expanded row of position t

// grid (H / 128, 2 halves, layers x sequence groups of up to 64); the weight tensor maps cover
// the layers stacked along the rows ([layers * H, R]).  `n_cols` = sequences of the group rounded
// up to 16 = MMA N = TMEM columns in use; `tmem_cols` the power of two allocated.
__global__ void __launch_bounds__(kUpdThreads) expanded_row_update_kernel(
    const __grid_constant__ CUtensorMap map_wa, const __grid_constant__ CUtensorMap map_wp,
    const RowUpdateArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int R = a.rdim, H = a.hdim;
    const int kblocks = R / kBK, chunks = R / 8;
    const int layer = blockIdx.z / a.seq_groups;
    const int h0 = blockIdx.x * kTcBN, half = blockIdx.y, s0 = (blockIdx.z - layer * a.seq_groups) * kUpdMaxSeq;
    const int n_here = min(a.n_seq - s0, kUpdMaxSeq);
    const int n_cols = (n_here + 15) & ~15;
    int tmem_cols = 32;
    while (tmem_cols < n_cols) tmem_cols *= 2;
    const uint32_t fmt = a.dtype == RLM_BF16 ? 1u : 0u;
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(n_cols >> 3) << 17) |
                           (static_cast<uint32_t>(kBM >> 4) << 24);

    // With the packed rows as the source nothing this kernel reads comes from the launch right before it
    // (the state append, which it then overlaps): the dependency wait moves to the end, where it only
    // keeps the stream's ordering chain intact.
    const bool early = a.packed != nullptr;
    const int t = static_cast<int>(*a.position);
    if (t < 0 || t >= a.max_t) {
        if (tid == 0 && a.status) atomicOr(a.status, RLM_DEV_POSITION);
        griddep_sync();
        return;
    }

    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const uint32_t w_bytes = static_cast<uint32_t>(kblocks) * kBM * 128u;
    unsigned char* w_tile = base;
    unsigned char* cur_tile = base + w_bytes;                 // [kblocks][n_cols][128 B]
    const uint32_t cur_kblock = static_cast<uint32_t>(n_cols) * 128u;

    const uint32_t bar_w = smem_u32(&bars[0]), bar_acc = smem_u32(&bars[1]);
    if (tid == 0) {
        const CUtensorMap* map = half ? &map_wp : &map_wa;
        asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
        mbar_init(bar_w, 1);
        mbar_init(bar_acc, 1);
        fence_barrier_init();
        failed = 0;
        mbar_expect_tx(bar_w, w_bytes);
        for (int kb = 0; kb < kblocks; ++kb)
            tma_load_2d(smem_u32(w_tile) + kb * kBM * 128u, map, kb * kBK, layer * H + h0, bar_w);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (!early) griddep_sync();
    // current operand rows of the group's sequences (zero rows up to n_cols), copied
    // asynchronously straight to their swizzled places
    const size_t op_row = static_cast<size_t>(R) * 2;
    const int items = n_cols * chunks;
    for (int i = tid; i < items; i += kUpdThreads) {
        const int j = i / chunks, c = i - j * chunks;
        const uint32_t dst = smem_u32(cur_tile) + swizzled(j, c, cur_kblock);
        if (j < n_here)
            cp_async16(dst, early ? static_cast<const char*>(a.packed) +
                                        (static_cast<size_t>(s0 + j) * a.packed_stride + layer * a.packed_layer + a.packed_offset) * 2 + 16 * c
                                  : static_cast<const char*>(a.operand_cache) +
                                        ((static_cast<size_t>(layer) * a.n_seq + s0 + j) * a.max_t + t) * op_row + 16 * c);
        else
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
    }
    cp_async_commit();
    cp_async_wait_all();
    fence_proxy_async();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (tid == 0) {
        bool ok = mbar_wait(bar_w, 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = 0; kb < kblocks; ++kb) {
                const uint64_t dw = smem_desc_sw128(smem_u32(w_tile) + kb * kBM * 128u);
                const uint64_t dc = smem_desc_sw128(smem_u32(cur_tile) + kb * cur_kblock);
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk)
                    umma_f16(tmem_base, dw + 2 * kk, dc + 2 * kk, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
        } else {
            failed = 1;
        }
        umma_commit(bar_acc);
    }
    __syncwarp();

    bool ready = mbar_wait(bar_acc, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    ready = ready && (*reinterpret_cast<volatile int*>(&failed) == 0);
    if (!__syncthreads_or(!ready)) {
        // this thread owns hidden column h0 + tid of the half: one 2-byte store per sequence,
        // a warp's 32 stores of one sequence are 64 contiguous bytes of its cache row
        const float bias = half == 0 ? load_scalar(a.first_bias, static_cast<int64_t>(layer) * H + h0 + tid, a.dtype) : 0.0f;
        const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;
        uint16_t* cache = static_cast<uint16_t*>(a.expanded_cache);
        for (int c = 0; c < n_cols; c += 16) {
            uint32_t v[16];
            tmem_ld16(tmem_base + lane_base + c, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (c + j >= n_here) continue;
                const float val = __uint_as_float(v[j]) + bias;
                uint16_t bits;
                if (a.dtype == RLM_BF16) {
                    __nv_bfloat16 hv = __float2bfloat16_rn(val);
                    bits = *reinterpret_cast<uint16_t*>(&hv);
                } else {
                    __half hv = __float2half_rn(val);
                    bits = *reinterpret_cast<uint16_t*>(&hv);
                }
                cache[((static_cast<size_t>(layer) * a.n_seq + s0 + c + j) * a.max_t + t) * 2 * H + half * H + h0 + tid] = bits;
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
    if (early) griddep_sync();       // every kernel waits for its predecessor before it lets its successor go
}

size_t gather_smem_bytes(int rdim, int k_out) { return 1024 + gather_plan(rdim, kBM / k_out).total; }

size_t update_smem_bytes(int rdim, int n_seq) {
    const int n_cols = ((n_seq < kUpdMaxSeq ? n_seq : kUpdMaxSeq) + 15) & ~15;
    return 1024 + static_cast<size_t>(rdim / kBK) * (kBM + n_cols) * 128;
}

}  // namespace

// Whether the tensor-core form applies; the callers fall back to the CUDA-core kernel otherwise.
bool hidden_tc_applicable(bool update, int n_rows, int rdim, int hdim, int k_out, int cache_dtype,
                          int weight_dtype, const void* expanded_cache, const void* out) {
    if (cache_dtype != weight_dtype || (cache_dtype != RLM_BF16 && cache_dtype != RLM_F16)) return false;
    if (rdim % kBK != 0 || hdim % kTcBN != 0 || k_out < 1 || k_out > 16) return false;
    if (static_cast<long long>(n_rows) * k_out < 256) return false;    // small launches: latency-bound form
    if (!aligned16(expanded_cache) || !aligned16(out)) return false;
    if (gather_smem_bytes(rdim, k_out) > static_cast<size_t>(kSmemDynamicLimit)) return false;
    if (update && update_smem_bytes(rdim, n_rows) > static_cast<size_t>(kSmemDynamicLimit)) return false;
    return true;
}

// Expanded rows of the current position for `layers` stacked caches in one launch.
int launch_row_update(void* expanded_cache, const void* operand_cache, const void* anchor_weight,
                      const void* partner_weight, const void* first_bias, const int64_t* position,
                      int layers, int n_seq, int max_t, int rdim, int hdim, int dtype, int32_t* status,
                      void* stream, const void* packed = nullptr, int64_t packed_stride = 0, int packed_layer = 0,
                      int packed_offset = 0) {
    RowUpdateArgs u{};
    u.packed = packed; u.packed_stride = packed_stride; u.packed_layer = packed_layer; u.packed_offset = packed_offset;
    u.expanded_cache = expanded_cache; u.operand_cache = operand_cache; u.first_bias = first_bias;
    u.position = position; u.status = status; u.n_seq = n_seq; u.max_t = max_t; u.rdim = rdim;
    u.hdim = hdim; u.dtype = dtype;
    u.seq_groups = (n_seq + kUpdMaxSeq - 1) / kUpdMaxSeq;
    CUtensorMap ma, mp;
    if (!make_map(&ma, anchor_weight, layers * hdim, rdim, rdim, kTcBN, dtype) ||
        !make_map(&mp, partner_weight, layers * hdim, rdim, rdim, kTcBN, dtype)) {
        set_error("relation_hidden: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    auto kernel = expanded_row_update_kernel;
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    dim3 grid(hdim / kTcBN, 2, layers * u.seq_groups);
    launch_kernel(kernel, grid, dim3(kUpdThreads), update_smem_bytes(rdim, n_seq), stream, ma, mp, u);
    count_launch();
    return check_launch("expanded_row_update_kernel");
}

int launch_hidden_tc(bool update, void* expanded_cache, const void* operand_cache,
                     const int32_t* anchor_index, const int32_t* partner_index,
                     const void* anchor_weight, const void* partner_weight, const void* product_weight,
                     const void* first_bias, const int64_t* position, const int32_t* row_batch, void* out,
                     int n_rows, int n_seq, int max_t, int rdim, int hdim, int k_out, int dtype,
                     int out_dtype, int32_t* status, void* stream) {
    const uint32_t fmt = dtype == RLM_BF16 ? 1u : 0u;
    if (update) {
        int rc = launch_row_update(expanded_cache, operand_cache, anchor_weight, partner_weight, first_bias,
                                   position, 1, n_seq, max_t, rdim, hdim, dtype, status, stream);
        if (rc != RLM_OK) return rc;
    }
    HiddenTcArgs a{};
    a.expanded_cache = expanded_cache; a.operand_cache = operand_cache; a.anchor_index = anchor_index;
    a.partner_index = partner_index; a.row_batch = row_batch; a.out = out; a.status = status;
    a.n_rows = n_rows; a.n_seq = n_seq; a.max_t = max_t; a.rdim = rdim; a.hdim = hdim; a.k_out = k_out;
    a.dtype = dtype; a.out_dtype = out_dtype;
    a.rows_per_tile = kBM / k_out;
    a.inv_k16 = (65536 + k_out - 1) / k_out;
    a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kTcBN >> 3) << 17) |
              (static_cast<uint32_t>(kBM >> 4) << 24);
    CUtensorMap mm;
    if (!make_map(&mm, product_weight, hdim, rdim, rdim, kTcBN, dtype)) {
        set_error("relation_hidden: cuTensorMapEncodeTiled failed");
        return RLM_ERR_LAUNCH;
    }
    using Kernel = void (*)(const CUtensorMap, const HiddenTcArgs);
    Kernel kernel = nullptr;
    if (dtype == RLM_BF16)
        kernel = out_dtype == RLM_F32 ? relation_hidden_tc_kernel<RLM_BF16, RLM_F32>
               : out_dtype == RLM_BF16 ? relation_hidden_tc_kernel<RLM_BF16, RLM_BF16>
                                       : relation_hidden_tc_kernel<RLM_BF16, RLM_F16>;
    else
        kernel = out_dtype == RLM_F32 ? relation_hidden_tc_kernel<RLM_F16, RLM_F32>
               : out_dtype == RLM_BF16 ? relation_hidden_tc_kernel<RLM_F16, RLM_BF16>
                                       : relation_hidden_tc_kernel<RLM_F16, RLM_F16>;
    const int row_tiles = (n_rows + a.rows_per_tile - 1) / a.rows_per_tile;
    const size_t rows_smem = 1024 + rows_plan(rdim, a.rows_per_tile).total;
    if (out_dtype != RLM_F32 && row_tiles >= 2 * sm_count() && hdim / kTcBN >= 2 &&
        rows_smem <= static_cast<size_t>(kSmemDynamicLimit)) {
        // many row tiles: a CTA per pair tile walks all hidden tiles (see relation_hidden_rows_kernel)
        Kernel rows_kernel =
            dtype == RLM_BF16 ? (out_dtype == RLM_BF16 ? relation_hidden_rows_kernel<RLM_BF16, RLM_BF16>
                                                       : relation_hidden_rows_kernel<RLM_BF16, RLM_F16>)
                              : (out_dtype == RLM_BF16 ? relation_hidden_rows_kernel<RLM_F16, RLM_BF16>
                                                       : relation_hidden_rows_kernel<RLM_F16, RLM_F16>);
        int rc = allow_large_smem(reinterpret_cast<const void*>(rows_kernel), kSmemPerCta);
        if (rc != RLM_OK) return rc;
        launch_kernel(rows_kernel, dim3(row_tiles), dim3(kRowsThreads), rows_smem, stream, mm, a);
        count_launch();
        return check_launch("relation_hidden_rows_kernel");
    }
    int rc = allow_large_smem(reinterpret_cast<const void*>(kernel), kSmemPerCta);
    if (rc != RLM_OK) return rc;
    dim3 grid(hdim / kTcBN, row_tiles);
    launch_kernel(kernel, dim3(grid), dim3(kTcThreads), gather_smem_bytes(rdim, k_out), stream, mm, a);
    count_launch();
    return check_launch("relation_hidden_tc_kernel");
}

}  // namespace rlm

extern "C" int rlm_expanded_cache_append_packed(void* expanded_cache, const void* packed, int64_t packed_row_stride,
                                                int packed_layer_stride, int operand_offset,
                                                const void* anchor_weight, const void* partner_weight,
                                                const void* first_bias, const int64_t* position, int layers,
                                                int batch, int max_t, int relation_dim, int hidden_dim,
                                                int dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (layers == 0 || batch == 0) return RLM_OK;
    if (!expanded_cache || !packed || !anchor_weight || !partner_weight || !first_bias || !position) {
        set_error("expanded_cache_append_packed: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (layers < 0 || batch < 0 || max_t < 1 || relation_dim < kBK || relation_dim % kBK != 0 ||
        hidden_dim < 128 || hidden_dim % 128 != 0 || operand_offset < 0 || operand_offset % 8 != 0 ||
        packed_layer_stride < operand_offset + relation_dim || packed_layer_stride % 8 != 0 ||
        packed_row_stride < static_cast<int64_t>(layers) * packed_layer_stride || packed_row_stride % 8 != 0) {
        set_error("expanded_cache_append_packed: need relation_dim a multiple of 64, hidden_dim a multiple of 128 and "
                  "packed rows whose layer stride, operand offset and row stride are multiples of 8 elements");
        return RLM_ERR_SHAPE;
    }
    if (dtype != RLM_BF16 && dtype != RLM_F16) {
        set_error("expanded_cache_append_packed: caches, packed rows and weights must be bfloat16 or float16");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(expanded_cache) || !aligned16(packed) || !aligned16(anchor_weight) || !aligned16(partner_weight)) {
        set_error("expanded_cache_append_packed: tensors must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    return launch_row_update(expanded_cache, nullptr, anchor_weight, partner_weight, first_bias, position, layers, batch,
                             max_t, relation_dim, hidden_dim, dtype, status, stream, packed, packed_row_stride,
                             packed_layer_stride, operand_offset);
}

extern "C" int rlm_expanded_cache_append(void* expanded_cache, const void* operand_cache,
                                         const void* anchor_weight, const void* partner_weight,
                                         const void* first_bias, const int64_t* position, int layers,
                                         int batch, int max_t, int relation_dim, int hidden_dim,
                                         int dtype, int32_t* status, void* stream) {
    using namespace rlm;
    if (layers == 0 || batch == 0) return RLM_OK;
    if (!expanded_cache || !operand_cache || !anchor_weight || !partner_weight || !first_bias || !position) {
        set_error("expanded_cache_append: NULL pointer");
        return RLM_ERR_NULL;
    }
    if (layers < 0 || batch < 0 || max_t < 1 || relation_dim < kBK || relation_dim % kBK != 0 ||
        hidden_dim < 128 || hidden_dim % 128 != 0) {
        set_error("expanded_cache_append: need relation_dim a multiple of 64 and hidden_dim a multiple of 128");
        return RLM_ERR_SHAPE;
    }
    if (dtype != RLM_BF16 && dtype != RLM_F16) {
        set_error("expanded_cache_append: caches and weights must be bfloat16 or float16");
        return RLM_ERR_UNSUPPORTED;
    }
    if (!aligned16(expanded_cache) || !aligned16(operand_cache) || !aligned16(anchor_weight) ||
        !aligned16(partner_weight)) {
        set_error("expanded_cache_append: tensors must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    return launch_row_update(expanded_cache, operand_cache, anchor_weight, partner_weight, first_bias, position,
                             layers, batch, max_t, relation_dim, hidden_dim, dtype, status, stream);
}

