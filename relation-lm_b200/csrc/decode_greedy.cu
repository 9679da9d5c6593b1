// Greedy next token of a decode step (sm_100a): per row the index of the largest of the first
// `vocab` logits (ties to the lowest index), optionally advancing the device position scalar
// of the decoder — the `logits.argmax(-1)` and `position += 1` that close a decode step, in one
// launch.  One CTA per row; 16-byte loads; warp redux arg-max on order-preserving keys.

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kGreedyThreads = 256;

struct GreedyArgs {
    const void* logits;
    int64_t* next_token;
    int64_t* position;       // optional: incremented by one
    int64_t row_stride;      // elements
    int rows, vocab, dtype;
};

__global__ void __launch_bounds__(kGreedyThreads) greedy_token_kernel(const GreedyArgs a) {
    __shared__ uint32_t warp_key[kGreedyThreads / 32];
    __shared__ int warp_idx[kGreedyThreads / 32];
    griddep_sync();
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int elem = a.dtype == RLM_F32 ? 4 : 2;
    const char* base = static_cast<const char*>(a.logits) + static_cast<size_t>(row) * a.row_stride * elem;
    uint32_t best = 0;
    int best_idx = 0x7fffffff;
    const int chunks = a.vocab / 8;
    for (int c = tid; c < chunks; c += kGreedyThreads) {
        float f[8];
        load8(base, 8 * c, a.dtype, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t key = float_key(f[i] + 0.0f);
            if (key > best || best_idx == 0x7fffffff) { best = key; best_idx = 8 * c + i; }
        }
    }
    for (int c = 8 * chunks + tid; c < a.vocab; c += kGreedyThreads) {        // tail columns
        const uint32_t key = float_key(load_scalar(base, c, a.dtype) + 0.0f);
        if (key > best || best_idx == 0x7fffffff || (key == best && c < best_idx)) { best = key; best_idx = c; }
    }
    warp_argmax_key(best, best_idx);
    if (lane == 0) { warp_key[warp] = best; warp_idx[warp] = best_idx; }
    __syncthreads();
    if (warp == 0) {
        best = lane < kGreedyThreads / 32 ? warp_key[lane] : 0u;
        best_idx = lane < kGreedyThreads / 32 ? warp_idx[lane] : 0x7fffffff;
        if (best_idx == 0x7fffffff) best = 0u;
        warp_argmax_key(best, best_idx);
        if (lane == 0) {
            a.next_token[row] = best_idx == 0x7fffffff ? 0 : best_idx;
            if (row == 0 && a.position) *a.position += 1;
        }
    }
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_greedy_token(const void* logits, int64_t row_stride, int64_t* next_token,
                                int64_t* position, int rows, int vocab, int dtype, void* stream) {
    using namespace rlm;
    if (rows == 0) return RLM_OK;
    if (!logits || !next_token) { set_error("greedy_token: NULL pointer"); return RLM_ERR_NULL; }
    if (rows < 0 || vocab < 1 || row_stride < vocab) {
        set_error("greedy_token: need a positive vocabulary no wider than the row stride");
        return RLM_ERR_SHAPE;
    }
    if (!valid_dtype(dtype)) { set_error("greedy_token: unknown dtype code"); return RLM_ERR_DTYPE; }
    if (!aligned16(logits) || (row_stride * (dtype == RLM_F32 ? 4 : 2)) % 16 != 0) {
        set_error("greedy_token: rows must be 16-byte aligned");
        return RLM_ERR_ALIGN;
    }
    GreedyArgs a{logits, next_token, position, row_stride, rows, vocab, dtype};
    launch_kernel(greedy_token_kernel, dim3(rows), dim3(kGreedyThreads), 0, stream, a);
    count_launch();
    return check_launch("greedy_token_kernel");
}
