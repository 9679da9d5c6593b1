// Sliding decode state: drop the oldest rows of position-indexed caches in place (sm_100a).
//
// The decode state of the reference is a set of caches with one row per position of a fixed
// context (src/relation_lm/inference/packed_cache.py:10-17 names them; the router's caches and
// block statistics follow src/relation_lm/kernels/router_cache.py:256-291), and "persistent
// ring-buffer state and contexts beyond 512" is an open item of its roadmap (docs/roadmap.md:8).
// A decoder that has filled its context goes on here by sliding the state: every cache
// [outer, rows, row bytes] moves rows [shift, rows) to [0, rows - shift) — whole blocks of the
// router, so block statistics slide by whole rows of their own tensors — and the position is
// lowered by the same amount.  What a later step can select is what a ring of the same capacity
// would still hold; rows [rows - shift, rows) keep their old content, which no kernel reads before
// the append has rewritten it (positions beyond the current one are never candidates).
//
// One launch slides up to 16 tensors.  A thread owns one 16-byte column of one [rows, row bytes]
// matrix and, of that column, the rows r = q (mod P) for a divisor P of the shift: the row that
// replaces row r, r + shift, is then one of its own, so threads never touch each other's bytes and
// the move needs no barrier and no second buffer.  It walks its rows upwards, eight at a time —
// eight loads, then eight stores; a row is always read before it is overwritten because its reader
// is the same thread, earlier in program order.  P is chosen on the host so that the launch has
// about a thousand threads per SM: the kernel is bound by the bytes it keeps in flight (128 per
// thread), and a decode batch of eight sequences has only 30 k columns.  Warps cover adjacent
// columns, so every access is a full line.  HBM-bound: every surviving byte is read once and
// written once.

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kSlThreads = 256;
constexpr int kSlMaxTensors = 16;
constexpr int kSlAhead = 8;                       // rows a thread keeps in flight

struct SlideArgs {
    char* base[kSlMaxTensors];
    long long first_item[kSlMaxTensors + 1];      // prefix sums of outer * chunks * split
    int rows[kSlMaxTensors];
    int chunks[kSlMaxTensors];                    // 16-byte columns per row
    int shift[kSlMaxTensors];
    int split[kSlMaxTensors];                     // P: row classes per column (a divisor of the shift)
    int n;
};

__global__ void __launch_bounds__(kSlThreads, 4) state_slide_kernel(const SlideArgs a) {
    griddep_sync();
    const long long stride = static_cast<long long>(gridDim.x) * kSlThreads;
    for (long long item = static_cast<long long>(blockIdx.x) * kSlThreads + threadIdx.x; item < a.first_item[a.n];
         item += stride) {
        int k = 0;
        while (item >= a.first_item[k + 1]) ++k;
        const long long local = item - a.first_item[k];
        const int chunks = a.chunks[k], rows = a.rows[k], shift = a.shift[k], split = a.split[k];
        // columns fastest (adjacent threads, adjacent bytes), then the row class, then the matrix
        const int col = static_cast<int>(local % chunks);
        const long long rest = local / chunks;
        const int q = static_cast<int>(rest % split);
        const long long outer = rest / split;
        const size_t row_bytes = static_cast<size_t>(chunks) * 16;
        char* column = a.base[k] + static_cast<size_t>(outer) * rows * row_bytes + static_cast<size_t>(col) * 16;
        const int last = rows - shift;                        // rows [0, last) receive a new content
        for (int r = q; r < last; r += kSlAhead * split) {
            uint4 v[kSlAhead];
#pragma unroll
            for (int i = 0; i < kSlAhead; ++i)
                if (r + i * split < last)
                    v[i] = *reinterpret_cast<const uint4*>(column + static_cast<size_t>(r + i * split + shift) * row_bytes);
#pragma unroll
            for (int i = 0; i < kSlAhead; ++i)
                if (r + i * split < last)
                    *reinterpret_cast<uint4*>(column + static_cast<size_t>(r + i * split) * row_bytes) = v[i];
        }
    }
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_state_slide(void* const* tensors, const int64_t* n_outer, const int64_t* rows,
                               const int64_t* row_bytes, const int64_t* shift_rows, int n_tensors, void* stream) {
    using namespace rlm;
    if (n_tensors == 0) return RLM_OK;
    if (!tensors || !n_outer || !rows || !row_bytes || !shift_rows) {
        set_error("state_slide: NULL argument");
        return RLM_ERR_NULL;
    }
    if (n_tensors < 0 || n_tensors > kSlMaxTensors) {
        set_error("state_slide: 1 to 16 tensors per call");
        return RLM_ERR_SHAPE;
    }
    SlideArgs a{};
    long long columns = 0;
    int n = 0;
    for (int k = 0; k < n_tensors; ++k) {
        if (!tensors[k]) { set_error("state_slide: NULL tensor"); return RLM_ERR_NULL; }
        if (n_outer[k] < 0 || rows[k] < 1 || rows[k] > 0x7fffffff || row_bytes[k] < 1 ||
            row_bytes[k] / 16 > 0x7fffffff || shift_rows[k] < 0 || shift_rows[k] >= rows[k]) {
            set_error("state_slide: needs rows >= 1 and 0 <= shift < rows");
            return RLM_ERR_SHAPE;
        }
        if (row_bytes[k] % 16 != 0 || !aligned16(tensors[k])) {
            set_error("state_slide: rows must be multiples of 16 bytes on a 16-byte aligned base");
            return RLM_ERR_ALIGN;
        }
        if (shift_rows[k] == 0 || n_outer[k] == 0) continue;      // nothing moves
        a.base[n] = static_cast<char*>(tensors[k]);
        a.rows[n] = static_cast<int>(rows[k]);
        a.chunks[n] = static_cast<int>(row_bytes[k] / 16);
        a.shift[n] = static_cast<int>(shift_rows[k]);
        a.first_item[n + 1] = n_outer[k] * (row_bytes[k] / 16);   // columns of this tensor, for now
        columns += a.first_item[n + 1];
        ++n;
    }
    if (columns == 0) return RLM_OK;
    // row classes per column: the largest divisor of the shift that keeps the launch within about a
    // thousand threads per SM (and leaves every thread at least a few rows)
    const long long wanted = 1024ll * sm_count() / columns;
    long long items = 0;
    for (int k = 0; k < n; ++k) {
        int split = 1;
        for (int p = 2; p <= a.shift[k] && p <= wanted && p <= 1024 && p * 4 <= a.rows[k] - a.shift[k]; ++p)
            if (a.shift[k] % p == 0) split = p;
        a.split[k] = split;
        const long long mine = a.first_item[k + 1] * split;
        a.first_item[k] = items;
        items += mine;
    }
    a.first_item[n] = items;
    a.n = n;
    // a thread per item while that fills the machine, then a grid-stride walk
    long long ctas = (items + kSlThreads - 1) / kSlThreads;
    const long long most = 8ll * sm_count();
    if (ctas > most) ctas = most;
    launch_kernel(state_slide_kernel, dim3(static_cast<unsigned>(ctas)), dim3(kSlThreads), 0, stream, a);
    count_launch();
    return check_launch("state_slide_kernel");
}
