// L2 prefetch of tensors a decode step is about to read (sm_100a).
//
// One launch walks up to 16 address ranges and issues `prefetch.global.L2` for every 128-byte line,
// ranges in the order given (the order the step will need them).  It moves no data into the SMs and
// keeps no state: it is meant to run on a side stream (a sibling branch of the step's CUDA graph)
// while the first kernels of the step execute, so that the weights and caches of the later
// kernels — which a step that starts with a cold L2 would otherwise fetch from DRAM one dependent
// round trip at a time — are already on their way.

#include "rlm_common.cuh"

namespace rlm {
namespace {

constexpr int kPfThreads = 256;
constexpr int kPfMaxRanges = 16;

struct PrefetchArgs {
    const char* base[kPfMaxRanges];
    unsigned long long lines[kPfMaxRanges];     // 128-byte lines per range
    int n;
};

__global__ void __launch_bounds__(kPfThreads) l2_prefetch_kernel(const PrefetchArgs a) {
    const unsigned long long stride = static_cast<unsigned long long>(gridDim.x) * kPfThreads;
    const unsigned long long first = static_cast<unsigned long long>(blockIdx.x) * kPfThreads + threadIdx.x;
    for (int r = 0; r < a.n; ++r)
        for (unsigned long long i = first; i < a.lines[r]; i += stride)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a.base[r] + i * 128ull));
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_l2_prefetch(const void* const* ranges, const int64_t* bytes, int n_ranges, void* stream) {
    using namespace rlm;
    if (n_ranges == 0) return RLM_OK;
    if (!ranges || !bytes || n_ranges < 0 || n_ranges > kPfMaxRanges) {
        set_error("l2_prefetch: 1 to 16 ranges");
        return RLM_ERR_SHAPE;
    }
    PrefetchArgs a{};
    unsigned long long total = 0;
    for (int r = 0; r < n_ranges; ++r) {
        if (!ranges[r] || bytes[r] < 0) { set_error("l2_prefetch: NULL range or negative size"); return RLM_ERR_NULL; }
        // whole lines inside the range: the first line starts at the next 128-byte boundary
        const uintptr_t lo = (reinterpret_cast<uintptr_t>(ranges[r]) + 127) & ~static_cast<uintptr_t>(127);
        const uintptr_t hi = (reinterpret_cast<uintptr_t>(ranges[r]) + static_cast<uintptr_t>(bytes[r])) & ~static_cast<uintptr_t>(127);
        a.base[r] = reinterpret_cast<const char*>(lo);
        a.lines[r] = hi > lo ? (hi - lo) / 128 : 0;
        total += a.lines[r];
    }
    a.n = n_ranges;
    if (total == 0) return RLM_OK;
    unsigned long long ctas = (total + kPfThreads * 8ull - 1) / (kPfThreads * 8ull);
    const unsigned long long most = static_cast<unsigned long long>(sm_count());
    if (ctas > most) ctas = most;
    // an ordinary launch: the kernel depends on nothing and nothing waits for its data
    l2_prefetch_kernel<<<dim3(static_cast<unsigned>(ctas)), dim3(kPfThreads), 0, static_cast<cudaStream_t>(stream)>>>(a);
    count_launch();
    return check_launch("l2_prefetch_kernel");
}
