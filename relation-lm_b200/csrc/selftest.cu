// Self-test of the bounded device-side wait (extension; test support).
//
// Every kernel of the library waits for its bulk copies with mbar_wait(): a try-wait loop that
// gives up after a cycle limit, reports RLM_DEV_TIMEOUT through the status word and lets the
// kernel return instead of spinning for ever.  That path never runs in a healthy process, so
// this entry point runs it on purpose in the only harmless way: one CTA initialises an
// mbarrier that no copy and no thread will ever complete, waits on it with a limit of a few
// thousand cycles, and reports the expiry like any other kernel.  Nothing faults, nothing hangs.

#include "rlm_common.cuh"

namespace rlm {
namespace {

__global__ void bounded_wait_selftest_kernel(int32_t* status, long long limit, long long* waited) {
    __shared__ __align__(8) unsigned long long barrier;
    const uint32_t bar = smem_u32(&barrier);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    const long long start = clock64();
    const bool arrived = mbar_wait_limit(bar, 0, limit);     // nobody arrives: the wait must expire
    const long long spent = clock64() - start;
    if (__syncthreads_or(!arrived)) {
        if (threadIdx.x == 0) {
            if (status) atomicOr(status, RLM_DEV_TIMEOUT);
            if (waited) *waited = spent;
        }
        return;
    }
    if (threadIdx.x == 0 && waited) *waited = -1;            // unreachable: the barrier completed
}

}  // namespace
}  // namespace rlm

extern "C" int rlm_selftest_bounded_wait(int32_t* status, int64_t cycle_limit, int64_t* waited_cycles,
                                         void* stream) {
    using namespace rlm;
    if (!status) { set_error("selftest_bounded_wait: status word required"); return RLM_ERR_NULL; }
    if (cycle_limit < 1 || cycle_limit > (1ll << 24)) {
        set_error("selftest_bounded_wait: cycle limit must be between 1 and 2^24 (a few milliseconds)");
        return RLM_ERR_SHAPE;
    }
    launch_kernel(bounded_wait_selftest_kernel, dim3(1), dim3(64), 0, stream, status,
                  static_cast<long long>(cycle_limit), reinterpret_cast<long long*>(waited_cycles));
    count_launch();
    return check_launch("bounded_wait_selftest_kernel");
}
