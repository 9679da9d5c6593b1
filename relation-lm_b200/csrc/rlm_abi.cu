// Library identity, error reporting and launch bookkeeping.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <set>
#include <utility>

#include "rlm_common.cuh"

namespace rlm {
namespace {
thread_local char g_error[512] = "";
std::atomic<int64_t> g_launches{0};
std::mutex g_attr_mutex;
std::set<std::pair<const void*, int>> g_attr_done;
}  // namespace

void set_error(const char* message) {
    std::snprintf(g_error, sizeof(g_error), "%s", message ? message : "");
}

// Per host thread: a decode loop that opts in on its own thread cannot change how another
// thread's launches (for instance the plain operators, whose callers know nothing of the
// ordering rule that comes with programmatic launch) are issued.
thread_local int g_programmatic = 0;
bool programmatic_launch_enabled() { return g_programmatic != 0; }

int sm_count() {
    static std::atomic<int> cached[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) { cudaGetLastError(); return 148; }
    int n = cached[device].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = 148;
        }
        cached[device].store(n, std::memory_order_relaxed);
    }
    return n;
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_launch(const char* kernel_name) {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return RLM_OK;
    char buffer[400];
    std::snprintf(buffer, sizeof(buffer), "%s: %s", kernel_name, cudaGetErrorString(e));
    set_error(buffer);
    return RLM_ERR_LAUNCH;
}

int allow_large_smem(const void* kernel, int bytes) {
    // `bytes` is the per-CTA total the hardware offers; static shared memory of the kernel
    // counts against it, so the dynamic limit is the remainder.
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaGetDevice failed");
        return RLM_ERR_LAUNCH;
    }
    std::lock_guard<std::mutex> lock(g_attr_mutex);
    auto key = std::make_pair(kernel, device);
    if (g_attr_done.count(key)) return RLM_OK;
    cudaFuncAttributes attr;
    cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 bytes - static_cast<int>(attr.sharedSizeBytes));
    if (e != cudaSuccess) {
        cudaGetLastError();   // do not leave the error for the next launch check
        set_error(cudaGetErrorString(e));
        return RLM_ERR_LAUNCH;
    }
    g_attr_done.insert(key);
    return RLM_OK;
}
}  // namespace rlm

extern "C" int rlm_set_programmatic_launch(int enabled) {
    const int previous = rlm::g_programmatic;
    rlm::g_programmatic = enabled ? 1 : 0;
    return previous;
}
extern "C" int rlm_abi_version(void) { return RLM_ABI_VERSION; }
extern "C" const char* rlm_last_error(void) { return rlm::g_error; }
extern "C" int64_t rlm_launch_count(void) { return rlm::g_launches.load(std::memory_order_relaxed); }
