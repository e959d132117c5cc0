// Library-wide host helpers: version, last-error string, cached device properties.
#include <atomic>
#include <stdio.h>
#include <string.h>

#include "mok_common.cuh"

namespace mok {
namespace {
thread_local char g_last_error[512] = "";
std::atomic<long long> g_launches{0};
}

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_last_error(const char* what, cudaError_t err) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(err));
}

int fail_cuda(const char* what, cudaError_t err) {
    set_last_error(what, err);
    return MOK_ERR_CUDA;
}

int sm_count() {
    static int cached[16] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 16 && cached[dev] > 0) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < 16) cached[dev] = n;
    return n;
}

}  // namespace mok

extern "C" int mok_version(void) { return 100; }

extern "C" const char* mok_last_error(void) { return mok::g_last_error; }

extern "C" long long mok_launch_count(void) { return mok::g_launches.load(); }
