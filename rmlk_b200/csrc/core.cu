// Library-wide helpers: thread-local error text, device capability cache, version.
#include <atomic>
#include "common.cuh"

#include <cstdlib>
#include <mutex>

namespace rmlk {

static thread_local std::string g_last_error;

void set_last_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return RMLK_ERR_CUDA_BASE + static_cast<int>(e);
}

int sm_count() {
    // Immutable per-device capability table, filled on first use.
    static std::atomic<int> counts[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = counts[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        counts[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

bool dep_launch_enabled() {
    static const bool v = [] {
        const char* e = getenv("RMLK_B200_NO_PDL");
        return !(e && e[0] == '1');
    }();
    return v;
}

}  // namespace rmlk

extern "C" const char* rmlk_b200_last_error(void) { return rmlk::g_last_error.c_str(); }
extern "C" const char* rmlk_b200_version(void) { return "rmlk_b200 0.1 (sm_100a)"; }
extern "C" size_t rmlk_b200_dtype_size(int dtype) { return rmlk::dtype_size(dtype); }
