// Error plumbing and bookkeeping shared by the C-ABI entry points.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "pa_common.cuh"

namespace pa {

static thread_local char g_error[512] = "";
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t err, const char *what) {
    snprintf(g_error, sizeof g_error, "%s: %s (%d)", what, cudaGetErrorString(err),
             static_cast<int>(err));
    return PA_ERR_CUDA;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

}  // namespace pa

extern "C" int pa_version(void) { return 103; }  // 103: refinement merges / seeds by selection, narrow CTAs
extern "C" const char *pa_last_error(void) { return pa::g_error; }
extern "C" int64_t pa_launch_count(void) { return pa::g_launches.load(std::memory_order_relaxed); }
