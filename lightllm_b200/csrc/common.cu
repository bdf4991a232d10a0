// Error reporting shared by every exported function of the library.
#include "common.cuh"

#include <cstdarg>
#include <cstdio>

static thread_local char g_last_error[1024] = "";
static unsigned long long g_launches = 0;

int llb_fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return -1;
}

int llb_check_launch(const char* what) {
    ++g_launches;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return llb_fail("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

// The message of the last failed call on this thread ("" if none failed yet).
LLB_EXPORT const char* llb_last_error() { return g_last_error; }

// Kernels launched by this library so far (every launch is followed by one llb_check_launch).
LLB_EXPORT unsigned long long llb_launch_count() { return g_launches; }

// Version tag checked by the Python binding, so that a stale library is rebuilt.
LLB_EXPORT int llb_abi_version() { return 21; }
