// Shared declarations of the kernel library: dtype codes, error reporting, small device helpers.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a stream,
// allocates nothing, and returns 0 or a negative code after storing a message that
// llb_last_error() returns.  The reference reports CUDA faults by printing and carrying on
// (src/engine/engine_server.cpp:1427-1432); here a failed precondition or launch is an error
// the caller sees.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLB_EXPORT extern "C" __attribute__((visibility("default")))

enum LlbDtype { LLB_F32 = 0, LLB_BF16 = 1 };

// Epilogues of the dense contractions.
enum LlbEpilogue {
    LLB_EPI_STORE = 0,      // out[M,N]  (activation dtype) = acc (+ bias)
    LLB_EPI_STORE_F32 = 1,  // out[M,N]  float             = acc (+ bias)
    LLB_EPI_RESIDUAL = 2,   // res[M,N]  float            += acc (+ bias)
    LLB_EPI_SWIGLU = 3      // out[M,N/2] = silu(acc[2j] + b[2j]) * (acc[2j+1] + b[2j+1])
};

int llb_fail(const char* fmt, ...);          // stores the message, returns -1
int llb_check_launch(const char* what);      // cudaGetLastError() -> 0 or llb_fail

#define LLB_REQUIRE(cond, ...)                 \
    do {                                       \
        if (!(cond)) return llb_fail(__VA_ARGS__); \
    } while (0)

__device__ __forceinline__ float llb_to_float(float v) { return v; }
__device__ __forceinline__ float llb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T llb_from_float(float v);
template <> __device__ __forceinline__ float llb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 llb_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float llb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float llb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// x / (1 + exp(-x)) in float, as src/ops/elementwise.cu:27-33 computes SiLU.
__device__ __forceinline__ float llb_silu(float x) { return x / (1.0f + expf(-x)); }

static inline int llb_ceil_div(int a, int b) { return (a + b - 1) / b; }
