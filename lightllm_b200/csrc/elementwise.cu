// Elementwise helpers of a block's arrangements beyond the plain pre-norm one: the residual stream in
// the compute dtype (a branch without a norm before it), a normed branch added into the stream, and a
// normed stream written back.  The residual add itself is src/ops/elementwise.cu:9-12 of the reference;
// here the common case has it inside the contractions' epilogues and only the rarer arrangements come here.
#include "common.cuh"

namespace {

// dst[i] = (ACCUMULATE ? dst[i] : 0) + src[i], converted through float.
template <typename TS, typename TD, bool ACCUMULATE>
__global__ void cast_add_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = llb_to_float(src[i]);
        if (ACCUMULATE) v += llb_to_float(dst[i]);
        dst[i] = llb_from_float<TD>(v);
    }
}

template <typename TS, typename TD>
int launch_cast(const void* src, void* dst, long long n, int accumulate, cudaStream_t stream) {
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 1184 ? (n + threads - 1) / threads : 1184);
    if (accumulate)
        cast_add_kernel<TS, TD, true><<<blocks, threads, 0, stream>>>((const TS*)src, (TD*)dst, n);
    else
        cast_add_kernel<TS, TD, false><<<blocks, threads, 0, stream>>>((const TS*)src, (TD*)dst, n);
    return llb_check_launch("cast_add");
}

}  // namespace

// dst[i] = src[i] (accumulate == 0) or dst[i] + src[i], for n elements; each side float or bf16.
LLB_EXPORT int llb_cast_add(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, int accumulate,
                            cudaStream_t stream) {
    if (n == 0) return 0;
    LLB_REQUIRE(n > 0 && src != nullptr && dst != nullptr, "cast_add: bad arguments");
    if (src_dtype == LLB_F32 && dst_dtype == LLB_F32) return launch_cast<float, float>(src, dst, n, accumulate, stream);
    if (src_dtype == LLB_F32 && dst_dtype == LLB_BF16) return launch_cast<float, __nv_bfloat16>(src, dst, n, accumulate, stream);
    if (src_dtype == LLB_BF16 && dst_dtype == LLB_F32) return launch_cast<__nv_bfloat16, float>(src, dst, n, accumulate, stream);
    if (src_dtype == LLB_BF16 && dst_dtype == LLB_BF16)
        return launch_cast<__nv_bfloat16, __nv_bfloat16>(src, dst, n, accumulate, stream);
    return llb_fail("cast_add: unknown dtypes %d, %d", src_dtype, dst_dtype);
}
