// RMSNorm over rows of the residual stream, optionally only over a list of rows.
//
// ss = sum_d x_d^2 in float (src/ops/norm.cu:19-23); inv = 1 / sqrt(ss / D + eps) (:48-49);
// y_d = x_d * inv * w_d, then the cast (:50-54).  One block per row; the reference uses two
// launches and a global buffer for ss, here the row stays in registers between the passes
// when it fits.
#include <type_traits>

#include "common.cuh"

// Launch with the programmatic-stream-serialization attribute (the kernel calls griddepcontrol.wait itself).
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <typename TI, typename TW, typename TO, int PER_THREAD>
__global__ void rmsnorm_kernel(const TI* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int D, float eps) {
    // Programmatic dependent launch: let the next kernel start its preamble, then wait for the one before.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const TI* xr = x + (size_t)src * D;
    TO* o = out + (size_t)r * D;

    float v[PER_THREAD > 0 ? PER_THREAD : 1];
    float ss = 0.0f;
    if (PER_THREAD > 0) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            v[i] = d < D ? llb_to_float(xr[d]) : 0.0f;
            ss += v[i] * v[i];
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            const float a = llb_to_float(xr[d]);
            ss += a * a;
        }
    }
    __shared__ float warp_part[32];
    __shared__ float total;
    ss = llb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? warp_part[threadIdx.x] : 0.0f;
        t = llb_warp_sum(t);
        if (threadIdx.x == 0) total = t;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(total / (float)D + eps);
    if (PER_THREAD > 0) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            if (d < D) o[d] = llb_from_float<TO>(v[i] * inv * llb_to_float(w[d]));
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x)
            o[d] = llb_from_float<TO>(llb_to_float(xr[d]) * inv * llb_to_float(w[d]));
    }
}

// Four consecutive elements as one 16-byte (float) or 8-byte (bf16) access.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// One warp per row of a float input whose width is a multiple of 4 and at most 128 * NV: the row stays in
// registers as NV float4 per lane, the sum needs shuffles only, loads and stores are 16 / 8 bytes wide.
template <typename TW, typename TO, int NV>
__global__ void __launch_bounds__(256) rmsnorm_warp_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                                                           TO* __restrict__ out, const int* __restrict__ rows, int R,
                                                           int D, float eps) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float4 v[NV];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        v[i] = d < D ? *reinterpret_cast<const float4*>(xr + d) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
    ss = llb_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    TO* o = out + (size_t)r * D;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int d = (i * 32 + lane) * 4;
        if (d < D) {
            const float4 g = load4(w + d);
            store4(o + d, make_float4(v[i].x * inv * g.x, v[i].y * inv * g.y, v[i].z * inv * g.z, v[i].w * inv * g.w));
        }
    }
}

template <typename TI, typename TW, typename TO>
static int launch_rmsnorm(const void* x, const void* w, void* out, const int* rows, int R, int D, float eps,
                          cudaStream_t stream) {
    const int threads = 256;
    cudaError_t e;
    if (std::is_same<TI, float>::value && D % 4 == 0 && D <= 128 * 16 && (uintptr_t)x % 16 == 0 &&
        (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0 && R >= 8) {
        const dim3 grid((R + 7) / 8);
        if (D <= 128 * 8)
            e = launch_pdl(rmsnorm_warp_kernel<TW, TO, 8>, grid, dim3(threads), stream, (const float*)x, (const TW*)w,
                           (TO*)out, rows, R, D, eps);
        else
            e = launch_pdl(rmsnorm_warp_kernel<TW, TO, 16>, grid, dim3(threads), stream, (const float*)x, (const TW*)w,
                           (TO*)out, rows, R, D, eps);
    } else if (D <= threads * 4)
        e = launch_pdl(rmsnorm_kernel<TI, TW, TO, 4>, dim3(R), dim3(threads), stream, (const TI*)x, (const TW*)w, (TO*)out, rows, D, eps);
    else if (D <= threads * 16)
        e = launch_pdl(rmsnorm_kernel<TI, TW, TO, 16>, dim3(R), dim3(threads), stream, (const TI*)x, (const TW*)w, (TO*)out, rows, D, eps);
    else
        e = launch_pdl(rmsnorm_kernel<TI, TW, TO, 0>, dim3(R), dim3(threads), stream, (const TI*)x, (const TW*)w, (TO*)out, rows, D, eps);
    if (e != cudaSuccess) return llb_fail("rmsnorm: launch failed: %s", cudaGetErrorString(e));
    return llb_check_launch("rmsnorm");
}

template <typename TI, typename TW>
static int dispatch_out(int out_dtype, const void* x, const void* w, void* out, const int* rows, int R, int D,
                        float eps, cudaStream_t s) {
    if (out_dtype == LLB_F32) return launch_rmsnorm<TI, TW, float>(x, w, out, rows, R, D, eps, s);
    if (out_dtype == LLB_BF16) return launch_rmsnorm<TI, TW, __nv_bfloat16>(x, w, out, rows, R, D, eps, s);
    return llb_fail("rmsnorm: unknown output dtype %d", out_dtype);
}

template <typename TI>
static int dispatch_w(int w_dtype, int out_dtype, const void* x, const void* w, void* out, const int* rows, int R,
                      int D, float eps, cudaStream_t s) {
    if (w_dtype == LLB_F32) return dispatch_out<TI, float>(out_dtype, x, w, out, rows, R, D, eps, s);
    if (w_dtype == LLB_BF16) return dispatch_out<TI, __nv_bfloat16>(out_dtype, x, w, out, rows, R, D, eps, s);
    return llb_fail("rmsnorm: unknown weight dtype %d", w_dtype);
}

// x [*, D], w [D], out [R, D]; rows: R source-row indices into x, or null for rows 0..R-1.
LLB_EXPORT int llb_rmsnorm(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                           const int* rows, int R, int D, float eps, cudaStream_t stream) {
    if (R == 0) return 0;
    LLB_REQUIRE(R > 0 && D > 0, "rmsnorm: bad sizes R=%d D=%d", R, D);
    if (x_dtype == LLB_F32) return dispatch_w<float>(w_dtype, out_dtype, x, w, out, rows, R, D, eps, stream);
    if (x_dtype == LLB_BF16) return dispatch_w<__nv_bfloat16>(w_dtype, out_dtype, x, w, out, rows, R, D, eps, stream);
    return llb_fail("rmsnorm: unknown input dtype %d", x_dtype);
}
