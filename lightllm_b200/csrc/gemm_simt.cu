// Dense contraction on CUDA cores with float accumulation: the true 32-bit path of every
// linear layer, and the path for shapes the tensor-core kernel refuses.
//
// C[M,N] = A[M,K] * W[N,K]^T, W stored [out, in] as in the checkpoint
// (src/engine/engine_server.cpp:1542-1544; the reference calls cublasSgemm for it,
// src/ops/gemm.cu:92-97, and keeps tiled teaching kernels at :44-81).  Products and sums are
// float FFMA: no tensor cores, no TF32.  Epilogues add the bias (which the reference never
// loads, engine_server.cpp:436-450), add into the float residual stream
// (engine_server.cpp:1870-1871), or apply SiLU(gate)*up on interleaved rows
// (src/ops/elementwise.cu:27-33, engine_server.cpp:1875-1878).
//
// Two kernels: a 64x64x16 tile kernel for many rows, and a row-streaming kernel for few rows
// (decode), where every weight row is read once by one warp with 16-byte loads.
#include "common.cuh"

namespace {

template <typename TO, int EPI>
struct Epilogue {
    // Called with two adjacent columns (n even) so that SwiGLU sees its gate/up pair.
    static __device__ __forceinline__ void pair(float a0, float a1, int m, int n, int N, void* out,
                                                float* residual, bool has1) {
        if (EPI == LLB_EPI_STORE) {
            TO* o = (TO*)out + (size_t)m * N + n;
            o[0] = llb_from_float<TO>(a0);
            if (has1) o[1] = llb_from_float<TO>(a1);
        } else if (EPI == LLB_EPI_STORE_F32) {
            float* o = (float*)out + (size_t)m * N + n;
            o[0] = a0;
            if (has1) o[1] = a1;
        } else if (EPI == LLB_EPI_RESIDUAL) {
            float* r = residual + (size_t)m * N + n;
            r[0] += a0;
            if (has1) r[1] += a1;
        } else {  // SWIGLU: column pair (2j, 2j+1) -> output column j of N/2
            TO* o = (TO*)out + (size_t)m * (N / 2) + (n >> 1);
            o[0] = llb_from_float<TO>(llb_silu(a0) * a1);
        }
    }
};

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TO, int EPI>
__global__ void __launch_bounds__(256) gemm_tile_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        const float* __restrict__ bias, void* __restrict__ out,
                                                        float* __restrict__ residual, int M, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;  // 0..1023 over a 64x16 tile
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            const int am = m0 + r, wn = n0 + r;
            As[kk][r] = (am < M && k < K) ? llb_to_float(A[(size_t)am * K + k]) : 0.0f;
            Ws[kk][r] = (wn < N && k < K) ? llb_to_float(W[(size_t)wn * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const bool has1 = n + 1 < N;
            float a0 = acc[i][j], a1 = acc[i][j + 1];
            if (bias) {
                a0 += bias[n];
                if (has1) a1 += bias[n + 1];
            }
            Epilogue<TO, EPI>::pair(a0, a1, m, n, N, out, residual, has1);
        }
    }
}

// Few rows (M <= MAXM): one warp owns a pair of weight rows (n, n+1) and streams them once.
// Lane l reads elements k = (c*32 + l)*VEC .. +VEC-1 of each chunk c; sums are float.
template <typename TA, typename TW, typename TO, int EPI, int MAXM, int VEC>
__global__ void __launch_bounds__(256) gemm_rows_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        const float* __restrict__ bias, void* __restrict__ out,
                                                        float* __restrict__ residual, int M, int N, int K) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int n = warp * 2;
    if (n >= N) return;
    const bool has1 = n + 1 < N;
    const TW* w0 = W + (size_t)n * K;
    const TW* w1 = W + (size_t)(has1 ? n + 1 : n) * K;
    float acc0[MAXM], acc1[MAXM];
#pragma unroll
    for (int m = 0; m < MAXM; ++m) acc0[m] = acc1[m] = 0.0f;

    for (int k = lane * VEC; k < K; k += 32 * VEC) {
        float x0[VEC], x1[VEC];
        if (VEC == 8) {  // 16-byte loads of bf16 weights
            const uint4 p0 = *reinterpret_cast<const uint4*>(w0 + k);
            const uint4 p1 = *reinterpret_cast<const uint4*>(w1 + k);
            const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&p0);
            const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&p1);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f0 = __bfloat1622float2(h0[i]);
                const float2 f1 = __bfloat1622float2(h1[i]);
                x0[2 * i] = f0.x; x0[2 * i + 1] = f0.y;
                x1[2 * i] = f1.x; x1[2 * i + 1] = f1.y;
            }
        } else if (VEC == 4) {  // 16-byte loads of float weights
            const float4 p0 = *reinterpret_cast<const float4*>(w0 + k);
            const float4 p1 = *reinterpret_cast<const float4*>(w1 + k);
            x0[0] = p0.x; x0[1] = p0.y; x0[2] = p0.z; x0[3] = p0.w;
            x1[0] = p1.x; x1[1] = p1.y; x1[2] = p1.z; x1[3] = p1.w;
        } else {
            x0[0] = llb_to_float(w0[k]);
            x1[0] = llb_to_float(w1[k]);
        }
#pragma unroll
        for (int m = 0; m < MAXM; ++m) {
            if (m < M) {
                const TA* a = A + (size_t)m * K + k;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    const float av = llb_to_float(a[i]);
                    acc0[m] = fmaf(av, x0[i], acc0[m]);
                    acc1[m] = fmaf(av, x1[i], acc1[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MAXM; ++m) {
        if (m < M) {  // M is uniform over the warp, so every lane takes part in the shuffles
            float a0 = llb_warp_sum(acc0[m]);
            float a1 = llb_warp_sum(acc1[m]);
            if (lane == 0) {
                if (bias) {
                    a0 += bias[n];
                    if (has1) a1 += bias[n + 1];
                }
                Epilogue<TO, EPI>::pair(a0, a1, m, n, N, out, residual, has1);
            }
        }
    }
}

template <typename TA, typename TW, typename TO, int EPI>
int launch(const void* A, const void* W, const void* bias, void* out, float* residual, int M, int N, int K,
           cudaStream_t stream) {
    const TA* a = (const TA*)A;
    const TW* w = (const TW*)W;
    const float* b = (const float*)bias;
    constexpr int MAXM = 8;
    if (M <= MAXM) {
        const int warps = (N + 1) / 2;
        const int threads = 128;
        const int blocks = llb_ceil_div(warps * 32, threads);
        constexpr int WVEC = sizeof(TW) == 2 ? 8 : 4;
        const bool aligned = (K % WVEC == 0) && ((uintptr_t)W % 16 == 0);
        if (aligned)
            gemm_rows_kernel<TA, TW, TO, EPI, MAXM, WVEC><<<blocks, threads, 0, stream>>>(a, w, b, out, residual, M, N, K);
        else
            gemm_rows_kernel<TA, TW, TO, EPI, MAXM, 1><<<blocks, threads, 0, stream>>>(a, w, b, out, residual, M, N, K);
        return llb_check_launch("gemm_rows");
    }
    dim3 grid(llb_ceil_div(N, BN), llb_ceil_div(M, BM));
    LLB_REQUIRE(grid.y <= 65535, "gemm: M=%d is too large for one launch", M);
    gemm_tile_kernel<TA, TW, TO, EPI><<<grid, 256, 0, stream>>>(a, w, b, out, residual, M, N, K);
    return llb_check_launch("gemm_tile");
}

template <typename TA, typename TW>
int dispatch_epilogue(int epi, const void* A, const void* W, const void* bias, void* out, float* residual, int M,
                      int N, int K, cudaStream_t s) {
    switch (epi) {
        case LLB_EPI_STORE: return launch<TA, TW, TA, LLB_EPI_STORE>(A, W, bias, out, residual, M, N, K, s);
        case LLB_EPI_STORE_F32: return launch<TA, TW, float, LLB_EPI_STORE_F32>(A, W, bias, out, residual, M, N, K, s);
        case LLB_EPI_RESIDUAL: return launch<TA, TW, float, LLB_EPI_RESIDUAL>(A, W, bias, out, residual, M, N, K, s);
        case LLB_EPI_SWIGLU: return launch<TA, TW, TA, LLB_EPI_SWIGLU>(A, W, bias, out, residual, M, N, K, s);
    }
    return llb_fail("gemm: unknown epilogue %d", epi);
}

}  // namespace

// A [M,K] (a_dtype), W [N,K] (w_dtype), bias [N] float or null.  `out` is [M,N] of a_dtype
// (STORE), [M,N] float (STORE_F32) or [M,N/2] of a_dtype (SWIGLU, N even); `residual` is
// [M,N] float (RESIDUAL).  Supported: (float,float), (bf16,bf16), (bf16 activations, float weights).
LLB_EXPORT int llb_gemm_simt(const void* A, int a_dtype, const void* W, const void* bias, int w_dtype, void* out,
                             float* residual, int epilogue, int M, int N, int K, cudaStream_t stream) {
    if (M == 0) return 0;
    LLB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    LLB_REQUIRE(epilogue != LLB_EPI_SWIGLU || N % 2 == 0, "gemm: SwiGLU epilogue needs an even N, got %d", N);
    LLB_REQUIRE(epilogue != LLB_EPI_RESIDUAL || residual != nullptr, "gemm: residual epilogue without residual");
    LLB_REQUIRE(epilogue == LLB_EPI_RESIDUAL || out != nullptr, "gemm: output pointer is null");
    if (a_dtype == LLB_F32 && w_dtype == LLB_F32)
        return dispatch_epilogue<float, float>(epilogue, A, W, bias, out, residual, M, N, K, stream);
    if (a_dtype == LLB_BF16 && w_dtype == LLB_BF16)
        return dispatch_epilogue<__nv_bfloat16, __nv_bfloat16>(epilogue, A, W, bias, out, residual, M, N, K, stream);
    if (a_dtype == LLB_BF16 && w_dtype == LLB_F32)
        return dispatch_epilogue<__nv_bfloat16, float>(epilogue, A, W, bias, out, residual, M, N, K, stream);
    return llb_fail("gemm: unsupported dtype pair activations=%d weights=%d", a_dtype, w_dtype);
}
