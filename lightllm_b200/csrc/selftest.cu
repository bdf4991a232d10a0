// A self-test of the way every tensor-core kernel of this library gives up on a wait: a block whose roles wait on
// a barrier that nothing ever completes, with a short time limit.  The role whose limit runs out raises the block's
// abort flag, the other role sees the flag and falls through, the block reports through the error flag in global
// memory, frees its tensor memory and returns; the context stays usable.  Nothing traps, and no wait is unbounded.
// The reference has no counterpart: its kernels have no waits, and it reports CUDA faults by printing
// (src/engine/engine_server.cpp:1427-1432).
#include <cuda_bf16.h>

#include "tcgen05_common.cuh"

namespace {
using namespace t5;

__global__ void __launch_bounds__(96) wait_expires_kernel(int* error_flag, int* trace, long long limit_cycles) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_s = 0;
        mbar_init_fence();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 32);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_flag = &abort_s;
    if (warp == 1 && lane == 0) {
        // the role whose own limit runs out
        const bool ok = mbar_wait_limit(&bar, 0, abort_flag, limit_cycles);
        if (trace) trace[0] = ok ? 1 : 2;
    } else if (warp == 2 && lane == 0) {
        // a role with the library's ordinary limit (seconds): it must leave because the other role gave up
        const bool ok = mbar_wait(&bar, 0, abort_flag);
        if (trace) trace[1] = ok ? 1 : 2;
    }
    tc_fence_before();
    __syncthreads();
    if (abort_s && threadIdx.x == 0 && error_flag) atomicExch(error_flag, 6);
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 32);
    }
}
// What issuing tcgen05.mma costs the issuing thread, alone and beside busy warps.  One block: warp `issuer` issues
// `iters` groups of four 128 x N x 16 MMAs (A from shared memory, or from tensor memory when a_tmem) back to back, then
// one commit, and waits for it; `neighbours` other warps (from warp 0 on, so one or two per scheduler) meanwhile run
// either 16 independent FMA chains each (kind 1: a stream that never stalls) or a softmax-like loop (kind 2: read 64
// columns of tensor memory, 64 exponentials, pack, write 32 columns back).  out[0] = cycles for all MMAs to be issued,
// out[1] = cycles of the commit, out[2] = cycles until the commit arrives.  The operands are zeros; only time matters.
template <int N, bool A_TMEM>
__global__ void __launch_bounds__(384) mma_issue_kernel(long long* out, int iters, int issuer, int neighbours, int kind) {
    __shared__ __align__(1024) uint8_t a_s[128 * 128];
    __shared__ __align__(1024) uint8_t b_s[128 * 128];
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
    __shared__ volatile int issued_s;         // the neighbours stay busy until the issuer is through (or their own limit)
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 128 * 128 / 4; i += blockDim.x) {
        reinterpret_cast<uint32_t*>(a_s)[i] = 0;
        reinterpret_cast<uint32_t*>(b_s)[i] = 0;
    }
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_s = 0;
        issued_s = 0;
        mbar_init_fence();
    }
    if (warp == 0) tmem_alloc(&tmem_slot, 256);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    constexpr uint32_t IDESC = idesc_bf16(128, N, 0);
    if (warp == issuer) {
        const long long t0 = clock64();
        if (lane == 0) {
            for (int it = 0; it < iters; ++it) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t db = desc_kmajor(smem_u32(b_s) + k * 32);
                    if (A_TMEM) {
                        asm volatile(
                            "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                            ::"r"(tmem), "r"(tmem + 128 + k * 8), "l"(db), "r"(IDESC), "r"(k > 0 ? 1u : 0u) : "memory");
                    } else {
                        umma_bf16(tmem, desc_kmajor(smem_u32(a_s) + k * 32), db, IDESC, k > 0 ? 1u : 0u);
                    }
                }
            }
        }
        __syncwarp();
        const long long t1 = clock64();
        issued_s = 1;
        if (lane == 0) umma_commit(&bar);
        __syncwarp();
        const long long t2 = clock64();
        mbar_wait(&bar, 0, &abort_s);
        const long long t3 = clock64();
        if (lane == 0) {
            out[0] = t1 - t0;
            out[1] = t2 - t1;
            out[2] = t3 - t2;
        }
    } else if (warp < neighbours && kind == 1) {
        float x[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = threadIdx.x * 0.001f + j;
        for (int i = 0; i < 64 * iters && !issued_s; ++i) {
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int j = 0; j < 16; ++j) x[j] = fmaf(x[j], 1.0001f, 0.5f);
        }
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) a += x[j];
        if (a == 123.456f) out[3] = 1;
    } else if (warp < neighbours && kind == 2) {
        const uint32_t tl = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        float acc = 0.0f;
        for (int i = 0; i < 4 * iters && !issued_s; ++i) {
            uint32_t a[32], b[32], w[32];
            tmem_ld32_nowait(tl, a);
            tmem_ld32_nowait(tl + 32, b);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                float p0, p1, p2, p3;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(__uint_as_float(a[2 * e]) * 0.1f));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(__uint_as_float(a[2 * e + 1]) * 0.1f));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p2) : "f"(__uint_as_float(b[2 * e]) * 0.1f));
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p3) : "f"(__uint_as_float(b[2 * e + 1]) * 0.1f));
                acc += p0 + p1 + p2 + p3;
                const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1), g = __floats2bfloat162_rn(p2, p3);
                w[e] = *reinterpret_cast<const uint32_t*>(&h);
                w[16 + e] = *reinterpret_cast<const uint32_t*>(&g);
            }
            // columns 200..231: beside the accumulator (0..N-1 <= 127) and the A operand (128..159)
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
                "%15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                ::"r"(tl + 200), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]),
                  "r"(w[8]), "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15]), "r"(w[16]),
                  "r"(w[17]), "r"(w[18]), "r"(w[19]), "r"(w[20]), "r"(w[21]), "r"(w[22]), "r"(w[23]), "r"(w[24]), "r"(w[25]),
                  "r"(w[26]), "r"(w[27]), "r"(w[28]), "r"(w[29]), "r"(w[30]), "r"(w[31])
                : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        if (acc == 123.456f) out[3] = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
}
}  // namespace

// The microbenchmark above: n in {16, 64, 128} accumulator columns, `neighbours` in 0..8 busy warps of `kind` (1: FMA
// chains, 2: softmax-like), issuing warp 8.  out: three long longs on the device.
LLB_EXPORT int llb_selftest_mma_issue(long long* out, int n, int a_tmem, int neighbours, int kind, int iters,
                                      cudaStream_t stream) {
    LLB_REQUIRE(out != nullptr && (n == 16 || n == 64 || n == 128) && neighbours >= 0 && neighbours <= 8 &&
                (kind == 1 || kind == 2 || neighbours == 0) && iters > 0 && iters <= 4096,
                "selftest_mma_issue: n must be 16, 64 or 128, at most 8 neighbours of kind 1 or 2, at most 4096 iterations");
    if (a_tmem) {
        if (n == 16) mma_issue_kernel<16, true><<<1, 384, 0, stream>>>(out, iters, 8, neighbours, kind);
        else if (n == 64) mma_issue_kernel<64, true><<<1, 384, 0, stream>>>(out, iters, 8, neighbours, kind);
        else mma_issue_kernel<128, true><<<1, 384, 0, stream>>>(out, iters, 8, neighbours, kind);
    } else {
        if (n == 16) mma_issue_kernel<16, false><<<1, 384, 0, stream>>>(out, iters, 8, neighbours, kind);
        else if (n == 64) mma_issue_kernel<64, false><<<1, 384, 0, stream>>>(out, iters, 8, neighbours, kind);
        else mma_issue_kernel<128, false><<<1, 384, 0, stream>>>(out, iters, 8, neighbours, kind);
    }
    return llb_check_launch("selftest_mma_issue");
}

// Launches one block whose waits run out after `limit_cycles` SM cycles (a million is about half a millisecond).
// error_flag: the int that ops.check_async_errors reads; trace: two ints (or null) that receive 2 for each role that
// left its wait without the barrier having completed.
LLB_EXPORT int llb_selftest_wait_expires(int* error_flag, int* trace, long long limit_cycles, cudaStream_t stream) {
    LLB_REQUIRE(error_flag != nullptr && limit_cycles > 0 && limit_cycles <= 200000000ll,
                "selftest: the limit must lie between 1 and 2e8 cycles");
    wait_expires_kernel<<<1, 96, 0, stream>>>(error_flag, trace, limit_cycles);
    return llb_check_launch("selftest_wait_expires");
}
