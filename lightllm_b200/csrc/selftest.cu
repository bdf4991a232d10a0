// A self-test of the way every tensor-core kernel of this library gives up on a wait: a block whose roles wait on
// a barrier that nothing ever completes, with a short time limit.  The role whose limit runs out raises the block's
// abort flag, the other role sees the flag and falls through, the block reports through the error flag in global
// memory, frees its tensor memory and returns; the context stays usable.  Nothing traps, and no wait is unbounded.
// The reference has no counterpart: its kernels have no waits, and it reports CUDA faults by printing
// (src/engine/engine_server.cpp:1427-1432).
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
}  // namespace

// Launches one block whose waits run out after `limit_cycles` SM cycles (a million is about half a millisecond).
// error_flag: the int that ops.check_async_errors reads; trace: two ints (or null) that receive 2 for each role that
// left its wait without the barrier having completed.
LLB_EXPORT int llb_selftest_wait_expires(int* error_flag, int* trace, long long limit_cycles, cudaStream_t stream) {
    LLB_REQUIRE(error_flag != nullptr && limit_cycles > 0 && limit_cycles <= 200000000ll,
                "selftest: the limit must lie between 1 and 2e8 cycles");
    wait_expires_kernel<<<1, 96, 0, stream>>>(error_flag, trace, limit_cycles);
    return llb_check_launch("selftest_wait_expires");
}
