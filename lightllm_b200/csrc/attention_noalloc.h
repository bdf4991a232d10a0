// An entry point of the kernel library for callers that cannot allocate device memory.
//
// This function has no counterpart in the reference (wjb554/lightllm has no split-KV entry that
// works without a caller-provided or freshly allocated buffer); it exists for this library's users.
//
// Who needs it: code that runs where cudaMalloc is not allowed or not wanted.  Examples are a
// host thread that launches work while another stream is being captured into a CUDA graph (an
// allocation there is an error), a plug-in that was handed raw device pointers by a host
// application and must not touch the application's memory pools, and a real-time loop that may
// not take the allocator's lock.  Split-KV decode attention needs scratch memory for the partial
// results of the splits; the regular entry point (llb_paged_attention) takes that scratch from
// the caller.  This one keeps it inside the library instead.
//
// How: the scratch is one file-scope `static __device__` array of LLB_NOALLOC_SCRATCH_FLOATS
// floats (8 MiB), aligned to 256 bytes.  Every GPU on which the library's module gets loaded
// holds these 8 MiB until the process exits.  The first call with nsplit > 1 on a device looks up
// the array's device address (cudaGetSymbolAddress) and remembers it; make that first call before
// any stream capture begins.  No call allocates or frees anything, on the device or through any
// library.
//
// Limits and rules:
//   * with nsplit > 1, num_tiles * Hq * BQ * nsplit * (hd + 2) must not exceed
//     LLB_NOALLOC_SCRATCH_FLOATS, else the call fails with a message that states both numbers
//     and launches nothing.  A call with nsplit == 1 never touches the array: it has no size
//     limit and does not look up the array's address;
//   * all calls share the one array, and it keeps what the last call left there.  Nothing in it
//     has to start at zero: every split writes its whole partial (an empty split writes
//     m = -inf, l = 0) before the merge reads it;
//   * two calls that overlap on the GPU (different streams, or graph branches) race on the
//     array; callers must order them.
//
// Arguments and results are those of llb_paged_attention (attention_simt.cu) without `scratch`.
#pragma once
#include <cuda_runtime.h>

#define LLB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or a negative code with the message available from llb_last_error().
int llb_paged_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                                const int* tile_span, const int* tile_q0, int num_tiles, const int* span_row,
                                const int* span_len, const int* span_pos, const int* block_table, int max_pages,
                                int page_size, int Hq, int Hkv, int hd, int window, float scale, int BQ, int nsplit,
                                cudaStream_t stream);

// The size of the built-in scratch in floats (LLB_NOALLOC_SCRATCH_FLOATS), for callers that plan their splits.
long long llb_noalloc_scratch_floats(void);

#ifdef __cplusplus
}
#endif
