// Token embedding gather into the float residual stream.
//
// out[t, :] = table[ids[t], :]  (src/ops/embedding.cu:9-18).  The reference replaces an id
// outside [0, V) by 0; here such an id writes zeros and raises the device error flag, which
// the engine reports as an error.
#include "common.cuh"

template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                 float* __restrict__ out, int D, int V, int* __restrict__ err) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0 && err) atomicExch(err, 1);
    const TW* row = table + (size_t)(ok ? id : 0) * D;
    float* o = out + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = ok ? llb_to_float(row[d]) : 0.0f;
}

// ids [T] int32, table [V, D] (float or bf16), out [T, D] float, err: one int or null.
LLB_EXPORT int llb_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int D,
                             int V, int* err, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && V > 0, "embedding: bad sizes T=%d D=%d V=%d", T, D, V);
    const int threads = D >= 256 ? 256 : 128;
    if (table_dtype == LLB_F32)
        embedding_kernel<float><<<T, threads, 0, stream>>>(ids, (const float*)table, out, D, V, err);
    else if (table_dtype == LLB_BF16)
        embedding_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, D, V, err);
    else
        return llb_fail("embedding: unknown table dtype %d", table_dtype);
    return llb_check_launch("embedding");
}
