// Rotary position encoding of q and k, fused with the write of k and v into cache pages.
//
// Rotation (src/ops/rope.cu:54-59): for a pair (a, b) of one head, with angle = pos * inv_freq[i]:
//     a' = a*cos - b*sin,   b' = b*cos + a*sin
// NeoX pairing is (i, i + rotary_dim/2); interleaved pairing is (2i, 2i+1).  The reference's
// kernel rotates only one pair per head (its thread index doubles as the pair index,
// rope.cu:41-60); here every pair below rotary_dim is rotated and the rest passes through.
// The reference computes cos and sin on the host for every layer of every step
// (src/engine/engine_server.cpp:1553-1589); here they come from the position and a table of
// inverse frequencies inside the kernel, in float, with cosf/sinf (not the fast intrinsics).
//
// The cache row of a token is slot_mapping[t] = page * page_size + offset, so k and v land at
// pool[slot][kv_head][:] (layout [pages, page_size, kv_heads, head_dim] as
// src/kv_cache/block_allocator.cpp:24-27).  A negative slot writes nothing.
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                                     int rotary_dim, int interleaved, T* __restrict__ q_out,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hkv, int hd,
                                     int write_kv) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int qkv_stride = (Hq + 2 * Hkv) * hd;
    const T* row = qkv + (size_t)t * qkv_stride;
    const int slot = (write_kv && slot_mapping) ? slot_mapping[t] : -1;
    const int half = rotary_dim / 2;
    const int pairs_per_head = hd - half;  // `half` rotated pairs + (hd - rotary_dim) pass-through singles
    // Items: for q heads and k heads, one item per rotated pair and one per pass-through element.
    const int n_rot_items = (Hq + Hkv) * pairs_per_head;
    for (int it = threadIdx.x; it < n_rot_items; it += blockDim.x) {
        const int head = it / pairs_per_head;  // 0..Hq-1 are q heads, then k heads
        const int j = it - head * pairs_per_head;
        const T* src = row + (size_t)head * hd;
        T* dst;
        if (head < Hq) {
            dst = q_out + ((size_t)t * Hq + head) * hd;
        } else {
            if (slot < 0) continue;
            dst = k_cache + ((size_t)slot * Hkv + (head - Hq)) * hd;
        }
        if (j < half) {
            const int ia = interleaved ? 2 * j : j;
            const int ib = interleaved ? 2 * j + 1 : j + half;
            const float angle = (float)pos * inv_freq[j];
            const float c = cosf(angle), s = sinf(angle);
            const float a = llb_to_float(src[ia]), b = llb_to_float(src[ib]);
            dst[ia] = llb_from_float<T>(a * c - b * s);
            dst[ib] = llb_from_float<T>(b * c + a * s);
        } else {
            const int d = rotary_dim + (j - half);
            dst[d] = src[d];
        }
    }
    if (slot >= 0) {
        const T* vsrc = row + (size_t)(Hq + Hkv) * hd;
        T* vdst = v_cache + (size_t)slot * Hkv * hd;
        for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) vdst[i] = vsrc[i];
    }
}

// qkv [T, (Hq + 2*Hkv) * hd]; q_out [T, Hq*hd]; k_cache/v_cache [slots, Hkv, hd];
// inv_freq [rotary_dim/2] float (unused when rotary_dim == 0); write_kv = 0 leaves the cache alone.
LLB_EXPORT int llb_rope_kv_write(const void* qkv, int dtype, const int* positions, const int* slot_mapping,
                                 const float* inv_freq, int rotary_dim, int interleaved, void* q_out,
                                 void* k_cache, void* v_cache, int T, int Hq, int Hkv, int hd, int write_kv,
                                 cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && Hq > 0 && Hkv >= 0 && hd > 0, "rope_kv_write: bad sizes T=%d Hq=%d Hkv=%d hd=%d", T, Hq,
                Hkv, hd);
    LLB_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
                "rope_kv_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    LLB_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "rope_kv_write: inv_freq is null");
    const int threads = 256;
    if (dtype == LLB_F32)
        rope_kv_write_kernel<float><<<T, threads, 0, stream>>>(
            (const float*)qkv, positions, slot_mapping, inv_freq, rotary_dim, interleaved, (float*)q_out,
            (float*)k_cache, (float*)v_cache, Hq, Hkv, hd, write_kv);
    else if (dtype == LLB_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            (const __nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, rotary_dim, interleaved,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, hd, write_kv);
    else
        return llb_fail("rope_kv_write: unknown dtype %d", dtype);
    return llb_check_launch("rope_kv_write");
}

// cos and sin of pos * inv_freq for every token of a step and every rotary pair, computed once per
// step (the reference recomputes them on the host for every layer, src/engine/engine_server.cpp:1553-1589).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ table, int T, int half, int transposed) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * half) return;
    // token-major [T, half], or pair-major [half, T] (consecutive threads then walk along the tokens)
    const int t = transposed ? i % T : i / half;
    const int f = transposed ? i / T : i - t * half;
    const float angle = (float)positions[t] * inv_freq[f];
    table[i] = make_float2(cosf(angle), sinf(angle));
}

// table [T, half] of (cos, sin) pairs as float2, or [half, T] with transposed != 0.
LLB_EXPORT int llb_rope_table(const int* positions, const float* inv_freq, float* table, int T, int half,
                              int transposed, cudaStream_t stream) {
    if (T == 0 || half == 0) return 0;
    LLB_REQUIRE(T > 0 && half > 0 && positions && inv_freq && table, "rope_table: bad arguments");
    const int n = T * half;
    rope_table_kernel<<<llb_ceil_div(n, 256), 256, 0, stream>>>(positions, inv_freq, (float2*)table, T, half,
                                                                transposed ? 1 : 0);
    return llb_check_launch("rope_table");
}
