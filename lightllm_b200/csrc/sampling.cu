// Token selection on the device: greedy argmax, and temperature sampling with the top-k,
// top-p and min-p filters, one block per row of logits.
//
// Order of operations as src/ops/sampling.cpp:22-335: temperature < 1e-5 is greedy (first
// index of the strictly largest logit, :36-59); else logits * 1/max(T, 1e-8) (:81-84); top-k
// keeps values >= the k-th largest, ties kept (:91-137); softmax with the maximum subtracted
// (:143-193); top-p keeps the most probable tokens until their mass reaches p and
// renormalises (:198-243); min-p drops probabilities below min_p * max and renormalises
// (:248-278); the draw is the first index whose cumulative mass reaches the uniform number,
// skipping entries without mass (:284-334).  The reference sorts on the CPU; here each filter
// is a threshold on the value found by a bitwise search over the float's ordered bit pattern
// (32 counting passes), so a tie at the top-p boundary keeps all tied tokens where the
// reference's sort keeps an unspecified subset.  The uniform number comes from the caller
// (one per row), so the random stream belongs to the request, not to the kernel.
#include "common.cuh"

#include <cooperative_groups.h>
#include <math.h>

namespace cg = cooperative_groups;

namespace {

constexpr int THREADS = 1024;

// Order-preserving map from float to unsigned: a < b  <=>  key(a) < key(b).
__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ float block_sum(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = llb_warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.0f;
    if (w == 0) {
        t = llb_warp_sum(t);
        if (lane == 0) sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}

__device__ float block_max(float v, float* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = llb_warp_max(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float t = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : -INFINITY;
    if (w == 0) {
        t = llb_warp_max(t);
        if (lane == 0) sh[32] = t;
    }
    __syncthreads();
    return sh[32];
}

// First index of the largest value of a row.
// ``none`` is what a row without any value above -inf (or with NaNs only) gives.
__device__ int block_argmax(const float* x, int V, float* shf, int* shi, int none = 0) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best) { best = v; bi = i; }   // ascending i per thread keeps its first maximum
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { shf[w] = best; shi[w] = bi; }
    __syncthreads();
    if (w == 0) {
        best = lane < (blockDim.x >> 5) ? shf[lane] : -INFINITY;
        bi = lane < (blockDim.x >> 5) ? shi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) shi[32] = (bi == 0x7fffffff) ? none : bi;
    }
    __syncthreads();
    return shi[32];
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int V, long long stride,
                                                         int* __restrict__ out) {
    __shared__ float shf[33];
    __shared__ int shi[33];
    const int r = blockIdx.x;
    const int idx = block_argmax(logits + (size_t)r * stride, V, shf, shi);
    if (threadIdx.x == 0) out[r] = idx;
}

// The same over a long row, by many blocks: block (s, r) takes the s-th piece of row r and offers its first maximum to
// the row's slot as one 64-bit number (the value's ordered key above, 2^32 - 1 - index below: the larger value wins,
// among equal values the smaller index) with an atomic maximum.  The block that counts itself last on the row's
// counter writes the index and leaves slot and counter zero for the next launch.  A row without any value above
// -inf offers nothing and gets index 0, as in the one-block kernel.
constexpr int SPLIT_THREADS = 256;
constexpr int SPLIT_ELEMS = 4096;            // elements of a row per block

__global__ void __launch_bounds__(SPLIT_THREADS) argmax_split_kernel(const float* __restrict__ logits, int V, long long stride,
                                                                     unsigned long long* __restrict__ slots,
                                                                     int* __restrict__ counters, int* __restrict__ out) {
    __shared__ float shf[33];
    __shared__ int shi[33];
    const int r = blockIdx.y;
    const int begin = blockIdx.x * SPLIT_ELEMS;
    const int n = min(SPLIT_ELEMS, V - begin);
    const int idx = block_argmax(logits + (size_t)r * stride + begin, n, shf, shi, /*none=*/-1);
    if (threadIdx.x == 0) {
        if (idx >= 0) {
            const float v = logits[(size_t)r * stride + begin + idx] + 0.0f;        // -0 counts as +0
            const unsigned long long offer = ((unsigned long long)ordered_key(v) << 32) |
                                             (unsigned long long)(0xffffffffu - (unsigned)(begin + idx));
            atomicMax(slots + r, offer);
        }
        __threadfence();
        if (atomicAdd(counters + r, 1) == (int)gridDim.x - 1) {
            __threadfence();
            const unsigned long long best = atomicExch(slots + r, 0ull);
            out[r] = best == 0ull ? 0 : (int)(0xffffffffu - (unsigned)(best & 0xffffffffull));
            atomicExch(counters + r, 0);
        }
    }
}

// params per row: temperature, top_p, min_p, uniform; top_k per row as int.
__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int V, long long stride,
                                                         const float* __restrict__ temperature,
                                                         const int* __restrict__ top_k,
                                                         const float* __restrict__ top_p,
                                                         const float* __restrict__ min_p,
                                                         const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float shf[33];
    __shared__ int shi[33];
    __shared__ float chunk_sum[THREADS];
    const int r = blockIdx.x;
    const float* x = logits + (size_t)r * stride;
    const float temp = temperature[r];
    if (temp < 1e-5f) {
        const int idx = block_argmax(x, V, shf, shi);
        if (threadIdx.x == 0) out[r] = idx;
        return;
    }
    const float inv_temp = 1.0f / fmaxf(temp, 1e-8f);
    const int k = top_k ? top_k[r] : 0;
    const float tp = top_p ? top_p[r] : 1.0f;
    const float mp = min_p ? min_p[r] : 0.0f;

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, x[i] * inv_temp);
    mx = block_max(mx, shf);
    if (mx == -INFINITY || !(mx == mx)) {  // every logit is -inf, or NaN: fall back to argmax
        const int idx = block_argmax(x, V, shf, shi);
        if (threadIdx.x == 0) out[r] = idx;
        return;
    }

    // top-k: key of the k-th largest scaled logit (largest K with count(key >= K) >= k).
    unsigned key_k = 0u;
    if (k > 0 && k < V) {
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = key_k | (1u << bit);
            float cnt = 0.0f;
            for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += ordered_key(x[i] * inv_temp) >= cand ? 1.0f : 0.0f;
            cnt = block_sum(cnt, shf);
            if (cnt >= (float)k) key_k = cand;
        }
    }
    // e_i = exp(x_i/T - max) of the kept entries; everything below is in terms of e (max e = 1).
    auto e_of = [&](int i) -> float {
        const float s = x[i] * inv_temp;
        if (ordered_key(s) < key_k) return 0.0f;
        return expf(s - mx);
    };
    float z = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) z += e_of(i);
    z = block_sum(z, shf);

    // top-p: largest threshold on e whose kept mass still reaches p * z.
    unsigned key_p = 0u;
    if (tp < 1.0f) {
        const float need = tp * z;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = key_p | (1u << bit);
            float mass = 0.0f;
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float e = e_of(i);
                if (e > 0.0f && ordered_key(e) >= cand) mass += e;
            }
            mass = block_sum(mass, shf);
            if (mass >= need) key_p = cand;
        }
    }
    // min-p: probabilities below min_p * max probability are dropped; max e is 1.
    const float e_min = mp > 0.0f ? mp : 0.0f;
    auto kept_of = [&](int i) -> float {
        const float e = e_of(i);
        if (e <= 0.0f || ordered_key(e) < key_p || e < e_min) return 0.0f;
        return e;
    };

    // Draw: first index whose running mass reaches u * total.  Threads own contiguous chunks.
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int begin = min(V, (int)threadIdx.x * per), end = min(V, begin + per);
    float mine = 0.0f;
    for (int i = begin; i < end; ++i) mine += kept_of(i);
    chunk_sum[threadIdx.x] = mine;
    const float total = block_sum(mine, shf);   // contains the barriers that publish chunk_sum
    if (threadIdx.x == 0) {
        int choice = -1;
        if (total > 0.0f) {
            const float target = uniform[r] * total;
            float run = 0.0f;
            int c = 0;
            for (; c < (int)blockDim.x; ++c) {
                if (chunk_sum[c] > 0.0f && run + chunk_sum[c] >= target) break;
                run += chunk_sum[c];
            }
            if (c < (int)blockDim.x) {
                const int b = min(V, c * per), e = min(V, b + per);
                int last_mass = -1;
                for (int i = b; i < e; ++i) {
                    const float m = kept_of(i);
                    if (m > 0.0f) {
                        last_mass = i;
                        run += m;
                        if (run >= target) { choice = i; break; }
                    }
                }
                if (choice < 0) choice = last_mass;
            }
            if (choice < 0) {  // rounding left the target above the total: last entry with mass
                for (int i = V - 1; i >= 0 && choice < 0; --i)
                    if (kept_of(i) > 0.0f) choice = i;
            }
        }
        shi[32] = choice;
    }
    __syncthreads();
    int choice = shi[32];
    if (choice < 0) choice = block_argmax(x, V, shf, shi);   // uniform over the block
    if (threadIdx.x == 0) out[r] = choice;
}

// ---------------------------------------------------------------------------------------------------------------
// The same selection for long rows (a vocabulary of 150,000), by a cluster of CL blocks per row.  The one-block
// kernel walks the whole row in memory for every counting pass (32 per filter, each with an exponential per
// element): 0.2 ms for temperature alone and 2 ms with all filters at this size.  Here block b of the cluster keeps
// its part of the row in shared memory (first the scaled logits, then their exponentials, then the kept masses), so a
// pass is a walk over shared memory, a reduction in the block and one exchange in the cluster: every block
// publishes its partial result in its own shared memory, the cluster meets on its barrier, and every block adds up
// all parts in rank order, so that all blocks hold the same bits and take the same branches.  The published
// values alternate between two places: a block writes the place of pass n+2 only after the barrier of pass n+1,
// which every block reaches only after it has read pass n.
constexpr int CL = 8;
constexpr int CL_THREADS = 512;

struct ClusterExchange {
    float f[2];
    int i[2];
    int turn;
};

__device__ __forceinline__ float cluster_sum(cg::cluster_group& cl, ClusterExchange* xc, float block_value) {
    const int t = xc->turn;
    if (threadIdx.x == 0) xc->f[t] = block_value;
    cl.sync();
    float total = 0.0f;
#pragma unroll
    for (int b = 0; b < CL; ++b) total += cl.map_shared_rank(xc, b)->f[t];
    __syncthreads();                       // everyone has read `turn` before it moves
    if (threadIdx.x == 0) xc->turn = t ^ 1;
    __syncthreads();
    return total;
}

__device__ __forceinline__ float cluster_max(cg::cluster_group& cl, ClusterExchange* xc, float block_value) {
    const int t = xc->turn;
    if (threadIdx.x == 0) xc->f[t] = block_value;
    cl.sync();
    float best = -INFINITY;
#pragma unroll
    for (int b = 0; b < CL; ++b) best = fmaxf(best, cl.map_shared_rank(xc, b)->f[t]);
    __syncthreads();
    if (threadIdx.x == 0) xc->turn = t ^ 1;
    __syncthreads();
    return best;
}

// First index of the largest value of the whole row (0 if nothing lies above -inf), the same in every block.
__device__ int cluster_argmax(cg::cluster_group& cl, ClusterExchange* xc, const float* x, int begin, int n, float* shf,
                              int* shi) {
    const int local = n > 0 ? block_argmax(x + begin, n, shf, shi, -1) : -1;
    const int t = xc->turn;
    if (threadIdx.x == 0) {
        xc->f[t] = local >= 0 ? x[begin + local] : -INFINITY;
        xc->i[t] = local >= 0 ? begin + local : -1;
    }
    cl.sync();
    float best = -INFINITY;
    int at = -1;
#pragma unroll
    for (int b = 0; b < CL; ++b) {          // ascending ranks hold ascending indices: a later equal value does not win
        const ClusterExchange* o = cl.map_shared_rank(xc, b);
        const int oi = o->i[t];
        const float ov = o->f[t];
        if (oi >= 0 && (at < 0 || ov > best)) { best = ov; at = oi; }
    }
    __syncthreads();
    if (threadIdx.x == 0) xc->turn = t ^ 1;
    __syncthreads();
    return at < 0 ? 0 : at;
}

__global__ void __launch_bounds__(CL_THREADS) sample_cluster_kernel(const float* __restrict__ logits, int V, long long stride,
                                                                    int part, const float* __restrict__ temperature,
                                                                    const int* __restrict__ top_k,
                                                                    const float* __restrict__ top_p,
                                                                    const float* __restrict__ min_p,
                                                                    const float* __restrict__ uniform,
                                                                    int* __restrict__ out) {
    extern __shared__ float mine[];            // this block's `part` elements of the row
    __shared__ float shf[33];
    __shared__ int shi[33];
    __shared__ float chunk_sum[CL_THREADS];
    __shared__ ClusterExchange xc;
    cg::cluster_group cl = cg::this_cluster();
    const int rank = (int)cl.block_rank();
    const int r = blockIdx.y;
    const float* x = logits + (size_t)r * stride;
    const int begin = min(V, rank * part);
    const int n = min(part, V - begin);          // may be 0 for the last ranks of a short row
    if (threadIdx.x == 0) xc.turn = 0;
    __syncthreads();

    const float temp = temperature[r];
    if (temp < 1e-5f) {
        const int idx = cluster_argmax(cl, &xc, x, begin, n, shf, shi);
        if (rank == 0 && threadIdx.x == 0) out[r] = idx;
        cl.sync();                               // no block leaves while another may still read its shared memory
        return;
    }
    const float inv_temp = 1.0f / fmaxf(temp, 1e-8f);
    const int k = top_k ? top_k[r] : 0;
    const float tp = top_p ? top_p[r] : 1.0f;
    const float mp = min_p ? min_p[r] : 0.0f;

    float mx = -INFINITY;
    for (int i = threadIdx.x; i < n; i += CL_THREADS) {
        const float v = x[begin + i] * inv_temp;
        mine[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = cluster_max(cl, &xc, block_max(mx, shf));
    if (mx == -INFINITY || !(mx == mx)) {        // every logit is -inf, or NaN: fall back to argmax
        const int idx = cluster_argmax(cl, &xc, x, begin, n, shf, shi);
        if (rank == 0 && threadIdx.x == 0) out[r] = idx;
        cl.sync();
        return;
    }

    // top-k: key of the k-th largest scaled logit (largest K with count(key >= K) >= k).
    unsigned key_k = 0u;
    if (k > 0 && k < V) {
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = key_k | (1u << bit);
            float cnt = 0.0f;
            for (int i = threadIdx.x; i < n; i += CL_THREADS) cnt += ordered_key(mine[i]) >= cand ? 1.0f : 0.0f;
            cnt = cluster_sum(cl, &xc, block_sum(cnt, shf));
            if (cnt >= (float)k) key_k = cand;
        }
    }
    // e_i = exp(x_i/T - max) of the kept entries; everything below is in terms of e (max e = 1).
    float z = 0.0f;
    for (int i = threadIdx.x; i < n; i += CL_THREADS) {
        const float v = mine[i];
        const float e = ordered_key(v) < key_k ? 0.0f : expf(v - mx);
        mine[i] = e;
        z += e;
    }
    z = cluster_sum(cl, &xc, block_sum(z, shf));

    // top-p: largest threshold on e whose kept mass still reaches p * z.
    unsigned key_p = 0u;
    if (tp < 1.0f) {
        const float need = tp * z;
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned cand = key_p | (1u << bit);
            float mass = 0.0f;
            for (int i = threadIdx.x; i < n; i += CL_THREADS) {
                const float e = mine[i];
                if (e > 0.0f && ordered_key(e) >= cand) mass += e;
            }
            mass = cluster_sum(cl, &xc, block_sum(mass, shf));
            if (mass >= need) key_p = cand;
        }
    }
    // min-p: probabilities below min_p * max probability are dropped; max e is 1.  What is kept stays in `mine`.
    const float e_min = mp > 0.0f ? mp : 0.0f;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += CL_THREADS) {
        const float e = mine[i];
        if (e <= 0.0f || ordered_key(e) < key_p || e < e_min) mine[i] = 0.0f;
    }
    __syncthreads();

    // Draw: first index whose running mass reaches u * total.  Threads own contiguous chunks of their block's part,
    // blocks contiguous parts of the row.
    const int per = (part + CL_THREADS - 1) / CL_THREADS;
    const int cb = min(n, (int)threadIdx.x * per), ce = min(n, cb + per);
    float own = 0.0f;
    for (int i = cb; i < ce; ++i) own += mine[i];
    chunk_sum[threadIdx.x] = own;
    const float block_total = block_sum(own, shf);      // contains the barriers that publish chunk_sum
    // every block learns every block's total (the same exchange as cluster_sum, but the parts are kept)
    const int t = xc.turn;
    if (threadIdx.x == 0) xc.f[t] = block_total;
    cl.sync();
    float totals[CL];
    float total = 0.0f;
#pragma unroll
    for (int b = 0; b < CL; ++b) {
        totals[b] = cl.map_shared_rank(&xc, b)->f[t];
        total += totals[b];
    }
    __syncthreads();
    if (threadIdx.x == 0) xc.turn = t ^ 1;
    __syncthreads();
    if (!(total > 0.0f)) {                               // nothing kept (cannot happen with max e = 1, but stay safe)
        const int idx = cluster_argmax(cl, &xc, x, begin, n, shf, shi);
        if (rank == 0 && threadIdx.x == 0) out[r] = idx;
        cl.sync();
        return;
    }
    // the block in whose part the running mass reaches the target; if rounding leaves the target above the total,
    // the last block with mass, which then takes its last entry with mass
    const float target = uniform[r] * total;
    float run = 0.0f;
    int chosen = -1, last_with_mass = -1;
#pragma unroll
    for (int b = 0; b < CL; ++b) {
        if (chosen >= 0) continue;
        if (totals[b] > 0.0f) {
            last_with_mass = b;
            if (run + totals[b] >= target) { chosen = b; continue; }
        }
        run += totals[b];
    }
    const bool overshoot = chosen < 0;
    if (overshoot) chosen = last_with_mass;
    if (rank == chosen && threadIdx.x == 0) {
        int choice = -1;
        if (!overshoot) {
            int c = 0;
            for (; c < CL_THREADS; ++c) {
                if (chunk_sum[c] > 0.0f && run + chunk_sum[c] >= target) break;
                run += chunk_sum[c];
            }
            if (c < CL_THREADS) {
                const int b0 = min(n, c * per), e0 = min(n, b0 + per);
                int last_mass = -1;
                for (int i = b0; i < e0; ++i) {
                    const float m = mine[i];
                    if (m > 0.0f) {
                        last_mass = i;
                        run += m;
                        if (run >= target) { choice = i; break; }
                    }
                }
                if (choice < 0) choice = last_mass;
            }
        }
        if (choice < 0) {      // rounding left the target above the running mass: this block's last entry with mass
            for (int i = n - 1; i >= 0 && choice < 0; --i)
                if (mine[i] > 0.0f) choice = i;
        }
        out[r] = begin + choice;      // totals[chosen] > 0, so the block has an entry with mass
    }
    cl.sync();
}

}  // namespace

// logits [R, V] float with row stride `stride` elements; out [R] int32.  scratch (or null): 3 * scratch_rows ints,
// 8-byte aligned, zero on entry and left zero; with it, rows of 4 * 4096 elements or more are shared among blocks.
LLB_EXPORT int llb_argmax(const float* logits, int R, int V, long long stride, int* out, int* scratch, int scratch_rows,
                          cudaStream_t stream) {
    if (R == 0) return 0;
    LLB_REQUIRE(R > 0 && V > 0 && stride >= V, "argmax: bad sizes R=%d V=%d stride=%lld", R, V, stride);
    if (scratch && R <= scratch_rows && R <= 65535 && V >= 4 * SPLIT_ELEMS && (uintptr_t)scratch % 8 == 0) {
        unsigned long long* slots = (unsigned long long*)scratch;
        int* counters = scratch + 2 * (size_t)scratch_rows;
        argmax_split_kernel<<<dim3(llb_ceil_div(V, SPLIT_ELEMS), R), SPLIT_THREADS, 0, stream>>>(logits, V, stride, slots,
                                                                                               counters, out);
        return llb_check_launch("argmax");
    }
    argmax_kernel<<<R, THREADS, 0, stream>>>(logits, V, stride, out);
    return llb_check_launch("argmax");
}

// Per row: temperature [R]; top_k [R] int (0 = off) or null; top_p [R] (1 = off) or null;
// min_p [R] (0 = off) or null; uniform [R] in [0, 1).  out [R] int32.
LLB_EXPORT int llb_sample(const float* logits, int R, int V, long long stride, const float* temperature,
                          const int* top_k, const float* top_p, const float* min_p, const float* uniform, int* out,
                          cudaStream_t stream) {
    if (R == 0) return 0;
    LLB_REQUIRE(R > 0 && V > 0 && stride >= V, "sample: bad sizes R=%d V=%d stride=%lld", R, V, stride);
    LLB_REQUIRE(temperature && uniform && out, "sample: null argument");
    // long rows: a cluster of blocks per row, each with its part of the row in shared memory
    const int part = llb_ceil_div(V, CL);
    const size_t smem = (size_t)part * sizeof(float);
    if (V >= 8192 && smem <= 216 * 1024 && R <= 65535) {
        static size_t configured = 0;
        if (smem > configured) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return llb_fail("sample: cannot opt in to %zu bytes of shared memory: %s", smem,
                                                  cudaGetErrorString(e));
            configured = smem;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(CL, R);
        cfg.blockDim = dim3(CL_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, V, stride, part, temperature, top_k, top_p,
                                           min_p, uniform, out);
        if (e != cudaSuccess) return llb_fail("sample: launch failed: %s", cudaGetErrorString(e));
        return llb_check_launch("sample");
    }
    sample_kernel<<<R, THREADS, 0, stream>>>(logits, V, stride, temperature, top_k, top_p, min_p, uniform, out);
    return llb_check_launch("sample");
}
