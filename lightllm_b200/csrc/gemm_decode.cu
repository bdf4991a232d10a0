// The contraction of the decode step (at most 64 rows) on the tensor cores, fused with what stands
// before and after it so that a layer needs five launches instead of nine:
//
//   prologue NORM      the B operand is RMSNorm(residual) * weight, built by the block itself in shared
//                      memory (src/ops/norm.cu:19-55), instead of a separate norm kernel;
//   epilogue ROPE_KV   bias, rotary positions on q and k (src/ops/rope.cu:54-59, every pair), q to its
//                      buffer, k and v into their cache pages (src/kv_cache/paged_attention.cu:1150-1163);
//   epilogue SWIGLU    SiLU(gate) * up on interleaved weight rows (src/engine/engine_server.cpp:1875-1878);
//   epilogue RESIDUAL  adds into the float residual stream, split-K by atomic adds (engine_server.cpp:1870-1871);
//   epilogue STORE_F32 float output (the head's logits).
//
// The weights take the MMA's 128-row A role and stream through a TMA ring; the few activation rows are
// the B operand (BN = 16, 32 or 64 columns of tensor memory).  Every launch is a programmatic dependent
// launch: a block initialises its barriers, allocates tensor memory and already requests its first weight
// tiles while the kernel before it is still running, and only then waits for that kernel
// (griddepcontrol.wait) before it reads activations or writes anything.  Waits on mbarriers are bounded
// in time as in the other tensor-core kernels.
#include <utility>

#include "tcgen05_common.cuh"

namespace {

using namespace t5;

constexpr int TILE_M = 128;
constexpr int TILE_K = 64;
// Depth of the TMA ring: a block streams its weights at (bytes in flight) / latency.  Grids of a few blocks
// get a deep ring (8 stages, one block per SM); grids of many blocks (the head) a short one (4 stages), so
// that two blocks share an SM.
constexpr int DEEP = 8, SHALLOW = 4;
constexpr int NUM_THREADS = 192;
constexpr uint32_t A_BYTES = TILE_M * TILE_K * 2;

enum { DEPI_STORE_F32 = 1, DEPI_RESIDUAL = 2, DEPI_SWIGLU = 3, DEPI_ROPE_KV = 4 };

struct DecodeGemmParams {
    // NORM prologue
    const float* x;            // [*, K] float residual rows
    const int* x_rows;         // row r of the operand is x[x_rows[r]], or null for x[r]
    const void* norm_w;        // [K]
    int norm_w_bf16;
    float eps;
    // common
    const float* bias;         // [N] or null
    void* out;                 // SWIGLU: bf16 [M, N/2]; STORE_F32: float [M, N]
    float* residual;           // RESIDUAL: [M, N]
    int M, N, K, num_kb, kb_per_split;
    // ROPE_KV epilogue
    const int* slot_mapping;   // [M] cache row of each token, or null: nothing is written to the cache
    const float2* rope_table;  // [M, rotary_dim / 2] of (cos, sin) of pos * inv_freq
    int rotary_dim, interleaved, Hq, Hkv, hd;
    __nv_bfloat16* q_out;      // [M, Hq * hd]
    __nv_bfloat16* k_cache;    // [slots, Hkv, hd]
    __nv_bfloat16* v_cache;
    // split-K with a fused epilogue: partial sums meet in acc_scratch [BN, N] (zero between launches),
    // counters[n-tile] counts the splits that have arrived; the last one runs the epilogue and cleans up
    float* acc_scratch;
    int* counters;
    int* error_flag;
};

// How the rotary epilogue treats one output feature n (row `row` of the block's tile): whether it is rotated, with
// which row of the tile it pairs, which frequency it uses, and whether it is the pair's first member.
struct RopeRow {
    bool rotate, first;
    int partner, fi;
};
__device__ __forceinline__ RopeRow rope_row(const DecodeGemmParams& p, int n, int row) {
    RopeRow r;
    const int q_end = p.Hq * p.hd, k_end = q_end + p.Hkv * p.hd;
    const int head_row = n % p.hd;                    // q, k and v sections are multiples of hd
    const int half = p.rotary_dim / 2;
    r.rotate = n < p.N && n < k_end && head_row < p.rotary_dim;
    r.partner = row;
    r.fi = 0;
    r.first = true;
    if (r.rotate) {
        if (p.interleaved) { r.first = (head_row & 1) == 0; r.partner = r.first ? row + 1 : row - 1; r.fi = head_row >> 1; }
        else { r.first = head_row < half; r.partner = r.first ? row + half : row - half; r.fi = r.first ? head_row : head_row - half; }
    }
    return r;
}
// (cos, sin) and cache rows of tokens m0 .. m0+15 for that feature; the loads do not depend on each other.
__device__ __forceinline__ void rope_fetch(const DecodeGemmParams& p, const RopeRow& r, int n, int m0, float2 (&cs)[16],
                                           int (&slot)[16]) {
    const int half = p.rotary_dim / 2;
    const bool cached = n < p.N && n >= p.Hq * p.hd && p.slot_mapping != nullptr;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int m = m0 + j;
        cs[j] = (r.rotate && m < p.M) ? __ldg(p.rope_table + (size_t)m * half + r.fi) : make_float2(1.0f, 0.0f);
        slot[j] = (cached && m < p.M) ? __ldg(p.slot_mapping + m) : -1;
    }
}

template <int BN, int EPI, bool NORM, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const DecodeGemmParams p) {
    constexpr uint32_t B_BYTES = BN * TILE_K * 2;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    __shared__ __align__(8) uint64_t full_bar[8];
    __shared__ __align__(8) uint64_t empty_bar[8];
    __shared__ __align__(8) uint64_t acc_bar, b_ready_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s, last_s;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;                             // STAGES weight tiles
    uint8_t* b_tiles = smem + STAGES * A_BYTES;          // NORM: num_kb resident tiles; else STAGES tiles
    const int b_count = NORM ? p.num_kb : STAGES;
    (void)b_count;
    float* stage_f = (float*)a_tiles;     // ROPE_KV: [128][BN + 1] floats over the weight ring, which is idle by then
    volatile int* abort_flag = &abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TILE_M;                  // first weight row (output feature) of the block
    const int kb_begin = blockIdx.z * p.kb_per_split;
    const int kb_end = min(p.num_kb, kb_begin + p.kb_per_split);
    const int nkb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        mbar_init(&b_ready_bar, 128);
        abort_s = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x == 0) griddep_launch_dependents();

    if (nkb > 0) {
        if (warp == 0) {
            if (lane == 0) {
                // Weights do not depend on the kernel before this one: request the first tiles at once.
                const int pre = min(STAGES, nkb);
                for (int i = 0; i < pre; ++i) {
                    mbar_expect_tx(&full_bar[i], A_BYTES + (NORM ? 0u : B_BYTES));
                    tma_load_2d(a_tiles + i * A_BYTES, &map_w, (kb_begin + i) * TILE_K, n0, &full_bar[i]);
                }
                griddep_wait();
                if (!NORM)
                    for (int i = 0; i < pre; ++i)
                        tma_load_2d(b_tiles + i * B_BYTES, &map_x, (kb_begin + i) * TILE_K, 0, &full_bar[i]);
                for (int i = pre; i < nkb; ++i) {
                    const int s = i % STAGES;
                    if (!mbar_wait(&empty_bar[s], ((i / STAGES) & 1) ^ 1, abort_flag)) break;
                    mbar_expect_tx(&full_bar[s], A_BYTES + (NORM ? 0u : B_BYTES));
                    tma_load_2d(a_tiles + s * A_BYTES, &map_w, (kb_begin + i) * TILE_K, n0, &full_bar[s]);
                    if (!NORM) tma_load_2d(b_tiles + s * B_BYTES, &map_x, (kb_begin + i) * TILE_K, 0, &full_bar[s]);
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                constexpr uint32_t idesc = idesc_bf16(TILE_M, BN);
                bool ok = true;
                if (NORM) ok = mbar_wait(&b_ready_bar, 0, abort_flag);
                for (int i = 0; i < nkb && ok; ++i) {
                    const int s = i % STAGES;
                    ok = mbar_wait(&full_bar[s], (i / STAGES) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(a_tiles + s * A_BYTES);
                    const uint32_t b_addr = smem_u32(b_tiles + (size_t)(NORM ? kb_begin + i : s) * B_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_base, desc_kmajor(a_addr + k * 32), desc_kmajor(b_addr + k * 32), idesc,
                                  (i > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&acc_bar);
            }
        } else {
            const int quarter = warp & 3;
            griddep_wait();
            if (NORM) {
                // B operand = RMSNorm(x) * w for all K, as bf16 in the swizzled K-major tiles.  One warp per row.
                if (p.K <= 1024 && p.M <= 8) {
                    // Few short rows: a warp asks for both of its rows at once and keeps them in registers (8 float4
                    // per lane and row), so the statistics and the scaled copy cost one trip to memory, not four.
                    const int ra = warp - 2, rb = warp + 2;
                    const bool has_a = ra < p.M, has_b = rb < p.M;
                    const float* xa = p.x + (size_t)(has_a ? (p.x_rows ? p.x_rows[ra] : ra) : 0) * p.K;
                    const float* xb = p.x + (size_t)(has_b ? (p.x_rows ? p.x_rows[rb] : rb) : 0) * p.K;
                    float4 va[8], vb[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int k = (i * 32 + lane) * 4;
                        const bool in_k = k < p.K;
                        va[i] = (has_a && in_k) ? *reinterpret_cast<const float4*>(xa + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                        vb[i] = (has_b && in_k) ? *reinterpret_cast<const float4*>(xb + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    float sa = 0.0f, sb = 0.0f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        sa += va[i].x * va[i].x + va[i].y * va[i].y + va[i].z * va[i].z + va[i].w * va[i].w;
                        sb += vb[i].x * vb[i].x + vb[i].y * vb[i].y + vb[i].z * vb[i].z + vb[i].w * vb[i].w;
                    }
                    sa = llb_warp_sum(sa);
                    sb = llb_warp_sum(sb);
                    const float inva = 1.0f / sqrtf(sa / (float)p.K + p.eps), invb = 1.0f / sqrtf(sb / (float)p.K + p.eps);
                    // rows of the tile beyond M stay as they are: what the MMA makes of them is never read
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int k = (i * 32 + lane) * 4;       // 4 elements = half of a 16-byte chunk of the tile row
                        if ((k >> 6) < kb_begin || (k >> 6) >= kb_end) continue;
                        // columns from K to the end of the last tile are written as zeros: the weights there are the
                        // copy's zero fill, but zero times whatever the shared memory held before need not be zero
                        float nw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (k < p.K && p.norm_w_bf16) {
                            const uint2 u = *reinterpret_cast<const uint2*>((const __nv_bfloat16*)p.norm_w + k);
                            const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
                            const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
                            nw[0] = f0.x; nw[1] = f0.y; nw[2] = f1.x; nw[3] = f1.y;
                        } else if (k < p.K) {
                            const float4 c0 = *reinterpret_cast<const float4*>((const float*)p.norm_w + k);
                            nw[0] = c0.x; nw[1] = c0.y; nw[2] = c0.z; nw[3] = c0.w;
                        }
                        const int kb = k >> 6, q = (k & 63) >> 3, sub = (k & 7) * 2;       // tile, chunk, byte offset in it
                        if (has_a) {
                            const __nv_bfloat162 h0 = __floats2bfloat162_rn(va[i].x * inva * nw[0], va[i].y * inva * nw[1]);
                            const __nv_bfloat162 h1 = __floats2bfloat162_rn(va[i].z * inva * nw[2], va[i].w * inva * nw[3]);
                            uint8_t* dst = b_tiles + (size_t)kb * B_BYTES + (uint32_t)ra * 128 + ((q ^ (ra & 7)) * 16) + sub;
                            *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&h0),
                                                                        *reinterpret_cast<const uint32_t*>(&h1));
                        }
                        if (has_b) {
                            const __nv_bfloat162 h0 = __floats2bfloat162_rn(vb[i].x * invb * nw[0], vb[i].y * invb * nw[1]);
                            const __nv_bfloat162 h1 = __floats2bfloat162_rn(vb[i].z * invb * nw[2], vb[i].w * invb * nw[3]);
                            uint8_t* dst = b_tiles + (size_t)kb * B_BYTES + (uint32_t)rb * 128 + ((q ^ (rb & 7)) * 16) + sub;
                            *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&h0),
                                                                        *reinterpret_cast<const uint32_t*>(&h1));
                        }
                    }
                } else
                for (int r = warp - 2; r < BN; r += 4) {
                    const bool real = r < p.M;
                    const float* xr = p.x + (size_t)(real ? (p.x_rows ? p.x_rows[r] : r) : 0) * p.K;
                    float ss = 0.0f;
                    if (real)
                        for (int k = lane * 4; k < p.K; k += 128) {
                            const float4 v = *reinterpret_cast<const float4*>(xr + k);
                            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                        }
                    ss = llb_warp_sum(ss);
                    const float inv = 1.0f / sqrtf(ss / (float)p.K + p.eps);
                    // 16-byte chunks: chunk c of the row covers k = 8c .. 8c+7; tile kb = c / 8 (this split's tiles only)
                    for (int c = kb_begin * 8 + lane; c < kb_end * 8; c += 32) {
                        uint32_t w[4] = {0u, 0u, 0u, 0u};
                        const int k = c * 8;
                        if (real && k < p.K) {
                            const float4 a = *reinterpret_cast<const float4*>(xr + k);
                            const float4 b = *reinterpret_cast<const float4*>(xr + k + 4);
                            const float xv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                            float nw[8];
                            if (p.norm_w_bf16) {
                                const uint4 u = *reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.norm_w + k);
                                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float2 f = __bfloat1622float2(h[i]);
                                    nw[2 * i] = f.x; nw[2 * i + 1] = f.y;
                                }
                            } else {
                                const float4 c0 = *reinterpret_cast<const float4*>((const float*)p.norm_w + k);
                                const float4 c1 = *reinterpret_cast<const float4*>((const float*)p.norm_w + k + 4);
                                nw[0] = c0.x; nw[1] = c0.y; nw[2] = c0.z; nw[3] = c0.w;
                                nw[4] = c1.x; nw[5] = c1.y; nw[6] = c1.z; nw[7] = c1.w;
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(xv[2 * i] * inv * nw[2 * i],
                                                                               xv[2 * i + 1] * inv * nw[2 * i + 1]);
                                w[i] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                        }
                        const int kb = c >> 3, q = c & 7;
                        uint8_t* dst = b_tiles + (size_t)kb * B_BYTES + (uint32_t)r * 128 + ((q ^ (r & 7)) * 16);
                        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
                fence_async_smem();
                mbar_arrive(&b_ready_bar);
            }
            const int row = quarter * 32 + lane;     // row of the tile = TMEM lane = output feature
            const int n = n0 + row;
            // Rotary epilogue: what this output feature needs of the first 16 tokens (their angles' cos and sin,
            // their cache rows) is asked for now, while the tensor cores still work; loaded one by one inside the
            // loop over the tokens, each of these reads would be a round trip of its own.
            RopeRow rr;
            float2 cs_first[16];
            int slot_first[16];
            if (EPI == DEPI_ROPE_KV) {
                rr = rope_row(p, n, row);
                rope_fetch(p, rr, n, 0, cs_first, slot_first);
            }
            bool ok = mbar_wait(&acc_bar, 0, abort_flag);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            const bool meet = (EPI == DEPI_ROPE_KV || EPI == DEPI_SWIGLU) && gridDim.z > 1;
            if (meet) {
                // Partial sums of the splits meet in scratch; the split that arrives last runs the epilogue.
                if (ok) {      // uniform over the warp: tcgen05.ld is a warp-wide instruction
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        float v[16];
                        tmem_ld16(taddr + c0, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < p.M && n < p.N) atomicAdd(p.acc_scratch + (size_t)(c0 + j) * p.N + n, v[j]);
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) last_s = (atomicAdd(p.counters + blockIdx.x, 1) == (int)gridDim.z - 1) ? 1 : 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                ok = ok && last_s != 0;
                if (ok) __threadfence();
            }
            // This thread's row of the tile, 16 columns (tokens) at a time: from tensor memory, or from the
            // meeting place (which is left zeroed for the next launch).
            auto load16 = [&](int c0, float (&v)[16]) {
                if (!meet) {
                    tmem_ld16(taddr + c0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        v[j] = 0.0f;
                        if (c0 + j < p.M && n < p.N) {
                            float* a = p.acc_scratch + (size_t)(c0 + j) * p.N + n;
                            v[j] = __ldcg(a);
                            __stcg(a, 0.0f);
                        }
                    }
                }
            };
            const float bias = (p.bias && n < p.N && (meet || blockIdx.z == 0)) ? p.bias[n] : 0.0f;
            if (EPI == DEPI_ROPE_KV) {
                // Stage the tile (+ bias) as float; the barrier is reached by all four warps whatever happened.
                if (ok) {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        float v[16];
                        load16(c0, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j) stage_f[row * (BN + 1) + c0 + j] = v[j] + bias;
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (ok) {
                if (EPI == DEPI_ROPE_KV) {
                    // Rotate pairs of rows of one head and scatter to q and the cache pages, 16 tokens at a time.
                    if (n < p.N) {
                        const int q_end = p.Hq * p.hd, k_end = q_end + p.Hkv * p.hd;
                        for (int m0 = 0; m0 < p.M; m0 += 16) {
                            float2 cs[16];
                            int slot[16];
                            if (m0 == 0) {
#pragma unroll
                                for (int j = 0; j < 16; ++j) { cs[j] = cs_first[j]; slot[j] = slot_first[j]; }
                            } else {
                                rope_fetch(p, rr, n, m0, cs, slot);
                            }
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int m = m0 + j;
                                if (m >= p.M) break;
                                float val = stage_f[row * (BN + 1) + m];
                                if (rr.rotate) {
                                    const float other = stage_f[rr.partner * (BN + 1) + m];
                                    val = rr.first ? val * cs[j].x - other * cs[j].y : val * cs[j].x + other * cs[j].y;
                                }
                                const __nv_bfloat16 h = __float2bfloat16_rn(val);
                                if (n < q_end) {
                                    p.q_out[(size_t)m * q_end + n] = h;
                                } else if (slot[j] >= 0) {
                                    if (n < k_end) p.k_cache[(size_t)slot[j] * (p.Hkv * p.hd) + (n - q_end)] = h;
                                    else p.v_cache[(size_t)slot[j] * (p.Hkv * p.hd) + (n - k_end)] = h;
                                }
                            }
                        }
                    }
                } else {
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        float v[16];
                        load16(c0, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = c0 + j;
                            const float val = v[j] + bias;
                            if (EPI == DEPI_SWIGLU) {
                                const float other = __shfl_xor_sync(0xffffffffu, val, 1);   // gate: even rows, up: odd rows
                                if ((lane & 1) == 0 && m < p.M && n + 1 < p.N)
                                    ((__nv_bfloat16*)p.out)[(size_t)m * (p.N / 2) + (n >> 1)] =
                                        __float2bfloat16_rn(llb_silu(val) * other);
                            } else if (m < p.M && n < p.N) {
                                const size_t idx = (size_t)m * p.N + n;
                                if (EPI == DEPI_STORE_F32) ((float*)p.out)[idx] = val;
                                else if (gridDim.z == 1) p.residual[idx] += val;
                                else atomicAdd(p.residual + idx, val);
                            }
                        }
                    }
                }
                if (meet && warp == 2 && lane == 0) atomicExch(p.counters + blockIdx.x, 0);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_s && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 4);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Weight maps are cached by (pointer, shape); activations get a fresh map per launch.
struct MapKey {
    const void* ptr; long long rows, cols; int box;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box == o.box; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols << 20) ^ ((size_t)k.box << 44);
    }
};
int cached_map(const void* ptr, long long rows, long long cols, int box, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, box};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return 0; }
    }
    int rc = make_map_bf16(ptr, rows, cols, box, out);
    if (rc) return rc;
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

size_t smem_bytes(int BN, int stages, int b_tiles) {
    // the rotary epilogue stages its tile over the weight ring (128 x 65 floats < 8 x 16 KB)
    return (size_t)stages * A_BYTES + (size_t)b_tiles * BN * TILE_K * 2 + 1024;
}

template <int BN, int EPI, bool NORM, int STAGES>
int launch_stages(const CUtensorMap& mw, const CUtensorMap& mx, const DecodeGemmParams& p, int split_k, cudaStream_t stream) {
    const size_t smem = smem_bytes(BN, STAGES, NORM ? p.num_kb : STAGES);
    LLB_REQUIRE(smem <= 224 * 1024, "gemm_decode: K=%d with %d rows needs %zu bytes of shared memory", p.K, BN, smem);
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_decode_kernel<BN, EPI, NORM, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return llb_fail("gemm_decode: cannot opt in to %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
        configured = smem;
    }
    dim3 grid(llb_ceil_div(p.N, TILE_M), 1, split_k);
    cudaError_t e = launch_pdl(gemm_decode_kernel<BN, EPI, NORM, STAGES>, grid, dim3(NUM_THREADS), smem, stream, mw, mx, p);
    if (e != cudaSuccess) return llb_fail("gemm_decode: launch failed: %s", cudaGetErrorString(e));
    return llb_check_launch("gemm_decode");
}

template <int BN, int EPI, bool NORM>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const DecodeGemmParams& p, int split_k, cudaStream_t stream) {
    // the float-store epilogue is the head's: a vocabulary's worth of blocks
    if (EPI == DEPI_STORE_F32 && !NORM && llb_ceil_div(p.N, TILE_M) >= 256)
        return launch_stages<BN, EPI, NORM, SHALLOW>(mw, mx, p, split_k, stream);
    return launch_stages<BN, EPI, NORM, DEEP>(mw, mx, p, split_k, stream);
}

template <int BN, bool NORM>
int dispatch_epi(int epi, const CUtensorMap& mw, const CUtensorMap& mx, const DecodeGemmParams& p, int split_k,
                 cudaStream_t s) {
    switch (epi) {
        case DEPI_STORE_F32: return launch<BN, DEPI_STORE_F32, NORM>(mw, mx, p, split_k, s);
        case DEPI_RESIDUAL: return launch<BN, DEPI_RESIDUAL, NORM>(mw, mx, p, split_k, s);
        case DEPI_SWIGLU: return launch<BN, DEPI_SWIGLU, NORM>(mw, mx, p, split_k, s);
        case DEPI_ROPE_KV: return launch<BN, DEPI_ROPE_KV, NORM>(mw, mx, p, split_k, s);
    }
    return llb_fail("gemm_decode: unknown epilogue %d", epi);
}

template <bool NORM>
int dispatch_bn(int epi, const CUtensorMap& mw, const CUtensorMap& mx, const DecodeGemmParams& p, int split_k,
                cudaStream_t s) {
    if (p.M <= 16) return dispatch_epi<16, NORM>(epi, mw, mx, p, split_k, s);
    if (p.M <= 32) return dispatch_epi<32, NORM>(epi, mw, mx, p, split_k, s);
    return dispatch_epi<64, NORM>(epi, mw, mx, p, split_k, s);
}

}  // namespace

// Whether the fused decode contraction takes this shape.
LLB_EXPORT int llb_gemm_decode_supports(int M, int N, int K, int norm, int epilogue, int hd) {
    if (M < 1 || M > 64 || K % 8 != 0 || N < 1) return 0;
    const int BN = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    const int num_kb = llb_ceil_div(K, TILE_K);
    if (smem_bytes(BN, DEEP, norm ? num_kb : DEEP) > 224 * 1024) return 0;
    if (epilogue == DEPI_SWIGLU && N % 2) return 0;
    if (epilogue == DEPI_ROPE_KV && (hd < 2 || TILE_M % hd != 0)) return 0;
    return 1;
}

// W [N, K] bf16 (K a multiple of 8).  Activations: with norm != 0 the float rows x[x_rows[r]] (or x[r])
// of width K, normalised with norm_w (float, or bf16 when norm_w_bf16) and eps inside the kernel; else
// a_bf16 [M, K].  Epilogues: 1 store float out[M, N]; 2 add into residual[M, N] (split_k >= 1);
// 3 SwiGLU out[M, N/2] bf16; 4 rotary + q_out + cache write (N = (Hq + 2 Hkv) * hd; without
// slot_mapping only q is written and N = Hq * hd); rope_table [M, rotary_dim/2] holds (cos, sin) of each
// token's angle (llb_rope_table).  split_k > 1 with epilogue 3 or 4 needs acc_scratch (scratch_floats >= BN * N
// floats, all zero on entry and left zero) and counters (one int per 128 output features, zero on entry and left zero).
LLB_EXPORT int llb_gemm_decode(const void* W, const void* a_bf16, const float* x, const int* x_rows, const void* norm_w,
                               int norm_w_bf16, float eps, int norm, const float* bias, void* out, float* residual,
                               int epilogue, int M, int N, int K, int split_k,
                               const int* slot_mapping, const float* rope_table, int rotary_dim, int interleaved, int Hq,
                               int Hkv, int hd, void* q_out, void* k_cache, void* v_cache, float* acc_scratch,
                               long long scratch_floats, int* counters, int* error_flag, cudaStream_t stream) {
    if (M == 0) return 0;
    LLB_REQUIRE(llb_gemm_decode_supports(M, N, K, norm, epilogue, hd), "gemm_decode: unsupported shape M=%d N=%d K=%d", M, N, K);
    LLB_REQUIRE(((uintptr_t)W % 16 == 0), "gemm_decode: weights must be 16-byte aligned");
    LLB_REQUIRE(norm ? (x != nullptr && norm_w != nullptr && (uintptr_t)x % 16 == 0 && (uintptr_t)norm_w % 16 == 0)
                     : (a_bf16 != nullptr && (uintptr_t)a_bf16 % 16 == 0), "gemm_decode: bad activation operand");
    LLB_REQUIRE(split_k >= 1 && epilogue != DEPI_STORE_F32 || split_k == 1, "gemm_decode: the float-store epilogue takes no split_k");
    if (split_k > 1 && (epilogue == DEPI_ROPE_KV || epilogue == DEPI_SWIGLU))
        LLB_REQUIRE(acc_scratch != nullptr && counters != nullptr && scratch_floats >= (long long)(M <= 16 ? 16 : M <= 32 ? 32 : 64) * N,
                    "gemm_decode: split_k=%d with a fused epilogue needs %lld floats of zeroed scratch and counters",
                    split_k, (long long)(M <= 16 ? 16 : M <= 32 ? 32 : 64) * N);
    if (epilogue == DEPI_ROPE_KV) {
        const int hkv = slot_mapping ? Hkv : 0;
        LLB_REQUIRE(N == (Hq + 2 * hkv) * hd && rotary_dim % 2 == 0 && rotary_dim <= hd && q_out &&
                    (rotary_dim == 0 || rope_table), "gemm_decode: rotary epilogue arguments do not fit");
    }
    DecodeGemmParams p = {};
    p.x = x; p.x_rows = x_rows; p.norm_w = norm_w; p.norm_w_bf16 = norm_w_bf16; p.eps = eps;
    p.bias = bias; p.out = out; p.residual = residual; p.M = M; p.N = N; p.K = K;
    p.num_kb = llb_ceil_div(K, TILE_K);
    if (split_k > p.num_kb) split_k = p.num_kb;
    p.kb_per_split = llb_ceil_div(p.num_kb, split_k);
    split_k = llb_ceil_div(p.num_kb, p.kb_per_split);
    p.slot_mapping = slot_mapping; p.rope_table = (const float2*)rope_table; p.rotary_dim = rotary_dim;
    p.interleaved = interleaved; p.Hq = Hq; p.Hkv = slot_mapping ? Hkv : 0; p.hd = hd;
    p.q_out = (__nv_bfloat16*)q_out; p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
    p.acc_scratch = acc_scratch; p.counters = counters;
    p.error_flag = error_flag;
    CUtensorMap mw, mx;
    int rc = cached_map(W, N, K, TILE_M, &mw);
    if (rc) return rc;
    const int BN = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    if (norm) {
        mx = mw;   // unused
        return dispatch_bn<true>(epilogue, mw, mx, p, split_k, stream);
    }
    if ((rc = make_map_bf16(a_bf16, M, K, BN, &mx))) return rc;
    return dispatch_bn<false>(epilogue, mw, mx, p, split_k, stream);
}
