// Dense contraction on the 5th-generation tensor cores (sm_100a): bf16 operands staged in shared
// memory by TMA, tcgen05.mma issued by one thread, float accumulators in tensor memory (TMEM),
// read back with tcgen05.ld for a fused epilogue.
//
// C[M,N] = A[M,K] * W[N,K]^T with W stored [out, in] as in the checkpoint
// (src/engine/engine_server.cpp:1542-1544; the reference calls cuBLAS, src/ops/gemm.cu:92-97).
// Both operands are K-major, so either can take the MMA's 128-row "A" role:
//   * many rows (prefill):  A role = 128 activation rows, B role = BN weight rows;
//   * few rows (decode):    A role = 128 weight rows, B role = the activation rows (BN >= M),
//                           so that no tensor-core row is wasted on padding ("swap").
// Epilogues: store, store float, add into the float residual stream (with split-K: atomic adds),
// SiLU(gate)*up on interleaved weight rows; the bias is added first.
//
// One block computes one 128 x BN tile (two blocks share an SM, so that one's epilogue overlaps the
// other's main loop).  Warp 0 issues TMA loads through a ring of STAGES shared memory stages, warp 1
// allocates TMEM and issues the MMAs, warps 2..5 run the epilogue (each reads the 32 TMEM lanes it may
// access) and write whole 16-byte vectors per thread.  Every wait on an mbarrier is bounded in time: when it
// runs out the kernel raises a flag in global memory, lets every role fall through to the common
// exit, frees its TMEM and returns; the host reports the flag as an error.
#include <cuda.h>

#include <cstdlib>

#include <mutex>
#include <unordered_map>

#include "tcgen05_common.cuh"

namespace {

using namespace t5;

// SiLU for the bf16 epilogues: the fast exponential and division are far inside bf16's rounding.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

constexpr int TILE_M = 128;       // rows of the A role = TMEM lanes
constexpr int TILE_K = 64;        // bf16 elements per stage row = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 3;
constexpr int NUM_THREADS = 192;

struct GemmParams {
    void* out;              // STORE / SWIGLU: bf16; STORE_F32: float
    float* residual;        // RESIDUAL
    const float* bias;      // [N] or null
    int M, N, K;
    int num_kb;             // K blocks in all
    int kb_per_split;       // K blocks per grid.z slice (per split of the persistent kernel)
    int splits;             // persistent kernel: work items per tile along K
    int direct;             // residual epilogue with splits: every piece adds its part to the residual itself (TMA
                            // reduce-add), nothing meets in `partials`
    float* partials;        // [items, tile width, 128] float: the splits' accumulators meet here
    int* counters;          // [tiles, 8] zero before and after: arrivals per warp region of a tile
    int tma_out;            // the epilogue leaves through shared memory and TMA stores (map_out is valid)
    int* error_flag;        // raised when a wait ran out of time
    // rotary epilogue of the q/k/v projection (heads of 64, NeoX pairs, whole head rotated)
    const float2* rope_table;   // [hd/2, M] of (cos, sin): pair-major, so that a warp's rows read neighbouring entries
    const int* slot_mapping;    // [M] cache row of each token, negative: not written
    __nv_bfloat16* q_out;       // [M, Hq * hd]
    __nv_bfloat16* k_cache;     // [slots, Hkv, 64]
    __nv_bfloat16* v_cache;
    int Hq, Hkv;
};

// Epilogue of one thread in the row-major orientation: token row m, CHUNK consecutive output features
// starting at nb, accumulators in r.  Whole 16-byte vectors are written where the row allows.
template <int EPI, int CHUNK>
__device__ __forceinline__ void epilogue_row(const GemmParams& p, int m, int nb, const uint32_t (&r)[32]) {
    if (m < p.M && nb < p.N) {
        float v[CHUNK];
#pragma unroll
        for (int j = 0; j < CHUNK; ++j) v[j] = __uint_as_float(r[j]);
        const bool full = nb + CHUNK <= p.N;
        if (p.bias && blockIdx.z == 0) {
#pragma unroll
            for (int j = 0; j < CHUNK; ++j)
                if (full || nb + j < p.N) v[j] += p.bias[nb + j];
        }
        if (EPI == LLB_EPI_SWIGLU) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)m * (p.N / 2) + (nb >> 1);
            if (full && (p.N % 16) == 0) {     // 16-byte stores of 8 outputs
#pragma unroll
                for (int j = 0; j < CHUNK; j += 16) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(
                            silu_fast(v[j + 4 * e]) * v[j + 4 * e + 1],
                            silu_fast(v[j + 4 * e + 2]) * v[j + 4 * e + 3]);
                        w[e] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(o + (j >> 1)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < CHUNK; j += 2)
                    if (nb + j + 1 < p.N) o[j >> 1] = __float2bfloat16_rn(llb_silu(v[j]) * v[j + 1]);
            }
        } else if (EPI == LLB_EPI_STORE) {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)m * p.N + nb;
            if (full && (p.N % 8) == 0) {
#pragma unroll
                for (int j = 0; j < CHUNK; j += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                        w[e] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(o + j) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < CHUNK; ++j)
                    if (nb + j < p.N) o[j] = __float2bfloat16_rn(v[j]);
            }
        } else if (EPI == LLB_EPI_STORE_F32) {
            float* o = (float*)p.out + (size_t)m * p.N + nb;
            if (full && (p.N % 4) == 0) {
#pragma unroll
                for (int j = 0; j < CHUNK; j += 4)
                    *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < CHUNK; ++j)
                    if (nb + j < p.N) o[j] = v[j];
            }
        } else {
            float* o = p.residual + (size_t)m * p.N + nb;
            if (gridDim.z == 1 && full && (p.N % 4) == 0) {
#pragma unroll
                for (int j = 0; j < CHUNK; j += 4) {
                    float4 t = *reinterpret_cast<float4*>(o + j);
                    t.x += v[j]; t.y += v[j + 1]; t.z += v[j + 2]; t.w += v[j + 3];
                    *reinterpret_cast<float4*>(o + j) = t;
                }
            } else {
#pragma unroll
                for (int j = 0; j < CHUNK; ++j) {
                    if (nb + j < p.N) {
                        if (gridDim.z == 1) o[j] += v[j];
                        else atomicAdd(o + j, v[j]);
                    }
                }
            }
        }
    }
}

constexpr int EPI_ROPE64 = 4;     // q/k/v projection of heads of 64: bias, NeoX rotation, q store, K/V page write
constexpr int EPI_ROPE128 = 5;    // the same with heads of 128 (one head is one tile of 128 columns)
constexpr bool epi_is_rope(int epi) { return epi == EPI_ROPE64 || epi == EPI_ROPE128; }

template <int BN, int EPI, bool SWAP>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
    constexpr uint32_t A_BYTES = TILE_M * TILE_K * 2;
    constexpr uint32_t B_BYTES = BN * TILE_K * 2;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle needs 1024-byte alignment
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + STAGES * A_BYTES;
    uint64_t* full_bar = (uint64_t*)(b_tiles + STAGES * B_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* acc_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(acc_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a_row0 = blockIdx.x * TILE_M;     // first row of the A-role operand
    const int b_row0 = blockIdx.y * BN;         // first row of the B-role operand
    const int kb_begin = blockIdx.z * p.kb_per_split;
    const int kb_end = min(p.num_kb, kb_begin + p.kb_per_split);
    const int nkb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (nkb > 0) {
        if (warp == 0) {
            if (lane == 0) {
                for (int i = 0; i < nkb; ++i) {
                    const int s = i % STAGES;
                    const uint32_t phase = (i / STAGES) & 1;
                    if (!mbar_wait(&empty_bar[s], phase ^ 1, abort_flag)) break;
                    mbar_expect_tx(&full_bar[s], A_BYTES + B_BYTES);
                    const int kx = (kb_begin + i) * TILE_K;
                    tma_load_2d(a_tiles + s * A_BYTES, &map_a, kx, a_row0, &full_bar[s]);
                    tma_load_2d(b_tiles + s * B_BYTES, &map_b, kx, b_row0, &full_bar[s]);
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                constexpr uint32_t idesc = idesc_bf16(TILE_M, BN);
                bool ok = true;
                for (int i = 0; i < nkb && ok; ++i) {
                    const int s = i % STAGES;
                    const uint32_t phase = (i / STAGES) & 1;
                    ok = mbar_wait(&full_bar[s], phase, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(a_tiles + s * A_BYTES);
                    const uint32_t b_addr = smem_u32(b_tiles + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; ++k) {
                        umma_bf16(tmem_base, desc_kmajor(a_addr + k * UMMA_K * 2), desc_kmajor(b_addr + k * UMMA_K * 2),
                                  idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);      // frees the stage when these MMAs have read it
                }
                if (ok) umma_commit(acc_bar);         // the accumulator is complete
            }
        } else {
            // Epilogue: warp w may read TMEM lanes (w % 4) * 32 .. + 31.
            const int quarter = warp & 3;
            const bool ok = mbar_wait(acc_bar, 0, abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok) {
                const int row = quarter * 32 + lane;            // row of the tile = TMEM lane
                constexpr int CHUNK = BN >= 32 ? 32 : 16;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += CHUNK) {
                    uint32_t r[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0;
                    if (CHUNK == 32) tmem_ld32_nowait(taddr, r); else tmem_ld16_nowait(taddr, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (!SWAP) {
                        // row = token m, columns = output features n: 32 consecutive columns per thread
                        epilogue_row<EPI, CHUNK>(p, a_row0 + row, b_row0 + c0, r);
                    } else {
                        // row = output feature n, columns = tokens m
                        const int n = a_row0 + row;
                        const int mb = b_row0 + c0;
                        const float bias = (p.bias && n < p.N && blockIdx.z == 0) ? p.bias[n] : 0.0f;
#pragma unroll
                        for (int j = 0; j < CHUNK; ++j) {
                            const int m = mb + j;
                            float v = __uint_as_float(r[j]) + bias;
                            if (EPI == LLB_EPI_SWIGLU) {
                                const float other = __shfl_xor_sync(0xffffffffu, v, 1);   // gate in even rows, up in odd
                                if ((lane & 1) == 0 && m < p.M && n + 1 < p.N)
                                    ((__nv_bfloat16*)p.out)[(size_t)m * (p.N / 2) + (n >> 1)] =
                                        __float2bfloat16_rn(llb_silu(v) * other);
                            } else if (m < p.M && n < p.N) {
                                const size_t idx = (size_t)m * p.N + n;
                                if (EPI == LLB_EPI_STORE) ((__nv_bfloat16*)p.out)[idx] = __float2bfloat16_rn(v);
                                else if (EPI == LLB_EPI_STORE_F32) ((float*)p.out)[idx] = v;
                                else if (gridDim.z == 1) p.residual[idx] += v;
                                else atomicAdd(p.residual + idx, v);
                            }
                        }
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 1);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Many rows (prefill): a persistent kernel, one block per SM, that walks over the 128 x 128 output tiles.
// The TMA ring keeps running across tile boundaries, and the accumulator is double buffered in tensor
// memory (2 x 128 columns), so the epilogue of one tile overlaps the main loop of the next.
// Tiles are ordered rows-first, so that the blocks working at the same time share a few weight tiles in L2.
// ---------------------------------------------------------------------------------------------
// Tile width P_BN = 128 (6 stages) or 256 (4 stages): the wide tile re-uses each activation tile for twice as
// many output features, which matters because the main loop is bound by the bytes an SM can pull from L2.

// ---- Epilogue through shared memory and TMA ---------------------------------------------------------
// A thread owns one row of the tile, so its direct stores are 16-byte pieces of 32 different rows per warp
// instruction, which costs the memory system dearly (a third of o_proj's time).  Instead each epilogue warp owns a
// 4 KB staging tile (32 rows x 128 bytes, 128-byte swizzle), fills it from its accumulator chunks and hands it to
// the TMA engine, which writes whole rows (and clips at the matrix's edge): a store for out, a reduce-add for the
// residual stream.  One row of the staging tile takes 32 float outputs (one accumulator chunk), 64 bf16 outputs
// (two chunks) or 64 SiLU*mul outputs (four chunks).
template <int EPI> struct StagedOut {
    static constexpr int PIECES = (EPI == LLB_EPI_STORE) ? 2 : (EPI == LLB_EPI_SWIGLU) ? 4 : 1;   // chunks per staged row
};
// One accumulator chunk (32 columns starting at output feature nb, this lane's row) goes into the warp's staging
// tile as piece `piece` of the row; with the row's last piece the tile is handed to TMA at (row0, the row's first
// feature).  Whole-warp call.
template <int EPI>
__device__ __forceinline__ void staged_chunk(const GemmParams& p, const CUtensorMap* map_out, uint8_t* stage, int lane,
                                             int row0, int nb, int piece, const uint32_t (&r)[32]) {
    constexpr int PIECES = StagedOut<EPI>::PIECES;
    constexpr int CHUNKS = 8 / PIECES;               // 16-byte chunks of the 128-byte row that one piece fills
    if (piece == 0) {                                // the tile's last store must have read it
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
    }
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (p.bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (nb + j < p.N) v[j] += p.bias[nb + j];
    }
    uint8_t* row = stage + lane * 128;
    if (EPI == LLB_EPI_STORE_F32 || EPI == LLB_EPI_RESIDUAL) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(row + ((c ^ (lane & 7)) * 16)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    } else if (EPI == LLB_EPI_STORE) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * c + 2 * e], v[8 * c + 2 * e + 1]);
                w[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(row + (((piece * CHUNKS + c) ^ (lane & 7)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {      // SiLU(gate) * up on interleaved features: 32 accumulator columns give 16 outputs
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = 16 * c + 4 * e;
                const __nv_bfloat162 h = __floats2bfloat162_rn(silu_fast(v[j]) * v[j + 1], silu_fast(v[j + 2]) * v[j + 3]);
                w[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(row + (((piece * CHUNKS + c) ^ (lane & 7)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    if (piece == PIECES - 1) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            const int first = nb - (PIECES - 1) * 32;                     // first accumulator column of the staged row
            const int x = (EPI == LLB_EPI_SWIGLU) ? first / 2 : first;
            if (row0 < p.M && first < p.N) {         // a box that lies wholly outside the matrix is not issued
                if (EPI == LLB_EPI_RESIDUAL) tma_reduce_add_2d(map_out, smem_u32(stage), x, row0);
                else tma_store_2d(map_out, smem_u32(stage), x, row0);
                tma_store_commit();
            }
        }
    }
}

// Rotary epilogue of one warp: token rows row0 .. row0+31 (one per lane) and the 64 output features nb .. nb+63 of q,
// k or v (src/ops/rope.cu:54-59 on every pair; cache rows as src/kv_cache/paged_attention.cu:1150-1163).  With heads
// of 64 these are one whole head and both members of every pair (j, j + 32) are here; with heads of 128 they are half
// of a head, the pairs are (j, j + 64), and the other members come in `p0`, `p1` (the same columns of the head's other
// half).  The (cos, sin) table is laid out [pair][token], so the lanes of a warp read neighbouring entries.  q leaves
// through the warp's staging tile and one TMA store (64 bf16 are one 128-byte row of it) when `staged`; k and v go
// straight to their cache rows, which lie wherever the pages are.
template <int HD>
__device__ __forceinline__ void epilogue_rope_warp(const GemmParams& p, const CUtensorMap* map_q, uint8_t* stage,
                                                   bool staged, int lane, int row0, int nb, const uint32_t (&r0)[32],
                                                   const uint32_t (&r1)[32], const uint32_t (&p0)[32],
                                                   const uint32_t (&p1)[32]) {
    if (nb >= p.N) return;                       // uniform over the warp
    const int m = row0 + lane;
    const bool in_m = m < p.M;
    const int q_end = p.Hq * HD, k_end = q_end + p.Hkv * HD;
    const bool second_half = HD == 128 && (nb & 64) != 0;      // these columns are the pairs' second members
    float a[32], b[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        a[j] = __uint_as_float(r0[j]);
        b[j] = __uint_as_float(r1[j]);
        if (p.bias) { a[j] += p.bias[nb + j]; b[j] += p.bias[nb + 32 + j]; }
    }
    if (nb < k_end && in_m) {
        const float2* cs = p.rope_table + m;
        if (HD == 64) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float2 t = cs[(size_t)j * p.M];
                const float x = a[j], y = b[j];
                a[j] = x * t.x - y * t.y;
                b[j] = y * t.x + x * t.y;
            }
        } else {
            const int nbp = second_half ? nb - 64 : nb + 64;      // where the partners' bias lies
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                float pa = __uint_as_float(p0[j]), pb = __uint_as_float(p1[j]);
                if (p.bias) { pa += p.bias[nbp + j]; pb += p.bias[nbp + 32 + j]; }
                const float2 ta = cs[(size_t)j * p.M], tb = cs[(size_t)(32 + j) * p.M];
                a[j] = second_half ? a[j] * ta.x + pa * ta.y : a[j] * ta.x - pa * ta.y;
                b[j] = second_half ? b[j] * tb.x + pb * tb.y : b[j] * tb.x - pb * tb.y;
            }
        }
    }
    uint32_t wa[16], wb[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
        const __nv_bfloat162 g = __floats2bfloat162_rn(b[2 * e], b[2 * e + 1]);
        wa[e] = *reinterpret_cast<const uint32_t*>(&h);
        wb[e] = *reinterpret_cast<const uint32_t*>(&g);
    }
    if (nb < q_end && staged) {
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        uint8_t* row = stage + lane * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            *reinterpret_cast<uint4*>(row + ((c ^ (lane & 7)) * 16)) = make_uint4(wa[4 * c], wa[4 * c + 1], wa[4 * c + 2], wa[4 * c + 3]);
            *reinterpret_cast<uint4*>(row + (((4 + c) ^ (lane & 7)) * 16)) = make_uint4(wb[4 * c], wb[4 * c + 1], wb[4 * c + 2], wb[4 * c + 3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && row0 < p.M) {
            tma_store_2d(map_q, smem_u32(stage), nb, row0);
            tma_store_commit();
        }
        return;
    }
    if (!in_m) return;
    __nv_bfloat16* dst;
    if (nb < q_end) {
        dst = p.q_out + (size_t)m * q_end + nb;
    } else {
        const int slot = p.slot_mapping ? p.slot_mapping[m] : -1;
        if (slot < 0) return;
        dst = nb < k_end ? p.k_cache + (size_t)slot * (p.Hkv * HD) + (nb - q_end)
                         : p.v_cache + (size_t)slot * (p.Hkv * HD) + (nb - k_end);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<uint4*>(dst + 8 * c) = make_uint4(wa[4 * c], wa[4 * c + 1], wa[4 * c + 2], wa[4 * c + 3]);
        *reinterpret_cast<uint4*>(dst + 32 + 8 * c) = make_uint4(wb[4 * c], wb[4 * c + 1], wb[4 * c + 2], wb[4 * c + 3]);
    }
}

constexpr int P_THREADS = 64 + 256;      // TMA warp, MMA warp, eight epilogue warps (two per TMEM lane quarter)

// PAIR: two CTAs (a cluster of two) share a tile of 256 rows x 256 features: each loads its 128 rows of A and its half
// of B, the first CTA issues tcgen05.mma.cta_group::2 over both, and each drains its own 128 x 256 accumulator.  A block of
// K then costs a CTA 32 KB of operands for 512 cycles of tensor work, the 64 bytes per cycle an SM gets from L2, where
// the single-CTA wide tile needs 96.
template <int EPI, int P_BN, bool PAIR>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
    static_assert(!PAIR || P_BN == 256, "a pair's tile is 256 features wide");
    // KPS blocks of K share a stage (and a commit): the hand-over of a stage between the loading and the issuing thread
    // costs about 150 cycles beyond the MMAs of one block of K, which a pair's smaller stages leave room to halve.
    constexpr int KPS = PAIR ? 2 : 1;
    constexpr int P_STAGES = PAIR ? 3 : (P_BN == 256 ? 4 : 6);
    constexpr int ROWS_PER_TILE = PAIR ? 2 * TILE_M : TILE_M;
    constexpr uint32_t A_BYTES = TILE_M * TILE_K * 2;
    constexpr uint32_t B_BYTES = (PAIR ? P_BN / 2 : P_BN) * TILE_K * 2;
    constexpr uint32_t TMEM_COLS = 2 * P_BN;
    __shared__ __align__(8) uint64_t full_bar[P_STAGES];
    __shared__ __align__(8) uint64_t empty_bar[P_STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_slot_s;
    __shared__ int abort_s;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + P_STAGES * KPS * A_BYTES;
    uint8_t* out_tiles = b_tiles + P_STAGES * KPS * B_BYTES;       // eight staging tiles of 4 KB, one per epilogue warp
    volatile int* abort_flag = &abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;            // which CTA of the pair
    const int first_item = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int item_stride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int m_tiles = (p.M + ROWS_PER_TILE - 1) / ROWS_PER_TILE;
    const int n_tiles = (p.N + P_BN - 1) / P_BN;
    const int num_tiles = m_tiles * n_tiles;
    const int nkb = p.num_kb;
    const int splits = p.splits;
    const int num_items = num_tiles * splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], PAIR ? 16 : 8);        // one arrival per epilogue warp (of both CTAs of a pair)
        }
        abort_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) tmem_alloc2(&tmem_slot_s, TMEM_COLS);
        else tmem_alloc(&tmem_slot_s, TMEM_COLS);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync_all();       // both CTAs' barriers exist before either signals the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot_s;
    // Programmatic dependent launch: the kernel after this one may start its own set-up as blocks of this one leave
    // (it waits for this kernel's completion itself before it touches global memory); nothing here reads or writes
    // global memory before the kernel before this one has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int it = 0;                                  // k-blocks issued so far, over all tiles
            // pair: both CTAs' loads complete on the first CTA's barrier, which that CTA arms for both
            const uint32_t full_of_first = PAIR ? mapa_u32(smem_u32(&full_bar[0]), 0) : 0u;
            for (int w = first_item; w < num_items; w += item_stride) {
                const int t = w / splits, ks = w - t * splits;
                const int a_row0 = (t % m_tiles) * ROWS_PER_TILE + (int)rank * TILE_M;
                const int b_row0 = (t / m_tiles) * P_BN + (PAIR ? (int)rank * (P_BN / 2) : 0);
                const int kb0 = ks * p.kb_per_split, kb1 = min(nkb, kb0 + p.kb_per_split);
                bool ok = true;
                for (int kb = kb0; kb < kb1; kb += KPS, ++it) {
                    const int s = it % P_STAGES;
                    ok = mbar_wait(&empty_bar[s], ((it / P_STAGES) & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    if (PAIR) {
                        const int nk = min(KPS, kb1 - kb);
                        if (rank == 0) mbar_expect_tx(&full_bar[s], nk * 2 * (A_BYTES + B_BYTES));
                        for (int j = 0; j < nk; ++j) {
                            tma_load_2d_pair(a_tiles + (s * KPS + j) * A_BYTES, &map_a, (kb + j) * TILE_K, a_row0, full_of_first + s * 8);
                            tma_load_2d_pair(b_tiles + (s * KPS + j) * B_BYTES, &map_b, (kb + j) * TILE_K, b_row0, full_of_first + s * 8);
                        }
                    } else {
                        mbar_expect_tx(&full_bar[s], A_BYTES + B_BYTES);
                        tma_load_2d(a_tiles + s * A_BYTES, &map_a, kb * TILE_K, a_row0, &full_bar[s]);
                        tma_load_2d(b_tiles + s * B_BYTES, &map_b, kb * TILE_K, b_row0, &full_bar[s]);
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // One thread issues every MMA, and a lone thread runs its scalar instructions one after the other at
            // their full latency: a few dozen of them per block of K cost more than the four MMAs themselves.  So
            // the loop carries what it needs in registers: the stage's two operand descriptors (advanced by
            // constants; the address field of a descriptor is the shared-memory address / 16), the addresses of its
            // barriers, its phase bit.
            constexpr uint32_t idesc = idesc_bf16(ROWS_PER_TILE, P_BN);
            constexpr uint64_t A_STEP = A_BYTES >> 4, B_STEP = B_BYTES >> 4, K_STEP = (UMMA_K * 2) >> 4;
            const uint64_t da0 = desc_kmajor(smem_u32(a_tiles)), db0 = desc_kmajor(smem_u32(b_tiles));
            const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
            uint64_t da = da0, db = db0;
            uint32_t full = full0, empty = empty0, phase = 0;
            int s = 0, local = 0;
            bool ok = true;
            for (int w = first_item; w < num_items && ok; w += item_stride, ++local) {
                const int ks = w % splits;
                const int kb0 = ks * p.kb_per_split, kb1 = min(nkb, kb0 + p.kb_per_split);
                const int buf = local & 1;
                ok = mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag);   // the epilogue has drained it
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * P_BN;
                for (int kb = kb0; kb < kb1; kb += KPS) {
                    if (!mbar_try_wait_addr(full, phase)) {
                        ok = mbar_wait_addr(full, phase, abort_flag);
                        if (!ok) break;
                    }
                    if (PAIR) {
                        const int nk = min(KPS, kb1 - kb);
                        for (int j = 0; j < nk; ++j) {
                            const uint64_t ja = da + j * A_STEP, jb = db + j * B_STEP;
                            if (kb == kb0 && j == 0) umma2_bf16_first(acc, ja, jb, idesc);
                            else umma2_bf16_acc(acc, ja, jb, idesc);
                            umma2_bf16_acc(acc, ja + K_STEP, jb + K_STEP, idesc);
                            umma2_bf16_acc(acc, ja + 2 * K_STEP, jb + 2 * K_STEP, idesc);
                            umma2_bf16_acc(acc, ja + 3 * K_STEP, jb + 3 * K_STEP, idesc);
                        }
                        umma2_commit_both(empty);            // frees the stage in both CTAs
                    } else {
                        if (kb == kb0) umma_bf16_first(acc, da, db, idesc);
                        else umma_bf16_acc(acc, da, db, idesc);
                        umma_bf16_acc(acc, da + K_STEP, db + K_STEP, idesc);
                        umma_bf16_acc(acc, da + 2 * K_STEP, db + 2 * K_STEP, idesc);
                        umma_bf16_acc(acc, da + 3 * K_STEP, db + 3 * K_STEP, idesc);
                        umma_commit_addr(empty);
                    }
                    if (++s == P_STAGES) {
                        s = 0; da = da0; db = db0; full = full0; empty = empty0; phase ^= 1;
                    } else {
                        da += KPS * A_STEP; db += KPS * B_STEP; full += 8; empty += 8;
                    }
                }
                if (ok) {
                    if (PAIR) umma2_commit_both(smem_u32(&acc_full[buf]));
                    else umma_commit(&acc_full[buf]);
                }
            }
        }
    } else {
        const int quarter = warp & 3;                 // the TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;             // which half of the tile's columns it drains
        const int row = quarter * 32 + lane;
        int local = 0;
        constexpr int SEPI = epi_is_rope(EPI) ? LLB_EPI_STORE : EPI;
        // the SiLU*mul row of 64 outputs needs 128 accumulator columns per warp, which only the wide tile has
        const bool staged = p.tma_out != 0 && !epi_is_rope(EPI) && (EPI != LLB_EPI_SWIGLU || P_BN == 256);
        uint8_t* my_stage = out_tiles + (warp - 2) * 4096;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t acc_empty_of_first = PAIR ? mapa_u32(smem_u32(&acc_empty[0]), 0) : 0u;
        for (int w = first_item; w < num_items; w += item_stride, ++local) {
            const int t = w / splits;
            const int buf = local & 1;
            const int a_row0 = (t % m_tiles) * ROWS_PER_TILE + (int)rank * TILE_M, b_row0 = (t / m_tiles) * P_BN;
            if (!mbar_wait(&acc_full[buf], (local >> 1) & 1, abort_flag)) break;      // uniform over the warp
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool direct = EPI == LLB_EPI_RESIDUAL && p.direct != 0;      // uniform over the grid
            if (splits == 2 && !direct) {
                // Two pieces: each finishes one half of the tile's columns.  The warps whose half belongs to the other
                // piece first give their part of the accumulator away through memory and raise a flag; giving never
                // waits.  Then every warp takes a share of the block's own half: it waits for the other piece's part,
                // adds it to its own (a + b, whichever piece it is) and runs the epilogue.  The two pieces are
                // neighbours in the list of work items and every block of the grid is resident, so the wait ends; it
                // is bounded all the same.  The flag counts the two warps that have yet to read.
                const int ks = w - t * 2;
                constexpr int HALF_COLS = P_BN / 2;
                const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P_BN);
                if (half != ks) {
                    float* dst = p.partials + (size_t)w * TILE_M * HALF_COLS + row;      // [column][row]
#pragma unroll 1
                    for (int c0 = 0; c0 < HALF_COLS; c0 += 32) {
                        uint32_t r[32];
                        tmem_ld32_nowait(lane_base + half * HALF_COLS + c0, r);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 32; ++j) dst[(size_t)(c0 + j) * TILE_M] = __uint_as_float(r[j]);
                    }
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicExch(&p.counters[t * 8 + ks * 4 + quarter], 2);
                }
                int* flag = &p.counters[t * 8 + (1 - ks) * 4 + quarter];
                int there = 0;
                if (lane == 0) {
                    const long long t0 = clock64();
                    for (unsigned spins = 0;; ++spins) {
                        if (atomicAdd(flag, 0) != 0) { there = 1; break; }
                        if ((spins & 63u) == 63u && (*abort_flag || clock64() - t0 > WAIT_LIMIT_CYCLES)) {
                            *abort_flag = 1;
                            break;
                        }
                        __nanosleep(40);
                    }
                }
                there = __shfl_sync(0xffffffffu, there, 0);
                __threadfence();
                const float* src = p.partials + (size_t)(t * 2 + 1 - ks) * TILE_M * HALF_COLS + row;
                const int share0 = (half == ks) ? 0 : HALF_COLS / 2;          // the warp's columns of the block's own half
#pragma unroll 1
                for (int c0 = share0; c0 < share0 + HALF_COLS / 2; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32_nowait(lane_base + ks * HALF_COLS + c0, r);
                    float other[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) other[j] = there ? __ldcg(src + (size_t)(c0 + j) * TILE_M) : 0.0f;
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + other[j]);
                    if (there) {
                        if (staged && (HALF_COLS / 2) % (StagedOut<SEPI>::PIECES * 32) == 0)
                            staged_chunk<SEPI>(p, &map_out, my_stage, lane, a_row0 + quarter * 32, b_row0 + ks * HALF_COLS + c0,
                                               ((c0 - share0) >> 5) % StagedOut<SEPI>::PIECES, r);
                        else
                            epilogue_row<SEPI, 32>(p, a_row0 + row, b_row0 + ks * HALF_COLS + c0, r);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
                    if (there) atomicSub(flag, 1);
                }
                continue;
            }
            if (splits > 1 && !direct) {
                // This split's accumulator goes to the meeting place; the warp that arrives last at its
                // region of the tile (32 rows x half the columns) adds the splits up in their order, so the
                // sum does not depend on who came last, and runs the epilogue.
                // Layout [item][column][row]: the 32 lanes of a warp (32 rows) write and read 128 contiguous bytes.
                float* mine = p.partials + (size_t)w * TILE_M * P_BN + row;
#pragma unroll 1
                for (int c0 = half * (P_BN / 2); c0 < (half + 1) * (P_BN / 2); c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32_nowait(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P_BN + c0), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) mine[(size_t)(c0 + j) * TILE_M] = __uint_as_float(r[j]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
                    last = atomicAdd(&p.counters[t * 8 + (warp - 2)], 1) == splits - 1;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    const float* first = p.partials + (size_t)(t * splits) * TILE_M * P_BN + row;
#pragma unroll 1
                    for (int c0 = half * (P_BN / 2); c0 < (half + 1) * (P_BN / 2); c0 += 32) {
                        float acc[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = 0.0f;
                        for (int i = 0; i < splits; ++i) {
                            const float* src = first + ((size_t)i * P_BN + c0) * TILE_M;
#pragma unroll
                            for (int j = 0; j < 32; ++j) acc[j] += __ldcg(src + (size_t)j * TILE_M);
                        }
                        epilogue_row<(epi_is_rope(EPI) ? LLB_EPI_STORE : EPI), 32>(
                            p, a_row0 + row, b_row0 + c0, *reinterpret_cast<const uint32_t(*)[32]>(&acc[0]));
                    }
                    if (lane == 0) p.counters[t * 8 + (warp - 2)] = 0;
                }
                continue;
            }
            if (epi_is_rope(EPI)) {
                // 64 columns at a time: a head of 64 with both members of every rotary pair, or half of a head of 128
#pragma unroll 1
                for (int c0 = half * (P_BN / 2); c0 < (half + 1) * (P_BN / 2); c0 += 64) {
                    uint32_t r0[32], r1[32];
                    const uint32_t ta = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P_BN + c0);
                    tmem_ld32_nowait(ta, r0);
                    tmem_ld32_nowait(ta + 32, r1);
                    if (EPI == EPI_ROPE128) {      // the pairs' other members: the same columns of the head's other half (the tile is one head)
                        uint32_t p0[32], p1[32];
                        const uint32_t tp = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P_BN + (c0 ^ 64));
                        tmem_ld32_nowait(tp, p0);
                        tmem_ld32_nowait(tp + 32, p1);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        epilogue_rope_warp<128>(p, &map_out, my_stage, p.tma_out != 0, lane, a_row0 + quarter * 32, b_row0 + c0,
                                                r0, r1, p0, p1);
                    } else {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        epilogue_rope_warp<64>(p, &map_out, my_stage, p.tma_out != 0, lane, a_row0 + quarter * 32, b_row0 + c0,
                                               r0, r1, r0, r1);
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = half * (P_BN / 2); c0 < (half + 1) * (P_BN / 2); c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32_nowait(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * P_BN + c0), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (staged)
                        staged_chunk<SEPI>(p, &map_out, my_stage, lane, a_row0 + quarter * 32, b_row0 + c0,
                                           ((c0 - half * (P_BN / 2)) >> 5) % StagedOut<SEPI>::PIECES, r);
                    else
                        epilogue_row<SEPI, 32>(p, a_row0 + row, b_row0 + c0, r);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(acc_empty_of_first + buf * 8);      // the pair's accumulators are drained together
                else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
            }
        }
    }

    if (warp >= 2 && lane == 0) tma_store_wait_all();       // this warp's TMA stores have been written
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync_all();       // neither CTA leaves (or frees tensor memory) while the other may still use it
    if (abort_s && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 5);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (PAIR) tmem_dealloc2(tmem_base, TMEM_COLS);
        else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct MapKey {
    const void* ptr;
    int rows, K, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && K == o.K && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.K << 20) ^ ((size_t)k.box_rows << 40);
    }
};

// A tensor map over a row-major bf16 matrix [rows, K] with boxes of box_rows x 64 and the 128-byte swizzle.
int make_map(const void* ptr, int rows, int K, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, K, box_rows};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return 0;
        }
    }
    t5::EncodeTiledFn fn = t5::encode_tiled_fn();
    if (!fn) return llb_fail("gemm_tcgen05: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return llb_fail("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

template <int BN>
constexpr size_t smem_bytes() {
    return (size_t)STAGES * (TILE_M * TILE_K * 2 + BN * TILE_K * 2) + (2 * STAGES + 1) * 8 + 16 + 1024;
}

template <int BN, int EPI, bool SWAP>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = smem_bytes<BN>();
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI, SWAP>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return llb_fail("gemm_tcgen05: cannot opt in to %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
        configured = true;
    }
    gemm_tcgen05_kernel<BN, EPI, SWAP><<<grid, NUM_THREADS, smem, stream>>>(ma, mb, p);
    return llb_check_launch("gemm_tcgen05");
}

template <int EPI, int P_BN, bool PAIR = false>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const GemmParams& p,
                      cudaStream_t stream) {
    constexpr int KPS = PAIR ? 2 : 1;
    constexpr int P_STAGES = PAIR ? 3 : (P_BN == 256 ? 4 : 6);
    constexpr size_t smem = (size_t)P_STAGES * KPS * (TILE_M * TILE_K * 2 + (PAIR ? P_BN / 2 : P_BN) * TILE_K * 2) + 8 * 4096 + 1024;
    static bool configured = false;
    static int num_sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<EPI, P_BN, PAIR>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return llb_fail("gemm_tcgen05: cannot opt in to %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int tiles = llb_ceil_div(p.M, PAIR ? 2 * TILE_M : TILE_M) * llb_ceil_div(p.N, P_BN) * p.splits;
    const int units = PAIR ? num_sms / 2 : num_sms;              // blocks, or pairs of blocks
    const int grid = (tiles < units ? tiles : units) * (PAIR ? 2 : 1);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(P_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = PAIR ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_persistent_kernel<EPI, P_BN, PAIR>, ma, mb, mo, p);
    if (e != cudaSuccess) return llb_fail("gemm_tcgen05: launch failed: %s", cudaGetErrorString(e));
    return llb_check_launch("gemm_tcgen05_persistent");
}

// LLB_GEMM_PAIR=0 in the environment keeps the single-CTA tiles (for comparisons).
bool pair_tiles_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("LLB_GEMM_PAIR");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// Features from which the pair tiles are used (LLB_GEMM_PAIR_MIN_N in the environment, for comparisons).  Measured at
// 2,048 rows: 1,536 features (o_proj and down at the 1.5B sizes, which single tiles of 128 x 128 run in two uneven rounds,
// each waiting for operands) take 6.6 ms a prefill step with pair tiles against 8.1 ms without; 896 features gain nothing.
int pair_min_features() {
    static int n = -1;
    if (n < 0) {
        const char* e = getenv("LLB_GEMM_PAIR_MIN_N");
        n = e ? atoi(e) : 1024;
        if (n < 256) n = 256;
    }
    return n;
}

template <int P_BN, bool PAIR = false>
int dispatch_persistent(int epi, const CUtensorMap& ma, const CUtensorMap& mb, GemmParams p, cudaStream_t s) {
    // The output's tensor map for the staged epilogue: rows of 128 bytes (32 floats or 64 bf16) x 32 rows, 128-byte
    // swizzle.  Outputs whose base or row pitch is not a multiple of 16 bytes keep the direct stores.
    CUtensorMap mo = ma;
    {
        const bool f32 = epi == LLB_EPI_STORE_F32 || epi == LLB_EPI_RESIDUAL;
        const void* base = epi == LLB_EPI_RESIDUAL ? (const void*)p.residual : (const void*)p.out;
        const long long cols = epi == LLB_EPI_SWIGLU ? p.N / 2 : p.N;
        const long long pitch = cols * (f32 ? 4 : 2);
        t5::EncodeTiledFn fn = t5::encode_tiled_fn();
        if (fn && ((uintptr_t)base % 16 == 0) && pitch % 16 == 0 && (epi != LLB_EPI_SWIGLU || p.N % 2 == 0)) {
            cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)p.M};
            cuuint64_t strides[1] = {(cuuint64_t)pitch};
            cuuint32_t box[2] = {f32 ? 32u : 64u, 32u};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = fn(&mo, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return llb_fail("gemm_tcgen05: cuTensorMapEncodeTiled (output) failed with code %d", (int)r);
            p.tma_out = 1;
        }
    }
    // Pieces of a residual contraction without bias add their parts through the TMA store path themselves: float adds in
    // L2 commute up to rounding, and the meeting place (a round trip of every accumulator through memory, and a wait of
    // one piece for the other) is saved.
    p.direct = (epi == LLB_EPI_RESIDUAL && p.splits > 1 && p.bias == nullptr && p.tma_out) ? 1 : 0;
    if (PAIR && p.splits > 1 && !p.direct) return llb_fail("gemm_tcgen05: pair tiles cannot meet pieces along K");
    switch (epi) {
        case LLB_EPI_STORE: return launch_persistent<LLB_EPI_STORE, P_BN, PAIR>(ma, mb, mo, p, s);
        case LLB_EPI_STORE_F32: return launch_persistent<LLB_EPI_STORE_F32, P_BN, PAIR>(ma, mb, mo, p, s);
        case LLB_EPI_RESIDUAL: return launch_persistent<LLB_EPI_RESIDUAL, P_BN, PAIR>(ma, mb, mo, p, s);
        case LLB_EPI_SWIGLU: return launch_persistent<LLB_EPI_SWIGLU, P_BN, PAIR>(ma, mb, mo, p, s);
    }
    return llb_fail("gemm_tcgen05: unknown epilogue %d", epi);
}

template <int BN, bool SWAP>
int dispatch_epi(int epi, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t s) {
    switch (epi) {
        case LLB_EPI_STORE: return launch<BN, LLB_EPI_STORE, SWAP>(ma, mb, p, grid, s);
        case LLB_EPI_STORE_F32: return launch<BN, LLB_EPI_STORE_F32, SWAP>(ma, mb, p, grid, s);
        case LLB_EPI_RESIDUAL: return launch<BN, LLB_EPI_RESIDUAL, SWAP>(ma, mb, p, grid, s);
        case LLB_EPI_SWIGLU: return launch<BN, LLB_EPI_SWIGLU, SWAP>(ma, mb, p, grid, s);
    }
    return llb_fail("gemm_tcgen05: unknown epilogue %d", epi);
}

}  // namespace

// A [M,K] bf16, W [N,K] bf16, both row-major with K a multiple of 8 and 16-byte aligned bases;
// bias [N] float or null.  `out`: [M,N] bf16 (STORE), [M,N] float (STORE_F32), [M,N/2] bf16 (SWIGLU, N even);
// `residual`: [M,N] float (RESIDUAL).  split_k > 1 cuts K into that many pieces.  Up to 128 rows this is for
// RESIDUAL only (atomic adds).  Beyond, any epilogue may be split: the pieces meet in `partials` (at least
// llb_gemm_tcgen05_partial_floats(M, N, split_k) floats) and `counters` (8 ints per tile of 128 rows x 256 (N > 128)
// or 128 features, zero before the call and zero again after it), and the piece that arrives last adds them up
// in their order, so the result does not depend on the order of arrival (except a RESIDUAL contraction without bias
// whose output row is a multiple of 16 bytes: its pieces add themselves into `residual`, float adds that commute up
// to rounding, and the meeting place is not touched).  error_flag: one int that the kernel
// raises if a wait inside it ran out of time (the result is then invalid), or null.
LLB_EXPORT int llb_gemm_tcgen05(const void* A, const void* W, const float* bias, void* out, float* residual,
                                int epilogue, int M, int N, int K, int split_k, float* partials, int* counters,
                                int* error_flag, cudaStream_t stream) {
    if (M == 0) return 0;
    LLB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
    LLB_REQUIRE(K % 8 == 0, "gemm_tcgen05: K=%d is not a multiple of 8 (rows must be 16-byte multiples for TMA)", K);
    LLB_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tcgen05: operands must be 16-byte aligned");
    LLB_REQUIRE(epilogue != LLB_EPI_SWIGLU || N % 2 == 0, "gemm_tcgen05: SwiGLU epilogue needs an even N, got %d", N);
    LLB_REQUIRE(epilogue != LLB_EPI_RESIDUAL || residual != nullptr, "gemm_tcgen05: residual epilogue without residual");
    LLB_REQUIRE(epilogue == LLB_EPI_RESIDUAL || out != nullptr, "gemm_tcgen05: output pointer is null");
    LLB_REQUIRE(split_k >= 1 && (split_k == 1 || epilogue == LLB_EPI_RESIDUAL || M > 128),
                "gemm_tcgen05: split_k=%d with up to 128 rows needs the residual epilogue", split_k);
    LLB_REQUIRE(split_k == 1 || M <= 128 || (partials && counters),
                "gemm_tcgen05: split_k=%d beyond 128 rows needs the meeting place", split_k);
    GemmParams p = {};
    p.splits = 1;
    p.out = out; p.residual = residual; p.bias = bias; p.M = M; p.N = N; p.K = K;
    p.num_kb = llb_ceil_div(K, TILE_K);
    if (split_k > p.num_kb) split_k = p.num_kb;
    p.kb_per_split = llb_ceil_div(p.num_kb, split_k);
    split_k = llb_ceil_div(p.num_kb, p.kb_per_split);
    p.error_flag = error_flag;
    const bool swap = M <= 128;
    CUtensorMap ma, mb;
    int rc;
    if (swap) {
        const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        if ((rc = make_map(W, N, K, TILE_M, &ma))) return rc;
        if ((rc = make_map(A, M, K, bn, &mb))) return rc;
        dim3 grid(llb_ceil_div(N, TILE_M), 1, split_k);
        switch (bn) {
            case 16: return dispatch_epi<16, true>(epilogue, ma, mb, p, grid, stream);
            case 32: return dispatch_epi<32, true>(epilogue, ma, mb, p, grid, stream);
            case 64: return dispatch_epi<64, true>(epilogue, ma, mb, p, grid, stream);
            default: return dispatch_epi<128, true>(epilogue, ma, mb, p, grid, stream);
        }
    }
    constexpr int BN = 128;
    if ((rc = make_map(A, M, K, TILE_M, &ma))) return rc;
    p.splits = split_k;
    p.partials = partials;
    p.counters = counters;
    // Many rows and many features: pairs of CTAs on tiles of 256 x 256, each CTA loading its own rows and half of
    // the weights' tile.
    if (split_k == 1 && N >= pair_min_features() && M >= 512 && pair_tiles_enabled()) {
        if ((rc = make_map(W, N, K, 128, &mb))) return rc;
        return dispatch_persistent<256, true>(epilogue, ma, mb, p, stream);
    }
    // The wide tile wins wherever its padding of N costs little, and always when K is split (few tiles are what
    // splitting is for).
    if (N >= 2048 || (split_k > 1 && N > 128)) {
        if ((rc = make_map(W, N, K, 256, &mb))) return rc;
        return dispatch_persistent<256>(epilogue, ma, mb, p, stream);
    }
    if ((rc = make_map(W, N, K, BN, &mb))) return rc;
    return dispatch_persistent<128>(epilogue, ma, mb, p, stream);
}

// Floats of the meeting place that llb_gemm_tcgen05 needs beyond 128 rows with K cut into split_k pieces.
LLB_EXPORT long long llb_gemm_tcgen05_partial_floats(int M, int N, int split_k) {
    if (split_k <= 1 || M <= 128) return 0;
    const int bn = N > 128 ? 256 : 128;
    return (long long)llb_ceil_div(M, TILE_M) * llb_ceil_div(N, bn) * split_k * TILE_M * bn;
}
// Counters (ints) of that meeting place.
LLB_EXPORT long long llb_gemm_tcgen05_counters(int M, int N, int split_k) {
    if (split_k <= 1 || M <= 128) return 0;
    return (long long)llb_ceil_div(M, TILE_M) * llb_ceil_div(N, N > 128 ? 256 : 128) * 8;
}

// The q/k/v projection of a prompt portion with its whole epilogue on the tensor-core kernel: bias, NeoX rotation
// of q and k by rope_table [hd/2, M] of (cos, sin) (pair-major: llb_rope_table with transposed = 1), q to q_out
// [M, Hq*hd], k and v to the cache rows slot_mapping[m].
// Heads of 64 or 128 with the whole head rotated; N = (Hq + 2*Hkv) * hd.
LLB_EXPORT int llb_gemm_tcgen05_rope(const void* A, const void* W, const float* bias, int M, int N, int K,
                                     const float* rope_table, const int* slot_mapping, void* q_out, void* k_cache,
                                     void* v_cache, int Hq, int Hkv, int hd, int* error_flag, cudaStream_t stream) {
    if (M == 0) return 0;
    LLB_REQUIRE(M > 0 && K % 8 == 0 && (hd == 64 || hd == 128) && N == (Hq + 2 * Hkv) * hd && Hq > 0 && Hkv > 0,
                "gemm_tcgen05_rope: unsupported shape M=%d N=%d K=%d heads %d/%d of %d", M, N, K, Hq, Hkv, hd);
    LLB_REQUIRE(rope_table && q_out && k_cache && v_cache && slot_mapping, "gemm_tcgen05_rope: null argument");
    LLB_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
                ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) && ((uintptr_t)rope_table % 8 == 0),
                "gemm_tcgen05_rope: operands must be 16-byte aligned");
    GemmParams p = {};
    p.splits = 1;
    p.bias = bias; p.M = M; p.N = N; p.K = K;
    p.num_kb = llb_ceil_div(K, TILE_K);
    p.kb_per_split = p.num_kb;
    p.error_flag = error_flag;
    p.rope_table = (const float2*)rope_table; p.slot_mapping = slot_mapping;
    p.q_out = (__nv_bfloat16*)q_out; p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
    p.Hq = Hq; p.Hkv = Hkv;
    CUtensorMap ma, mb;
    int rc;
    if ((rc = make_map(A, M, K, TILE_M, &ma))) return rc;
    if ((rc = make_map(W, N, K, 128, &mb))) return rc;
    // q leaves through TMA stores of 64 bf16 x 32 rows (its row pitch, Hq * hd * 2 bytes, always allows it)
    CUtensorMap mq = ma;
    {
        t5::EncodeTiledFn fn = t5::encode_tiled_fn();
        if (!fn) return llb_fail("gemm_tcgen05_rope: cuTensorMapEncodeTiled is not available from the driver");
        cuuint64_t dims[2] = {(cuuint64_t)Hq * hd, (cuuint64_t)M};
        cuuint64_t strides[1] = {(cuuint64_t)Hq * hd * 2};
        cuuint32_t box[2] = {64u, 32u};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q_out, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return llb_fail("gemm_tcgen05_rope: cuTensorMapEncodeTiled (q) failed with code %d", (int)r);
        p.tma_out = 1;
    }
    // Many rows and features: pair tiles, as the plain contraction takes them (each CTA loads 128 of the tile's 256 weight
    // rows, which is the box of `mb` already).  Measured at 2,048 rows: 4,608 features (the 7B sizes) 25.0 ms a prefill step
    // against 26.1; 2,048 features (1.5B) and 1,152 (0.5B) gain nothing, so the rule starts at 4,096.
    if (M >= 512 && N >= 4 * pair_min_features() && pair_tiles_enabled())
        return hd == 128 ? launch_persistent<EPI_ROPE128, 256, true>(ma, mb, mq, p, stream)
                         : launch_persistent<EPI_ROPE64, 256, true>(ma, mb, mq, p, stream);
    return hd == 128 ? launch_persistent<EPI_ROPE128, 128>(ma, mb, mq, p, stream)
                     : launch_persistent<EPI_ROPE64, 128>(ma, mb, mq, p, stream);
}
