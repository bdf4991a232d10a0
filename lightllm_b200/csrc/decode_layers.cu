// The layers of a decode step (at most 64 rows, one token per request) as ONE persistent kernel.
//
// Launched kernel by kernel, a layer of a decode step is a chain of dependent launches (norm, q/k/v, attention,
// o_proj, norm, gate/up, down: src/engine/engine_server.cpp:1526-1881 runs them one by one too), each of which drains
// before the next starts, and the memory system idles in between: the step is paced by the chain, not by the bytes.
// Here one block per SM stays resident for all layers.  Every block owns a fixed share of the weight tiles of every
// contraction of every layer and streams them through one TMA ring that runs ahead across stage and layer
// boundaries (the weights depend on nothing), so HBM keeps working while a stage's results travel.  The stages of a
// layer meet on a counter in global memory (bounded waits, an error flag instead of a hang):
//
//   S1  q/k/v     B operand = bf16(residual * norm1_w) built by the block for its K range; the tile's partial sums are
//                 added (red.add) into qkv_acc [M, Nqkv]; the blocks that own the first row tile also add the rows' sums
//                 of squares into ss1 [M].  The norm's 1/rms is applied by the reader: (x * w) W^T * inv = norm(x) W^T.
//   S2  attention one item = (request, kv head, piece of the keys): q = rotate(qkv_acc * inv + bias) for the group's
//                 heads, keys and values from the request's pages (cp.async, mma.sync m16n8k16 as the decode attention
//                 kernel of this library); the piece that ends at the new token rotates and stores its k and v into the
//                 cache and attends to them from registers.  Partial (acc, m, l) per piece go to scratch.
//   S3  o_proj    B operand = the pieces of a head merged (softmax weights) as bf16; result added into the residual.
//   S4  gate/up   as S1 with norm2; sums into gu_acc [M, 2 I] and ss2 [M].
//   S5  down      B operand = bf16(silu(gate * inv) * (up * inv)); result added into the residual.
//
// Formulas: norm src/ops/norm.cu:19-55, rotation src/ops/rope.cu:54-59 (every pair), attention
// src/kv_cache/paged_attention.cu:115,153-163 (exact acc / l, the token's own key visible), SiLU
// src/ops/elementwise.cu:27-33.  Sums of squares, softmax, rotation angles and the residual sum are float.
//
// Roles of a block (320 threads): warp 0 requests weight tiles (TMA, no multicast), warp 1 issues tcgen05.mma into two
// accumulators in tensor memory, warps 2-9 build B operands, run the attention items, drain the accumulators and meet
// the other blocks.  A role is one warp per scheduler at most, so what it runs between two waits is kept short: a
// dependent instruction issues every few cycles, and a thousand of them are microseconds.  The launch is cooperative, so all blocks are resident; every wait has a time limit.
#include <math.h>

#include "tcgen05_common.cuh"
#include "warp_mma.cuh"

namespace {

using namespace t5;
using namespace wm;

constexpr int TILE_M = 128;
constexpr int TILE_K = 64;
constexpr uint32_t A_BYTES = TILE_M * TILE_K * 2;
constexpr int NUM_THREADS = 320;
constexpr int WORKERS = 256;          // warps 2-9
constexpr int KV_THREADS = 128;       // the workers that walk an attention item's keys (four warps with their own tiles)
constexpr int ATTN_BYTES = 64 * 1024;      // per-warp K/V buffers of the attention items, then their merge area
constexpr int MAX_GROUPS = 4;
constexpr int MAX_SPLITS = 32;

struct LayerDesc {
    CUtensorMap map_qkv, map_o, map_gu, map_down;      // weights [N, K] bf16, boxes of 128 rows x 64 columns
    const float* b_qkv;              // [Nqkv] or null
    const void* norm1_w;             // [D] bf16 or float
    const void* norm2_w;
    __nv_bfloat16* k_cache;          // [slots, Hkv, hd]
    __nv_bfloat16* v_cache;
    float eps1, eps2;
    int norm_w_bf16;
    int window;                      // 0: every earlier key is visible
    int group;                       // which block table / slot mapping of the step
    int pad_[5];
};
static_assert(sizeof(LayerDesc) % 64 == 0, "tensor maps inside an array of descriptors must stay 64-byte aligned");

struct FusedParams {
    const LayerDesc* layers;
    int num_layers;
    float* residual;                 // [M, D]
    int M, D, Hq, Hkv, hd, I, rotary_dim, interleaved;
    float scale_log2e;
    const float2* rope_table;        // [M, rotary_dim / 2] (cos, sin)
    const int* span_pos;             // [M] position of each request's token
    const int* block_tables[MAX_GROUPS];     // [M, max_pages]
    const int* slot_mapping[MAX_GROUPS];     // [M]
    int max_pages, page_size, nsplit;
    float* qkv_acc;                  // [M, Nqkv]
    float* gu_acc;                   // [M, 2 I]
    float* ss1;                      // [64]
    float* ss2;                      // [64]
    float* part_acc;                 // [M, Hkv, nsplit, G, hd]
    float* part_ml;                  // [M, Hkv, nsplit, G, 2]
    unsigned* sync;                  // [0] arrivals at the stage barriers, [1] blocks that have finished
    int* error_flag;
    unsigned long long* timeline;    // null, or room for (label, cycle) pairs that one block writes at its milestones
    int timeline_block;
};

struct StageInfo {
    const CUtensorMap* map;
    int N, K, NT, NKB;
};
enum { ST_QKV = 0, ST_O = 1, ST_GU = 2, ST_DOWN = 3 };

__device__ __forceinline__ StageInfo stage_info(const FusedParams& p, const LayerDesc* L, int st) {
    StageInfo s;
    if (st == ST_QKV) { s.map = &L->map_qkv; s.N = (p.Hq + 2 * p.Hkv) * p.hd; s.K = p.D; }
    else if (st == ST_O) { s.map = &L->map_o; s.N = p.D; s.K = p.Hq * p.hd; }
    else if (st == ST_GU) { s.map = &L->map_gu; s.N = 2 * p.I; s.K = p.D; }
    else { s.map = &L->map_down; s.N = p.D; s.K = p.I; }
    s.NT = (s.N + TILE_M - 1) / TILE_M;
    s.NKB = (s.K + TILE_K - 1) / TILE_K;
    return s;
}
// This block's share of a stage's (row tile, K block) pairs, row tile major: [lo, hi).
__device__ __forceinline__ void stage_range(const StageInfo& s, long long& lo, long long& hi) {
    const long long W = (long long)s.NT * s.NKB;
    lo = W * blockIdx.x / gridDim.x;
    hi = W * (blockIdx.x + 1) / gridDim.x;
}
// The same for every layer, so it is worked out once per launch (the divisions are slow for a lone warp) and kept
// in shared memory: where the block's tiles of each stage begin, how many they are, and its parts of the scratch arrays.
struct BlockPlan {
    int nt_first[4], kb_first[4], n_tiles[4], units[4], N[4], NKB[4];
    int zero_qkv_lo, zero_qkv_hi, zero_gu_lo, zero_gu_hi;
};
__device__ __forceinline__ void make_plan(const FusedParams& p, BlockPlan& plan) {
    for (int st = 0; st < 4; ++st) {
        const StageInfo si = stage_info(p, p.layers, st);
        long long lo, hi;
        stage_range(si, lo, hi);
        plan.nt_first[st] = (int)(lo / si.NKB);
        plan.kb_first[st] = (int)(lo - (long long)plan.nt_first[st] * si.NKB);
        plan.n_tiles[st] = (int)(hi - lo);
        plan.units[st] = hi > lo ? (int)((plan.kb_first[st] + (hi - lo) - 1) / si.NKB) + 1 : 0;
        plan.N[st] = si.N;
        plan.NKB[st] = si.NKB;
    }
    const long long nq = (long long)p.M * (p.Hq + 2 * p.Hkv) * p.hd, ng = (long long)p.M * 2 * p.I;
    plan.zero_qkv_lo = (int)(nq * blockIdx.x / gridDim.x); plan.zero_qkv_hi = (int)(nq * (blockIdx.x + 1) / gridDim.x);
    plan.zero_gu_lo = (int)(ng * blockIdx.x / gridDim.x); plan.zero_gu_hi = (int)(ng * (blockIdx.x + 1) / gridDim.x);
}
__device__ __forceinline__ const CUtensorMap* stage_map(const LayerDesc* L, int st) {
    return st == ST_QKV ? &L->map_qkv : st == ST_O ? &L->map_o : st == ST_GU ? &L->map_gu : &L->map_down;
}

__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
// Milestones of block 0 for tuning, in cycles of its SM: label = layer * 100 + stage * 10 + what (1 operands built,
// 2 drained / items done, 3 past the barrier; 5-7 inside a batch: slots free, operands stored, arrivals made).  Off (a null pointer) in normal use.
__device__ __forceinline__ void stamp(const FusedParams& p, unsigned& n, int label) {
    if (p.timeline != nullptr && (int)blockIdx.x == p.timeline_block && threadIdx.x == 64) {
        p.timeline[2 * n] = (unsigned long long)label;
        p.timeline[2 * n + 1] = (unsigned long long)clock64();
        ++n;
    }
}
__device__ __forceinline__ void red_add(float* addr, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* addr) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_inc(unsigned* addr) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(addr) : "memory");
}

// All blocks meet: arrivals are counted in sync[0], which only grows while the kernel runs (the block that finishes
// last sets it back to zero).  One worker thread arrives (a release: what the workers wrote before is visible to
// whoever sees the count) and polls; the wait gives up after the library's time limit or as soon as any block has
// raised the error flag.
__device__ __forceinline__ void grid_arrive(const FusedParams& p, unsigned& epoch) {
    ++epoch;
    worker_sync();
    if (threadIdx.x == 64) red_release_inc(p.sync);
}
// Between the two halves a block does what nobody waits for (clearing sums for a later stage, asking for cache rows).
__device__ __forceinline__ void grid_wait(const FusedParams& p, unsigned epoch, volatile int* abort_flag) {
    if (threadIdx.x == 64) {
        const unsigned target = epoch * gridDim.x;
        if (!*abort_flag) {
            const long long t0 = clock64();
            for (unsigned spins = 1; ld_acquire(p.sync) < target; ++spins) {
                if ((spins & 63u) == 0u) {
                    if (*(volatile int*)p.error_flag != 0) { *abort_flag = 1; break; }
                    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                        *abort_flag = 1;
                        atomicExch(p.error_flag, 7);
                        break;
                    }
                }
            }
        }
    }
    worker_sync();
}
__device__ __forceinline__ void grid_barrier(const FusedParams& p, unsigned& epoch, volatile int* abort_flag) {
    grid_arrive(p, epoch);
    grid_wait(p, epoch, abort_flag);
}

// ---- B operands: BN rows (tokens) x 64 columns of one K block, bf16, K-major with the 128-byte swizzle ------------
// A 16-byte chunk q (8 columns) of row m sits at m * 128 + ((q ^ (m & 7)) * 16).  Rows from M on are left as they
// are: the accumulator columns they produce are never read.
__device__ __forceinline__ void store_chunk(uint8_t* tile, int m, int q, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(tile + (uint32_t)m * 128 + ((q ^ (m & 7)) * 16)) =
        make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
// Consecutive tiles of one stage that are built together: tile t is K block (kb0 + t) mod NKB of row tile
// nt0 + (kb0 + t) / NKB and lives at ring position ring0 + t.
struct Batch {
    int kb0, nt0, n, NKB;
    uint32_t ring0;
};
// The builders keep R loads of a thread in flight before they use the first: one trip to memory for a batch, not one
// per tile.  A thread keeps its 16-byte chunk q of a row and walks over the batch's tiles, so there is no index
// arithmetic beyond a counter.  `live` is false after a wait has run out: nothing is loaded or stored then.

// x / (1 + e^-x) with the hardware's exponential and reciprocal: the result is rounded to bfloat16 right away.
__device__ __forceinline__ float silu_fast(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + fast_exp2(-1.4426950408889634f * x)));
    return x * r;
}
// The (tile, row) pairs of a batch are dealt over the threads' 32 row slots, eight threads (the 16-byte chunks) per
// pair: pair i is row i % M of tile i / M.  With few rows every thread still gets work.
// S1 / S4: bf16(x * norm_w) of the residual rows; the blocks that own row tile 0 add the rows' sums of squares there.
template <int STAGES, int R>
__device__ __forceinline__ void build_norm(const FusedParams& p, const void* norm_w, int norm_bf16, float* ss, const Batch& b,
                                           uint8_t* b_tiles, uint32_t b_bytes, bool live, int wt) {
    const int q = wt & 7, slot0 = wt >> 3, wslot = (wt & ~31) >> 3;
    const int pairs = b.n * p.M;
    for (int base = 0; base + wslot < pairs; base += R * (WORKERS / 8)) {       // warp-uniform: lanes exchange sums
        float4 xa[R], xb[R];
        uint4 w0[R], w1[R];
        int tile[R], row[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = base + r * (WORKERS / 8) + slot0;
            tile[r] = i / p.M;
            row[r] = i - tile[r] * p.M;
            xa[r] = xb[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            w0[r] = w1[r] = make_uint4(0u, 0u, 0u, 0u);
            int kb = b.kb0 + tile[r];
            while (kb >= b.NKB) kb -= b.NKB;
            const int k = kb * TILE_K + q * 8;
            if (live && i < pairs && k < p.D) {
                const float* x = p.residual + (size_t)row[r] * p.D + k;
                xa[r] = __ldcg(reinterpret_cast<const float4*>(x));
                xb[r] = __ldcg(reinterpret_cast<const float4*>(x + 4));
                if (norm_bf16) {
                    w0[r] = __ldg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)norm_w + k));
                } else {
                    w0[r] = __ldg(reinterpret_cast<const uint4*>((const float*)norm_w + k));
                    w1[r] = __ldg(reinterpret_cast<const uint4*>((const float*)norm_w + k + 4));
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = base + r * (WORKERS / 8) + slot0;
            const bool valid = live && i < pairs;
            float v[8] = {xa[r].x, xa[r].y, xa[r].z, xa[r].w, xb[r].x, xb[r].y, xb[r].z, xb[r].w};
            // the tile's row tile: tiles of row tile 0 carry the sums of squares (uniform over a pair's eight lanes)
            if (ss != nullptr && base + r * (WORKERS / 8) + wslot < pairs) {
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) sum = fmaf(v[j], v[j], sum);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if (valid && q == 0 && b.nt0 == 0 && b.kb0 + tile[r] < b.NKB) red_add(ss + row[r], sum);
            }
            if (valid) {
                float nw[8];
                if (norm_bf16) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w0[r]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(h[j]);
                        nw[2 * j] = f.x; nw[2 * j + 1] = f.y;
                    }
                } else {
                    const float* f0 = reinterpret_cast<const float*>(&w0[r]);
                    const float* f1 = reinterpret_cast<const float*>(&w1[r]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) { nw[j] = f0[j]; nw[4 + j] = f1[j]; }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= nw[j];
                store_chunk(b_tiles + ((b.ring0 + tile[r]) % STAGES) * b_bytes, row[r], q, v);
            }
        }
    }
}
// S5: silu(gate) * up of 64 intermediate columns from the interleaved sums of S4 (gate at 2j, up at 2j + 1).
template <int STAGES, int R>
__device__ __forceinline__ void build_swiglu(const FusedParams& p, float eps2, const Batch& b, uint8_t* b_tiles,
                                             uint32_t b_bytes, bool live, int wt) {
    const int q = wt & 7, slot0 = wt >> 3;
    const int pairs = b.n * p.M;
    for (int base = 0; base + slot0 < pairs; base += R * (WORKERS / 8)) {
        float4 t4[R][4];
        float ssv[R];
        int tile[R], row[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = base + r * (WORKERS / 8) + slot0;
            tile[r] = i / p.M;
            row[r] = i - tile[r] * p.M;
            ssv[r] = 1.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) t4[r][j] = make_float4(0.f, 0.f, 0.f, 0.f);
            int kb = b.kb0 + tile[r];
            while (kb >= b.NKB) kb -= b.NKB;
            const int j0 = kb * TILE_K + q * 8;
            if (live && i < pairs && j0 < p.I) {
                const float4* src = reinterpret_cast<const float4*>(p.gu_acc + (size_t)row[r] * 2 * p.I + 2 * j0);
#pragma unroll
                for (int j = 0; j < 4; ++j) t4[r][j] = __ldcg(src + j);
                ssv[r] = __ldcg(p.ss2 + row[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = base + r * (WORKERS / 8) + slot0;
            if (live && i < pairs) {
                const float inv = 1.0f / sqrtf(ssv[r] / (float)p.D + eps2);
                float out[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    out[2 * j] = silu_fast(t4[r][j].x * inv) * (t4[r][j].y * inv);
                    out[2 * j + 1] = silu_fast(t4[r][j].z * inv) * (t4[r][j].w * inv);
                }
                store_chunk(b_tiles + ((b.ring0 + tile[r]) % STAGES) * b_bytes, row[r], q, out);
            }
        }
    }
}
// S3: the attention output of 64 columns (one head, or half of one), its pieces merged by their softmax weights:
// out = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s.  The threads are dealt to (chunk, group of pieces) pairs;
// a thread merges its pieces in registers (their loads in flight together), the groups of a chunk meet in `stage`
// (12 floats per entry: m, l, -, -, eight sums), and one thread per chunk finishes.
constexpr int MERGE_FLOATS = 12;
template <int STAGES, int R>
__device__ __forceinline__ void build_merge(const FusedParams& p, const Batch& b, float* stage, uint8_t* b_tiles,
                                            uint32_t b_bytes, bool live, int wt) {
    const int G = p.Hq / p.Hkv, K = p.Hq * p.hd, cpt = p.M * 8;
    const int groups = cpt < WORKERS ? WORKERS / cpt : 1;       // threads per chunk
    const int grp = cpt < WORKERS ? wt / cpt : 0, c_first = cpt < WORKERS ? wt - grp * cpt : wt;
    int kb = b.kb0;
    for (int t = 0; t < b.n; ++t) {
        for (int c = c_first; c < cpt; c += WORKERS) {
            if (grp >= groups) break;
            const int m = c >> 3, q = c & 7, c0 = kb * TILE_K + q * 8;
            float mx = -INFINITY, l = 0.0f;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (live && c0 < K) {
                const int h = c0 / p.hd, d0 = c0 - h * p.hd, kvh = h / G, gi = h - kvh * G;
                const size_t first = ((size_t)(m * p.Hkv + kvh) * p.nsplit) * G + gi;      // piece sp: first + sp * G
                for (int sp0 = grp; sp0 < p.nsplit; sp0 += groups * R) {
                    float2 ml[R];
                    float4 a[R], bb[R];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const int sp = sp0 + r * groups;
                        ml[r] = make_float2(-INFINITY, 0.0f);
                        a[r] = bb[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (sp < p.nsplit) {
                            const size_t at = first + (size_t)sp * G;
                            ml[r] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + at * 2));
                            a[r] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + at * p.hd + d0));
                            bb[r] = __ldcg(reinterpret_cast<const float4*>(p.part_acc + at * p.hd + d0 + 4));
                        }
                    }
                    float mnew = mx;
#pragma unroll
                    for (int r = 0; r < R; ++r) mnew = fmaxf(mnew, ml[r].x);
                    if (mnew != -INFINITY) {
                        const float keep = mx == -INFINITY ? 0.0f : fast_exp2(mx - mnew);
                        l *= keep;
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] *= keep;
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            if (ml[r].x == -INFINITY) continue;          // an empty piece
                            const float w = fast_exp2(ml[r].x - mnew);
                            l = fmaf(w, ml[r].y, l);
                            acc[0] = fmaf(w, a[r].x, acc[0]); acc[1] = fmaf(w, a[r].y, acc[1]);
                            acc[2] = fmaf(w, a[r].z, acc[2]); acc[3] = fmaf(w, a[r].w, acc[3]);
                            acc[4] = fmaf(w, bb[r].x, acc[4]); acc[5] = fmaf(w, bb[r].y, acc[5]);
                            acc[6] = fmaf(w, bb[r].z, acc[6]); acc[7] = fmaf(w, bb[r].w, acc[7]);
                        }
                        mx = mnew;
                    }
                }
            }
            float* e = stage + ((size_t)grp * cpt + c) * MERGE_FLOATS;
            e[0] = mx; e[1] = l;
            *reinterpret_cast<float4*>(e + 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4*>(e + 8) = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
        worker_sync();
        if (grp == 0) {
            for (int c = c_first; c < cpt; c += WORKERS) {
                float mx = -INFINITY;
                for (int g = 0; g < groups; ++g) mx = fmaxf(mx, stage[((size_t)g * cpt + c) * MERGE_FLOATS]);
                float l = 0.0f;
                float out[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int g = 0; g < groups; ++g) {
                    const float* e = stage + ((size_t)g * cpt + c) * MERGE_FLOATS;
                    if (e[0] == -INFINITY) continue;
                    const float w = fast_exp2(e[0] - mx);
                    l = fmaf(w, e[1], l);
#pragma unroll
                    for (int i = 0; i < 8; ++i) out[i] = fmaf(w, e[4 + i], out[i]);
                }
                const float inv = l > 0.0f ? 1.0f / l : 0.0f;      // the piece with the new token always has l >= 1
#pragma unroll
                for (int i = 0; i < 8; ++i) out[i] *= inv;
                if (live) store_chunk(b_tiles + ((b.ring0 + t) % STAGES) * b_bytes, c >> 3, c & 7, out);
            }
        }
        worker_sync();            // the staging area is free again
        if (++kb == b.NKB) kb = 0;
    }
}

// ---- S2: one attention item ------------------------------------------------------------------------------------------
// A key/value tile [BK keys][HD] in shared memory; the 16-byte chunk c of row r sits at chunk c ^ (r & 7).
template <int HD> __device__ __forceinline__ uint32_t kv_tile_addr(uint32_t base, int row, int chunk) {
    return base + (uint32_t)row * (HD * 2) + (uint32_t)((chunk ^ (row & 7)) * 16);
}
// What a layer's attention needs besides its weights, copied out of the descriptor once per layer.
struct LayerCache {
    const float* b_qkv;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const int* block_table;
    const int* slot_mapping;
    float eps1;
    int window;
};
// What an attention item covers: request r, kv head kvh, piece sp of the cached keys [lo, hi) of the request.
struct ItemGeom {
    int sp, kvh, r, klo, khi;
    bool owner;                   // this piece also takes the new token itself
    const int* bt;
};
template <int BK>
__device__ __forceinline__ ItemGeom item_geom(const FusedParams& p, const LayerCache& L, int item) {
    ItemGeom g;
    g.sp = item % p.nsplit;
    const int pair = item / p.nsplit;
    g.kvh = pair % p.Hkv;
    g.r = pair / p.Hkv;
    const int qpos = __ldg(p.span_pos + g.r);
    const int hi = qpos;                                          // cached keys: positions below the new token's
    const int lo = L.window > 0 ? max(0, qpos - L.window + 1) : 0;
    int chunk = (hi - lo + p.nsplit - 1) / p.nsplit;
    chunk = ((chunk + BK - 1) / BK) * BK;
    g.klo = lo + g.sp * chunk;
    g.khi = min(hi, g.klo + chunk);
    g.owner = g.sp == p.nsplit - 1;
    g.bt = L.block_table + (size_t)g.r * p.max_pages;
    return g;
}
// Ask for the tile of BK keys that starts at kb for this warp: K into buffer `buf`, V into buffer 2 + buf.
template <int HD>
__device__ __forceinline__ void issue_kv_tile(const FusedParams& p, const LayerCache& L, const ItemGeom& g, uint32_t wbase,
                                              int buf, int kb, int lane) {
    constexpr int BK = HD == 64 ? 32 : 16, CH = HD / 8, TILE_BYTES = BK * HD * 2;
    const int kpos = kb + lane;
    long long slot = -1;
    if (lane < BK && kpos < g.khi) slot = (long long)__ldg(g.bt + kpos / p.page_size) * p.page_size + (kpos % p.page_size);
    const uint32_t kbase = wbase + buf * TILE_BYTES, vbase = wbase + (2 + buf) * TILE_BYTES;
    const size_t row_stride = (size_t)p.Hkv * HD;
#pragma unroll
    for (int it = 0; it < (BK * CH) / 32; ++it) {
        const int idx = it * 32 + lane;
        const int row = idx / CH, ch = idx % CH;
        const long long s = __shfl_sync(0xffffffffu, slot, row);
        const bool valid = s >= 0;
        const size_t off = (valid ? (size_t)s : 0) * row_stride + (size_t)g.kvh * HD + ch * 8;
        cp_async16(kv_tile_addr<HD>(kbase, row, ch), L.k_cache + off, valid);
        cp_async16(kv_tile_addr<HD>(vbase, row, ch), L.v_cache + off, valid);
    }
    cp_async_commit();
}
// Before the stage barrier: every key warp asks for its first tile of the block's first item.  The cached keys and
// values do not depend on this step, so their way from memory lies under the wait for the other blocks.
template <int HD>
__device__ __forceinline__ void attention_prefetch(const FusedParams& p, const LayerCache& L, int item, uint8_t* attn, int wt) {
    constexpr int BK = HD == 64 ? 32 : 16, TILE_BYTES = BK * HD * 2;
    if (wt >= KV_THREADS) return;
    const int warp = wt >> 5, lane = wt & 31;
    const ItemGeom g = item_geom<BK>(p, L, item);
    const int kb_first = g.klo + warp * BK, kb_second = kb_first + (KV_THREADS / 32) * BK;
    const uint32_t wbase = smem_u32(attn) + warp * 4 * TILE_BYTES;
    if (kb_first < g.khi) issue_kv_tile<HD>(p, L, g, wbase, 0, kb_first, lane);
    if (kb_second < g.khi) issue_kv_tile<HD>(p, L, g, wbase, 1, kb_second, lane);     // both of the warp's buffers
}

template <int HD>
__device__ void attention_item(const FusedParams& p, const LayerCache& L, int item, bool prefetched, uint8_t* attn,
                               __nv_bfloat16* q_s, float* new_s, int wt) {
    constexpr int BK = HD == 64 ? 32 : 16;       // keys per tile: 4 KB of K and of V either way
    constexpr int TILE_BYTES = BK * HD * 2;
    constexpr int KS = HD / 16;                  // k-steps of Q K^T
    constexpr int NT = HD / 8;                   // n-tiles of P V
    constexpr int NS = BK / 8;                   // n-tiles of S
    constexpr int QP = HD + 8;                   // pitch of the staged q rows (bf16)
    constexpr int KVW = KV_THREADS / 32;
    const int warp = wt >> 5, lane = wt & 31;
    const int G = p.Hq / p.Hkv;
    const ItemGeom geo = item_geom<BK>(p, L, item);
    const int sp = geo.sp, kvh = geo.kvh, r = geo.r, klo = geo.klo, khi = geo.khi;
    const bool owner = geo.owner;
    const int Nqkv = (p.Hq + 2 * p.Hkv) * p.hd;
    const float* acc_row = p.qkv_acc + (size_t)r * Nqkv;
    const uint32_t wbase = smem_u32(attn) + warp * 4 * TILE_BYTES;      // per key warp: K[2], V[2]
    const int kb_first = klo + warp * BK;
    if (!prefetched && wt < KV_THREADS && kb_first < khi) issue_kv_tile<HD>(p, L, geo, wbase, 0, kb_first, lane);

    // q of the group's heads (bias, the deferred 1/rms, rotation) as bf16 rows in shared memory; the owner also makes
    // the new token's k and v, keeps them (rounded to bf16, as a later step will read them from the cache) and writes
    // them to the cache.  A thread's elements are fetched together.
    {
        const float ssr = __ldcg(p.ss1 + r);
        const int half = p.rotary_dim / 2;
        const int n_q = G * HD, n_all = n_q + (owner ? 2 * HD : 0);
        const long long slot = owner ? (long long)__ldg(L.slot_mapping + r) : -1;
        for (int base = 0; base < n_all; base += 4 * WORKERS) {
            float val[4], oth[4], bv[4], bo[4];
            float2 cs[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * WORKERS + wt;
                val[u] = oth[u] = bv[u] = bo[u] = 0.0f;
                cs[u] = make_float2(1.0f, 0.0f);
                if (i < n_all) {
                    // feature n of the fused projection: a q head of the group, then k, then v of this kv head
                    int n, d;
                    bool rot = true;
                    if (i < n_q) { const int g = i / HD; d = i - g * HD; n = (kvh * G + g) * HD + d; }
                    else if (i < n_q + HD) { d = i - n_q; n = (p.Hq + kvh) * HD + d; }
                    else { d = i - n_q - HD; n = (p.Hq + p.Hkv + kvh) * HD + d; rot = false; }
                    val[u] = __ldcg(acc_row + n);
                    if (L.b_qkv) bv[u] = __ldg(L.b_qkv + n);
                    if (rot && d < p.rotary_dim) {
                        int partner, fi;
                        if (p.interleaved) { partner = (d & 1) ? n - 1 : n + 1; fi = d >> 1; }
                        else { partner = d < half ? n + half : n - half; fi = d < half ? d : d - half; }
                        oth[u] = __ldcg(acc_row + partner);
                        if (L.b_qkv) bo[u] = __ldg(L.b_qkv + partner);
                        cs[u] = __ldg(p.rope_table + (size_t)r * half + fi);
                    }
                }
            }
            const float inv = 1.0f / sqrtf(ssr / (float)p.D + L.eps1);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + u * WORKERS + wt;
                if (i >= n_all) continue;
                const int d = i < n_q ? i % HD : (i - n_q) % HD;
                const bool rot = i < n_q + HD && d < p.rotary_dim;
                const bool first = p.interleaved ? (d & 1) == 0 : d < half;
                const float v0 = fmaf(val[u], inv, bv[u]), v1 = fmaf(oth[u], inv, bo[u]);
                const float res = !rot ? v0 : first ? v0 * cs[u].x - v1 * cs[u].y : v0 * cs[u].x + v1 * cs[u].y;
                const __nv_bfloat16 h = __float2bfloat16_rn(res);
                if (i < n_q) {
                    q_s[(i / HD) * QP + d] = h;
                } else {
                    const bool is_v = i >= n_q + HD;
                    new_s[i - n_q] = __bfloat162float(h);
                    if (slot >= 0) (is_v ? L.v_cache : L.k_cache)[((size_t)slot * p.Hkv + kvh) * HD + d] = h;
                }
            }
        }
    }
    worker_sync();

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    if (wt < KV_THREADS) {
        uint32_t qf[KS][4];
        {
            const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
#pragma unroll
            for (int s = 0; s < KS; ++s) {
                qf[s][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(q_s + r0 * QP + s * 16 + c) : 0u;
                qf[s][1] = r1 < G ? *reinterpret_cast<const uint32_t*>(q_s + r1 * QP + s * 16 + c) : 0u;
                qf[s][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(q_s + r0 * QP + s * 16 + 8 + c) : 0u;
                qf[s][3] = r1 < G ? *reinterpret_cast<const uint32_t*>(q_s + r1 * QP + s * 16 + 8 + c) : 0u;
            }
        }
        int buf = 0;
        for (int kb = kb_first; kb < khi; kb += KVW * BK) {
            const int kb_next = kb + KVW * BK;
            if (kb_next < khi) {
                // (a prefetched item already has its second tile on the way)
                if (!(prefetched && kb == kb_first)) issue_kv_tile<HD>(p, L, geo, wbase, buf ^ 1, kb_next, lane);
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
            __syncwarp();
            const uint32_t kbase = wbase + buf * TILE_BYTES, vbase = wbase + (2 + buf) * TILE_BYTES;
            float s[NS][4];
#pragma unroll
            for (int i = 0; i < NS; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ks += 2) {
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    uint32_t b[4];
                    ldmatrix_x4(kv_tile_addr<HD>(kbase, i * 8 + (lane & 7), ks * 2 + (lane >> 3)), b);
                    mma_bf16(s[i], qf[ks], b[0], b[1]);
                    mma_bf16(s[i], qf[ks + 1], b[2], b[3]);
                }
            }
            const int c0 = (lane & 3) * 2;
            float mt[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < NS; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = kb + i * 8 + c0 + (e & 1);
                    const float v = key < khi ? s[i][e] * p.scale_log2e : -INFINITY;
                    s[i][e] = v;
                    mt[e >> 1] = fmaxf(mt[e >> 1], v);
                }
            }
            float corr[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mt[h] = fmaxf(mt[h], __shfl_xor_sync(0xffffffffu, mt[h], 1));
                mt[h] = fmaxf(mt[h], __shfl_xor_sync(0xffffffffu, mt[h], 2));
                const float m_new = fmaxf(m_run[h], mt[h]);       // finite: every tile has at least one key
                corr[h] = m_run[h] == -INFINITY ? 0.0f : fast_exp2(m_run[h] - m_new);
                m_run[h] = m_new;
            }
            float lt[2] = {0.0f, 0.0f};
            uint32_t pf[NS / 2][4];      // P as A fragments, one per k-step of 16 keys
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                const float p0 = fast_exp2(s[i][0] - m_run[0]), p1 = fast_exp2(s[i][1] - m_run[0]);
                const float p2 = fast_exp2(s[i][2] - m_run[1]), p3 = fast_exp2(s[i][3] - m_run[1]);
                lt[0] += p0 + p1;
                lt[1] += p2 + p3;
                pf[i >> 1][(i & 1) * 2 + 0] = pack_bf16(p0, p1);
                pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                lt[h] += __shfl_xor_sync(0xffffffffu, lt[h], 1);
                lt[h] += __shfl_xor_sync(0xffffffffu, lt[h], 2);
                l_run[h] = l_run[h] * corr[h] + lt[h];
            }
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int j = 0; j < NS / 2; ++j) {
#pragma unroll
                for (int i = 0; i < NT; i += 2) {
                    uint32_t b[4];
                    const int mat = lane >> 3;
                    ldmatrix_x4_trans(kv_tile_addr<HD>(vbase, j * 16 + (mat & 1) * 8 + (lane & 7), i + (mat >> 1)), b);
                    mma_bf16(o[i], pf[j], b[0], b[1]);
                    mma_bf16(o[i + 1], pf[j], b[2], b[3]);
                }
            }
            buf ^= 1;
            __syncwarp();
        }
    }

    // Merge the key warps through shared memory (the tile buffers are free now); the new token is one more entry.
    worker_sync();
    float* wacc = reinterpret_cast<float*>(attn);                       // [KVW + 1][16][HD]
    float* wml = wacc + (KVW + 1) * 16 * HD;                            // [KVW + 1][16][2]
    if (wt < KV_THREADS) {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            float* a0 = wacc + ((size_t)(warp * 16 + r0) * HD) + i * 8 + c;
            float* a1 = wacc + ((size_t)(warp * 16 + r0 + 8) * HD) + i * 8 + c;
            a0[0] = o[i][0]; a0[1] = o[i][1];
            a1[0] = o[i][2]; a1[1] = o[i][3];
        }
        if ((lane & 3) == 0) {
            wml[(warp * 16 + r0) * 2] = m_run[0];     wml[(warp * 16 + r0) * 2 + 1] = l_run[0];
            wml[(warp * 16 + r0 + 8) * 2] = m_run[1]; wml[(warp * 16 + r0 + 8) * 2 + 1] = l_run[1];
        }
    } else if (wt < KV_THREADS + 16) {      // the new token's score for each head of the group: q . k_new, both as bf16
        const int g = wt - KV_THREADS;
        float sc = -INFINITY;
        if (owner && g < G) {
            float dot = 0.0f;
            for (int d = 0; d < HD; ++d) dot = fmaf(__bfloat162float(q_s[g * QP + d]), new_s[d], dot);
            sc = dot * p.scale_log2e;
        }
        wml[(KVW * 16 + g) * 2] = sc;
        wml[(KVW * 16 + g) * 2 + 1] = owner ? 1.0f : 0.0f;
    }
    worker_sync();
    const size_t base = ((size_t)(r * p.Hkv + kvh) * p.nsplit + sp) * G;
    for (int i = wt; i < G * HD; i += WORKERS) {
        const int g = i / HD, d = i - g * HD;
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w <= KVW; ++w) Mx = fmaxf(Mx, wml[(w * 16 + g) * 2]);
        float Ls = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w <= KVW; ++w) {
            const float mw = wml[(w * 16 + g) * 2];
            if (mw != -INFINITY) {
                const float e = fast_exp2(mw - Mx);
                Ls = fmaf(e, wml[(w * 16 + g) * 2 + 1], Ls);
                a = fmaf(e, w < KVW ? wacc[(size_t)(w * 16 + g) * HD + d] : new_s[HD + d], a);
            }
        }
        p.part_acc[(base + g) * HD + d] = a;
        if (d == 0) *reinterpret_cast<float2*>(p.part_ml + (base + g) * 2) = make_float2(Mx, Ls);
    }
    worker_sync();            // the staged q, the new token and the merge area are free for the next item
}

template <int BN, int STAGES, int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1) decode_layers_kernel(const FusedParams p) {
    constexpr uint32_t B_BYTES = BN * TILE_K * 2;
    // Two units are in flight (one being drained): 2 x BN columns of tensor memory.  (Four accumulators per unit, one per
    // K step, were tried: the instructions are not paced by their dependency on one accumulator, about 170 cycles each
    // either way.)
    constexpr int NACC = 1;
    constexpr uint32_t TMEM_COLS = 2 * NACC * BN < 32 ? 32 : 2 * NACC * BN;
    constexpr int WORKER_WARPS = WORKERS / 32;
    __shared__ __align__(8) uint64_t full_a[STAGES], full_b[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
    __shared__ volatile int wait_ok[2];   // what the polling worker warp found, for the warps parked meanwhile (used in turn)
    __shared__ BlockPlan plan;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = a_tiles + STAGES * A_BYTES;
    uint8_t* attn = b_tiles + STAGES * B_BYTES;
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(attn + ATTN_BYTES);      // [16][hd + 8]
    float* new_s = reinterpret_cast<float*>(attn + ATTN_BYTES + 16 * (128 + 8) * 2);     // k then v of the new token: 2 hd
    volatile int* abort_flag = &abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&full_b[s], WORKER_WARPS);        // one arrival per worker warp
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], WORKER_WARPS);
        }
        abort_s = 0;
        mbar_init_fence();
    }
    if (threadIdx.x == 64) make_plan(p, plan);
    if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        // ---- weight tiles, in the order in which the block will use them, as far ahead as the ring allows ----------
        // A second cursor runs one ring further ahead and only asks for its tiles into L2, so that a slot that comes free
        // is refilled from there and not from memory.
        if (lane == 0) {
            struct Cursor {
                int l, st, i, nt, kb;
                __device__ __forceinline__ bool valid(const FusedParams& p) const { return l < p.num_layers; }
                __device__ __forceinline__ void settle(const FusedParams& p, const BlockPlan& plan) {     // skip empty stages
                    while (l < p.num_layers && i >= plan.n_tiles[st]) {
                        i = 0;
                        if (++st == 4) { st = 0; ++l; }
                        nt = plan.nt_first[st]; kb = plan.kb_first[st];
                    }
                }
                __device__ __forceinline__ void advance(const FusedParams& p, const BlockPlan& plan) {
                    ++i;
                    if (++kb == plan.NKB[st]) { kb = 0; ++nt; }
                    settle(p, plan);
                }
            };
            Cursor cur = {0, 0, 0, plan.nt_first[0], plan.kb_first[0]}, ahead = cur;
            cur.settle(p, plan);
            ahead.settle(p, plan);
            for (int k = 0; k < STAGES && ahead.valid(p); ++k) ahead.advance(p, plan);
            uint32_t it = 0;
            while (cur.valid(p)) {
                const int s = it % STAGES;
                if (!mbar_wait_polite(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(&full_a[s], A_BYTES);
                tma_load_2d(a_tiles + s * A_BYTES, stage_map(p.layers + cur.l, cur.st), cur.kb * TILE_K, cur.nt * TILE_M, &full_a[s]);
                if (ahead.valid(p)) {
                    tma_prefetch_2d(stage_map(p.layers + ahead.l, ahead.st), ahead.kb * TILE_K, ahead.nt * TILE_M);
                    ahead.advance(p, plan);
                }
                cur.advance(p, plan);
                ++it;
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core instructions ------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(TILE_M, BN);
            const uint32_t a_base = smem_u32(a_tiles), b_base = smem_u32(b_tiles);
            uint32_t it = 0, ua = 0;
            bool ok = true;
            for (int l = 0; l < p.num_layers && ok; ++l) {
                for (int st = 0; st < 4 && ok; ++st) {
                    const int NKB = plan.NKB[st], total = plan.n_tiles[st];
                    int kb0 = plan.kb_first[st];
                    for (int i = 0; i < total && ok;) {
                        const int n = min(NKB - kb0, total - i);
                        const int buf = ua & 1;
                        ok = mbar_wait_polite(&acc_empty[buf], ((ua >> 1) & 1) ^ 1, abort_flag);
                        for (int k = 0; k < n && ok; ++k, ++it) {
                            const int s = it % STAGES;
                            ok = mbar_wait_polite(&full_a[s], (it / STAGES) & 1, abort_flag) &&
                                 mbar_wait_polite(&full_b[s], (it / STAGES) & 1, abort_flag);
                            if (!ok) break;
                            tc_fence_after();
                            const uint64_t da = desc_kmajor(a_base + s * A_BYTES), db = desc_kmajor(b_base + s * B_BYTES);
                            const uint32_t d = tmem_base + buf * NACC * BN;
                            // the four K steps of a tile: 32 bytes further along the swizzled rows each (2 in descriptor units)
                            if (k == 0) umma_bf16_first(d, da, db, idesc); else umma_bf16_acc(d, da, db, idesc);
                            umma_bf16_acc(d, da + 2, db + 2, idesc);
                            umma_bf16_acc(d, da + 4, db + 4, idesc);
                            umma_bf16_acc(d, da + 6, db + 6, idesc);
                            umma_commit(&empty_bar[s]);          // the slot is free when these four have read it
                        }
                        if (ok) umma_commit(&acc_full[buf]);
                        ++ua;
                        i += n;
                        kb0 = 0;
                    }
                }
            }
        }
    } else {
        // ---- workers -------------------------------------------------------------------------------------------------
        const int wt = threadIdx.x - 64;
        const int quarter = warp & 3;            // the TMEM lanes this warp may read
        const int col_half = (warp - 2) >> 2;    // two warps share a quarter: each drains half of the columns
        uint32_t it = 0, ua = 0;
        unsigned epoch = 0, stamps = 0;
        int label = 0, wsel = 0;

        // Drain accumulator `u` (row tile nt of a stage with N outputs) into target [M, N] by atomic adds.
        auto drain = [&](uint32_t u, int nt, int N, float* target) {
            const int buf = u & 1;
            // One warp polls (on a scheduler that it shares with no other role); the others are parked at the barrier and
            // take no issue slots from the roles that work meanwhile.
            if (warp == 2) {
                const bool done = mbar_wait_polite(&acc_full[buf], (u >> 1) & 1, abort_flag);
                if (lane == 0) wait_ok[wsel] = done ? 1 : 0;
            }
            worker_sync();
            const bool ok = wait_ok[wsel] != 0;
            wsel ^= 1;
            tc_fence_after();
            const int n = nt * TILE_M + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * NACC * BN + ((uint32_t)(quarter * 32) << 16);
            float* out = target + n;
            // the four accumulators of the unit, 16 columns (tokens) at a time
            auto load_sum = [&](int c0, float (&v)[16]) {
                float w[16];
                tmem_ld16(taddr + c0, v);
#pragma unroll
                for (int a = 1; a < NACC; ++a) {
                    tmem_ld16(taddr + a * BN + c0, w);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += w[j];
                }
            };
            if (ok) {      // uniform over the warp: tcgen05.ld is a warp-wide instruction
                if (BN == 16) {          // one group of 16 columns: each of the two warps adds eight of them
                    float v[16];
                    load_sum(0, v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int m = col_half * 8 + j;
                        if (m < p.M && n < N) red_add(out + (size_t)m * N, col_half ? v[8 + j] : v[j]);
                    }
                } else {
#pragma unroll 1
                    for (int c0 = col_half * 16; c0 < BN && c0 < p.M; c0 += 32) {
                        float v[16];
                        load_sum(c0, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < p.M && n < N) red_add(out + (size_t)(c0 + j) * N, v[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        };
        // One contraction stage: B operands for this block's tiles, a batch at a time, then the accumulators.  A unit
        // (the tiles of one row tile) is drained two units behind the one being built, so that the tensor-core role
        // always finds an accumulator free and the ring keeps moving.
        auto gemm_stage = [&](int st, float* target, const void* norm_w, int norm_bf16, float eps2) {
            struct { int N, NKB; } si = {plan.N[st], plan.NKB[st]};
            const int n_tiles = plan.n_tiles[st], nt_first = plan.nt_first[st], kb_first = plan.kb_first[st];
            const int units = plan.units[st];
            const uint32_t u0 = ua;
            int next_drain = 0;
            int per_batch = STAGES;
            if (st == ST_O) per_batch = 1;
            for (int jb = 0; jb < n_tiles;) {
                const int je = min(n_tiles, jb + per_batch);
                const int last_unit = je == n_tiles ? units - 1 : (kb_first + je - 1) / si.NKB;
                while (next_drain + 2 <= last_unit) {
                    drain(u0 + next_drain, nt_first + next_drain, si.N, target);
                    ++next_drain;
                }
                bool live = true;
                // The stage's first tiles find their slots free: every accumulator of the stage before was drained before
                // the blocks met, so every earlier tensor-core instruction has completed.  Later batches wait (one lane;
                // the warp follows it).
                if (jb > 0) {
                    if (warp == 2) {
                        for (int j = jb; j < je; ++j) {
                            const uint32_t at = it + j;
                            live = mbar_wait_polite(&empty_bar[at % STAGES], ((at / STAGES) & 1) ^ 1, abort_flag) && live;
                        }
                        if (lane == 0) wait_ok[wsel] = live ? 1 : 0;
                    }
                    worker_sync();
                    live = wait_ok[wsel] != 0;
                    wsel ^= 1;
                }
                stamp(p, stamps, label + 5);
                Batch b;
                if (jb == 0) { b.kb0 = kb_first; b.nt0 = nt_first; }
                else { b.kb0 = (kb_first + jb) % si.NKB; b.nt0 = nt_first + (kb_first + jb) / si.NKB; }
                b.n = je - jb; b.NKB = si.NKB;
                b.ring0 = it + jb;
                if (st == ST_QKV) build_norm<STAGES, 4>(p, norm_w, norm_bf16, p.ss1, b, b_tiles, B_BYTES, live, wt);
                else if (st == ST_GU) build_norm<STAGES, 4>(p, norm_w, norm_bf16, p.ss2, b, b_tiles, B_BYTES, live, wt);
                else if (st == ST_O) build_merge<STAGES, 4>(p, b, reinterpret_cast<float*>(attn), b_tiles, B_BYTES, live, wt);
                else build_swiglu<STAGES, 2>(p, eps2, b, b_tiles, B_BYTES, live, wt);
                stamp(p, stamps, label + 6);
                fence_async_smem();          // every writer's stores are ordered before the tensor cores' reads
                __syncwarp();
                if (lane == 0)
                    for (int j = jb; j < je; ++j) mbar_arrive(&full_b[(it + j) % STAGES]);
                jb = je;
            }
            it += n_tiles;
            ua += units;
            stamp(p, stamps, label + 1);
            for (; next_drain < units; ++next_drain)
                drain(u0 + next_drain, nt_first + next_drain, si.N, target);
            stamp(p, stamps, label + 2);
        };
        auto zero_range = [&](float* buf, int lo, int hi) {        // this block's part of a scratch array
            for (int i = lo + wt; i < hi; i += WORKERS) buf[i] = 0.0f;
        };
        auto zero_sums = [&](float* ss) {
            if (blockIdx.x == 0 && wt < 64) ss[wt] = 0.0f;
        };

        // Everything that is added into starts at zero, whatever an earlier launch left.
        zero_range(p.qkv_acc, plan.zero_qkv_lo, plan.zero_qkv_hi);
        zero_range(p.gu_acc, plan.zero_gu_lo, plan.zero_gu_hi);
        zero_sums(p.ss1);
        zero_sums(p.ss2);
        grid_barrier(p, epoch, abort_flag);
        stamp(p, stamps, 3);

        for (int l = 0; l < p.num_layers; ++l) {
            const LayerDesc* L = p.layers + l;
            // the layer's scalars and pointers, read once (the descriptor lives in global memory)
            const void* norm1_w = L->norm1_w;
            const void* norm2_w = L->norm2_w;
            const int norm_bf16 = L->norm_w_bf16;
            const float eps2 = L->eps2;
            LayerCache lc;
            lc.b_qkv = L->b_qkv; lc.k_cache = L->k_cache; lc.v_cache = L->v_cache; lc.eps1 = L->eps1; lc.window = L->window;
            lc.block_table = p.block_tables[L->group]; lc.slot_mapping = p.slot_mapping[L->group];
            const int items = p.M * p.Hkv * p.nsplit;
#pragma unroll 1
            for (int st = 0; st < 4; ++st) {       // one copy of the stage's code for all four contractions: a role is a
                                                   // lone warp on its scheduler, and code it has to fetch anew costs it time
                label = (l + 1) * 100 + (st == ST_QKV ? 10 : st == ST_O ? 30 : st == ST_GU ? 40 : 50);
                float* target = st == ST_QKV ? p.qkv_acc : st == ST_GU ? p.gu_acc : p.residual;
                gemm_stage(st, target, st == ST_QKV ? norm1_w : norm2_w, norm_bf16, eps2);
                grid_arrive(p, epoch);
                // While the other blocks arrive: what nobody waits for.
                if (st == ST_QKV) {
                    if ((int)blockIdx.x < items) attention_prefetch<HD>(p, lc, blockIdx.x, attn, wt);
                    if (l > 0) {       // the last layer's feed-forward has read its sums; S4 of this layer adds into them again
                        zero_range(p.gu_acc, plan.zero_gu_lo, plan.zero_gu_hi);
                        zero_sums(p.ss2);
                    }
                } else if (st == ST_O) {      // S2 has read the projection's sums; the next layer adds into them again
                    zero_range(p.qkv_acc, plan.zero_qkv_lo, plan.zero_qkv_hi);
                    zero_sums(p.ss1);
                }
                grid_wait(p, epoch, abort_flag);
                stamp(p, stamps, label + 3);
                if (st == ST_QKV) {
                    label += 10;
                    for (int item = blockIdx.x; item < items; item += gridDim.x)      // no waits inside: nothing to give up on
                        attention_item<HD>(p, lc, item, item == (int)blockIdx.x, attn, q_s, new_s, wt);
                    stamp(p, stamps, label + 2);
                    grid_barrier(p, epoch, abort_flag);
                    stamp(p, stamps, label + 3);
                }
            }
        }
        // The block that finishes last puts the counters back to zero for the next launch.
        if (threadIdx.x == 64) {
            __threadfence();
            if (atomicAdd(p.sync + 1, 1u) == gridDim.x - 1) {
                atomicExch(p.sync, 0u);
                atomicExch(p.sync + 1, 0u);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_s && threadIdx.x == 0 && p.error_flag) atomicCAS(p.error_flag, 0, 8);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int BN> struct StagesFor { static constexpr int value = BN == 16 ? 8 : BN == 32 ? 7 : 6; };

template <int BN>
size_t fused_smem_bytes() {
    return (size_t)StagesFor<BN>::value * (A_BYTES + BN * TILE_K * 2) + ATTN_BYTES + 16 * (128 + 8) * 2 + 2 * 128 * 4 + 1024;
}

int num_sms() {
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (sms[dev] == 0) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev];
}

template <int BN, int HD>
int launch_fused(const FusedParams& p, cudaStream_t stream) {
    constexpr int STAGES = StagesFor<BN>::value;
    const size_t smem = fused_smem_bytes<BN>();
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_layers_kernel<BN, STAGES, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess)
            return llb_fail("decode_layers: cannot opt in to %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    const int grid = num_sms();
    LLB_REQUIRE(grid > 0, "decode_layers: cannot read the number of multiprocessors");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;       // all blocks resident at once: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_layers_kernel<BN, STAGES, HD>, p);
    if (e != cudaSuccess) return llb_fail("decode_layers: launch failed: %s", cudaGetErrorString(e));
    return llb_check_launch("decode_layers");
}
template <int BN>
int launch_fused_hd(const FusedParams& p, cudaStream_t stream) {
    return p.hd == 64 ? launch_fused<BN, 64>(p, stream) : launch_fused<BN, 128>(p, stream);
}

}  // namespace

// Bytes of one layer descriptor (an array of them lives in device memory, 64-byte aligned).
LLB_EXPORT int llb_decode_layers_desc_bytes() { return (int)sizeof(LayerDesc); }

// Whether the fused layers take these sizes.
LLB_EXPORT int llb_decode_layers_supports(int M, int D, int Hq, int Hkv, int hd, int I, int rotary_dim) {
    if (M < 1 || M > 64 || Hkv < 1 || Hq % Hkv != 0 || Hq / Hkv > 16) return 0;
    if (hd != 64 && hd != 128) return 0;
    if (D % 8 != 0 || I % 8 != 0 || D < 8 || I < 8) return 0;
    if (rotary_dim < 0 || rotary_dim > hd || rotary_dim % 2 != 0) return 0;
    return 1;
}

// Fills one descriptor in HOST memory (the caller copies the array to the device).  Weights are bf16, row-major
// [N, K], 16-byte aligned: w_qkv [(Hq + 2 Hkv) hd, D], w_o [D, Hq hd], w_gate_up [2 I, D] (gate and up rows
// interleaved), w_down [D, I].  b_qkv float or null; norm weights bf16 (norm_w_bf16 != 0) or float.
LLB_EXPORT int llb_decode_layers_describe(void* desc_host, const void* w_qkv, const void* w_o, const void* w_gate_up,
                                          const void* w_down, const float* b_qkv, const void* norm1_w, const void* norm2_w,
                                          int norm_w_bf16, float eps1, float eps2, void* k_cache, void* v_cache, int window,
                                          int group, int D, int Hq, int Hkv, int hd, int I) {
    LLB_REQUIRE(desc_host && w_qkv && w_o && w_gate_up && w_down && norm1_w && norm2_w && k_cache && v_cache,
                "decode_layers: a tensor of the layer is missing");
    LLB_REQUIRE(group >= 0 && group < MAX_GROUPS, "decode_layers: cache group %d is outside 0..%d", group, MAX_GROUPS - 1);
    LLB_REQUIRE(((uintptr_t)w_qkv | (uintptr_t)w_o | (uintptr_t)w_gate_up | (uintptr_t)w_down | (uintptr_t)norm1_w |
                 (uintptr_t)norm2_w | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0,
                "decode_layers: tensors must be 16-byte aligned");
    LayerDesc d = {};
    int rc;
    if ((rc = make_map_bf16(w_qkv, (long long)(Hq + 2 * Hkv) * hd, D, TILE_M, &d.map_qkv))) return rc;
    if ((rc = make_map_bf16(w_o, D, (long long)Hq * hd, TILE_M, &d.map_o))) return rc;
    if ((rc = make_map_bf16(w_gate_up, 2ll * I, D, TILE_M, &d.map_gu))) return rc;
    if ((rc = make_map_bf16(w_down, D, I, TILE_M, &d.map_down))) return rc;
    d.b_qkv = b_qkv; d.norm1_w = norm1_w; d.norm2_w = norm2_w;
    d.k_cache = (__nv_bfloat16*)k_cache; d.v_cache = (__nv_bfloat16*)v_cache;
    d.eps1 = eps1; d.eps2 = eps2; d.norm_w_bf16 = norm_w_bf16; d.window = window > 0 ? window : 0; d.group = group;
    memcpy(desc_host, &d, sizeof(d));
    return 0;
}

// Floats of scratch for a step of M rows (everything the stages add into or hand over).
LLB_EXPORT long long llb_decode_layers_scratch_floats(int M, int Hq, int Hkv, int hd, int I, int nsplit) {
    const long long Nqkv = (long long)(Hq + 2 * Hkv) * hd;
    return (long long)M * Nqkv + (long long)M * 2 * I + 128 + (long long)M * Hq * nsplit * (hd + 2);
}

// Runs num_layers layers over the float residual [M, D] in place.  layers: device array of descriptors
// (llb_decode_layers_describe).  rope_table [M, rotary_dim / 2] of (cos, sin) pairs (llb_rope_table), span_pos [M];
// block_tables / slot_mapping: one pointer per cache group (null where unused), block tables [M, max_pages].
// scratch: llb_decode_layers_scratch_floats floats, contents arbitrary.  sync: two unsigned ints, zero before the first
// launch and left zero (after a reported error the caller sets them to zero again).  error_flag: one int.
// timeline: null, or room for 2 * (2 + 64 * num_layers) 64-bit words: block 0's (label, SM cycle) milestones, for tuning.
LLB_EXPORT int llb_decode_layers(const void* layers, int num_layers, float* residual, int M, int D, int Hq, int Hkv, int hd,
                                 int I, int rotary_dim, int interleaved, float scale, const float* rope_table,
                                 const int* span_pos, const int* bt0, const int* bt1, const int* bt2, const int* bt3,
                                 const int* sm0, const int* sm1, const int* sm2, const int* sm3, int max_pages,
                                 int page_size, int nsplit, float* scratch, long long scratch_floats, unsigned* sync,
                                 int* error_flag, unsigned long long* timeline, int timeline_block, cudaStream_t stream) {
    if (num_layers == 0 || M == 0) return 0;
    LLB_REQUIRE(llb_decode_layers_supports(M, D, Hq, Hkv, hd, I, rotary_dim),
                "decode_layers: unsupported sizes M=%d D=%d heads %d/%d of %d, I=%d, rotary_dim=%d", M, D, Hq, Hkv, hd, I,
                rotary_dim);
    LLB_REQUIRE(layers && residual && span_pos && scratch && sync && error_flag && (rotary_dim == 0 || rope_table),
                "decode_layers: an argument is missing");
    LLB_REQUIRE((uintptr_t)layers % 64 == 0 && (uintptr_t)residual % 16 == 0 && (uintptr_t)scratch % 16 == 0,
                "decode_layers: descriptors must be 64-byte aligned, residual and scratch 16-byte aligned");
    LLB_REQUIRE(nsplit >= 1 && nsplit <= MAX_SPLITS && page_size > 0 && max_pages > 0,
                "decode_layers: split count %d is outside 1..%d, or bad page sizes", nsplit, MAX_SPLITS);
    LLB_REQUIRE(scratch_floats >= llb_decode_layers_scratch_floats(M, Hq, Hkv, hd, I, nsplit),
                "decode_layers: %lld floats of scratch are needed, %lld given",
                llb_decode_layers_scratch_floats(M, Hq, Hkv, hd, I, nsplit), scratch_floats);
    FusedParams p = {};
    p.layers = (const LayerDesc*)layers; p.num_layers = num_layers; p.residual = residual;
    p.M = M; p.D = D; p.Hq = Hq; p.Hkv = Hkv; p.hd = hd; p.I = I; p.rotary_dim = rotary_dim; p.interleaved = interleaved;
    p.scale_log2e = scale * 1.4426950408889634f;
    p.rope_table = (const float2*)rope_table; p.span_pos = span_pos;
    p.block_tables[0] = bt0; p.block_tables[1] = bt1; p.block_tables[2] = bt2; p.block_tables[3] = bt3;
    p.slot_mapping[0] = sm0; p.slot_mapping[1] = sm1; p.slot_mapping[2] = sm2; p.slot_mapping[3] = sm3;
    p.max_pages = max_pages; p.page_size = page_size; p.nsplit = nsplit;
    const long long Nqkv = (long long)(Hq + 2 * Hkv) * hd;
    // 16-byte aligned pieces: Nqkv and 2 I are multiples of 4 floats per row only if hd is (it is 64 or 128) and I % 2 == 0
    p.qkv_acc = scratch;
    p.gu_acc = p.qkv_acc + (long long)M * Nqkv;
    p.ss1 = p.gu_acc + (long long)M * 2 * I;
    p.ss2 = p.ss1 + 64;
    p.part_acc = p.ss2 + 64;
    p.part_ml = p.part_acc + (long long)M * Hq * nsplit * hd;
    p.sync = sync; p.error_flag = error_flag; p.timeline = timeline; p.timeline_block = timeline_block;
    if (M <= 16) return launch_fused_hd<16>(p, stream);
    if (M <= 32) return launch_fused_hd<32>(p, stream);
    return launch_fused_hd<64>(p, stream);
}
