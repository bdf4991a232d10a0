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
// Roles of a block (192 threads): warp 0 requests weight tiles (TMA, no multicast), warp 1 issues tcgen05.mma into two
// accumulators in tensor memory, warps 2-5 build B operands, run the attention items, drain the accumulators and meet
// the other blocks.  The launch is cooperative, so all blocks are resident; every wait has a time limit.
#include <math.h>

#include "tcgen05_common.cuh"

namespace {

using namespace t5;

constexpr int TILE_M = 128;
constexpr int TILE_K = 64;
constexpr uint32_t A_BYTES = TILE_M * TILE_K * 2;
constexpr int NUM_THREADS = 192;
constexpr int WORKERS = 128;
constexpr int ATTN_BYTES = 64 * 1024;      // per-warp K/V buffers of the attention items, then their merge area
constexpr int MAX_GROUPS = 4;
constexpr int MAX_SPLITS = 32;
constexpr int ATTN_WARPS = 4;

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

__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
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
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;     // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// All blocks meet: arrivals are counted in sync[0], which only grows while the kernel runs (the block that finishes
// last sets it back to zero).  One worker thread arrives and polls; the wait gives up after the library's time
// limit or as soon as any block has raised the error flag.
__device__ __forceinline__ void grid_barrier(const FusedParams& p, unsigned& epoch, volatile int* abort_flag) {
    ++epoch;
    worker_sync();                        // every worker's writes are ordered before thread 0's release
    if (threadIdx.x == 64) {
        __threadfence();
        red_release_inc(p.sync);
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
        __threadfence();
    }
    worker_sync();
}

// ---- B operands: BN rows (tokens) x 64 columns of one K block, bf16, K-major with the 128-byte swizzle ------------
// A 16-byte chunk q (8 columns) of row m sits at m * 128 + ((q ^ (m & 7)) * 16).  Rows from M on are left as they
// are: the accumulator columns they produce are never read.
__device__ __forceinline__ void store_chunk(uint8_t* tile, int m, int q, const float (&v)[8]) {
    *reinterpret_cast<uint4*>(tile + (uint32_t)m * 128 + ((q ^ (m & 7)) * 16)) =
        make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}
__device__ __forceinline__ void load_norm_w(const void* w, int bf16, int k, float (&nw)[8]) {
    if (bf16) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>((const __nv_bfloat16*)w + k));
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            nw[2 * i] = f.x; nw[2 * i + 1] = f.y;
        }
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4*>((const float*)w + k));
        const float4 b = __ldg(reinterpret_cast<const float4*>((const float*)w + k + 4));
        nw[0] = a.x; nw[1] = a.y; nw[2] = a.z; nw[3] = a.w; nw[4] = b.x; nw[5] = b.y; nw[6] = b.z; nw[7] = b.w;
    }
}
// S1 / S4: bf16(x * norm_w) of the residual rows; with `ss` the rows' sums of squares over this K block are added there.
__device__ __forceinline__ void build_b_norm(const FusedParams& p, const void* norm_w, int norm_bf16, int kb, float* ss,
                                             uint8_t* tile, int wt) {
    const int lane = wt & 31;
    for (int base = wt & ~31; base < p.M * 8; base += WORKERS) {
        const int idx = base + lane, m = idx >> 3, q = idx & 7, k = kb * TILE_K + q * 8;
        const bool valid = idx < p.M * 8;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (valid && k < p.D) {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(p.residual + (size_t)m * p.D + k));
            const float4 b = __ldcg(reinterpret_cast<const float4*>(p.residual + (size_t)m * p.D + k + 4));
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        if (ss != nullptr) {      // uniform over the block
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s = fmaf(v[i], v[i], s);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (valid && q == 0) red_add(ss + m, s);
        }
        if (valid) {
            if (k < p.D) {
                float nw[8];
                load_norm_w(norm_w, norm_bf16, k, nw);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] *= nw[i];
            }
            store_chunk(tile, m, q, v);
        }
    }
}
// S3: the attention output of 64 columns (one head, or half of one), its pieces merged by their softmax weights.
__device__ __forceinline__ void build_b_merge(const FusedParams& p, int kb, uint8_t* tile, int wt) {
    const int G = p.Hq / p.Hkv, K = p.Hq * p.hd;
    for (int idx = wt; idx < p.M * 8; idx += WORKERS) {
        const int m = idx >> 3, q = idx & 7, c0 = kb * TILE_K + q * 8;
        float out[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (c0 < K) {
            const int h = c0 / p.hd, d0 = c0 - h * p.hd, kvh = h / G, gi = h - kvh * G;
            const size_t first = ((size_t)(m * p.Hkv + kvh) * p.nsplit) * G + gi;     // piece sp: first + sp * G
            float mx = -INFINITY;
            for (int sp = 0; sp < p.nsplit; ++sp) mx = fmaxf(mx, __ldcg(p.part_ml + (first + (size_t)sp * G) * 2));
            float l = 0.0f;
            for (int sp = 0; sp < p.nsplit; ++sp) {
                const size_t at = first + (size_t)sp * G;
                const float ms = __ldcg(p.part_ml + at * 2);
                if (ms == -INFINITY) continue;          // an empty piece
                const float e = fast_exp2(ms - mx);
                l = fmaf(e, __ldcg(p.part_ml + at * 2 + 1), l);
                const float4 a = __ldcg(reinterpret_cast<const float4*>(p.part_acc + at * p.hd + d0));
                const float4 b = __ldcg(reinterpret_cast<const float4*>(p.part_acc + at * p.hd + d0 + 4));
                out[0] = fmaf(e, a.x, out[0]); out[1] = fmaf(e, a.y, out[1]); out[2] = fmaf(e, a.z, out[2]);
                out[3] = fmaf(e, a.w, out[3]); out[4] = fmaf(e, b.x, out[4]); out[5] = fmaf(e, b.y, out[5]);
                out[6] = fmaf(e, b.z, out[6]); out[7] = fmaf(e, b.w, out[7]);
            }
            const float inv = 1.0f / l;        // the piece with the new token always has l >= 1
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] *= inv;
        }
        store_chunk(tile, m, q, out);
    }
}
// S5: silu(gate) * up of 64 intermediate columns from the interleaved sums of S4 (gate at 2j, up at 2j + 1).
__device__ __forceinline__ void build_b_swiglu(const FusedParams& p, float eps2, int kb, uint8_t* tile, int wt) {
    for (int idx = wt; idx < p.M * 8; idx += WORKERS) {
        const int m = idx >> 3, q = idx & 7, j0 = kb * TILE_K + q * 8;
        float out[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (j0 < p.I) {
            const float inv = 1.0f / sqrtf(__ldcg(p.ss2 + m) / (float)p.D + eps2);
            const float4* src = reinterpret_cast<const float4*>(p.gu_acc + (size_t)m * 2 * p.I + 2 * j0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 t = __ldcg(src + i);
                out[2 * i] = llb_silu(t.x * inv) * (t.y * inv);
                out[2 * i + 1] = llb_silu(t.z * inv) * (t.w * inv);
            }
        }
        store_chunk(tile, m, q, out);
    }
}

// ---- S2: one attention item ------------------------------------------------------------------------------------------
template <int HD> __device__ __forceinline__ uint32_t kv_tile_addr(uint32_t base, int row, int chunk) {
    return base + (uint32_t)row * (HD * 2) + (uint32_t)((chunk ^ (row & 7)) * 16);
}
// The value of feature n of row r after bias (and the deferred 1/rms), rotated when it lies in the rotary part of a
// q or k head: pairs (d, d + half) or (2i, 2i + 1), angle index d mod half or d / 2.
__device__ __forceinline__ float rotated_feature(const FusedParams& p, const LayerDesc* L, const float* acc_row, float inv,
                                                 int r, int n, bool rotate) {
    const float val = fmaf(__ldcg(acc_row + n), inv, L->b_qkv ? __ldg(L->b_qkv + n) : 0.0f);
    const int d = n % p.hd;
    if (!rotate || d >= p.rotary_dim) return val;
    const int half = p.rotary_dim / 2;
    int partner, fi;
    bool first;
    if (p.interleaved) { first = (d & 1) == 0; partner = first ? n + 1 : n - 1; fi = d >> 1; }
    else { first = d < half; partner = first ? n + half : n - half; fi = first ? d : d - half; }
    const float other = fmaf(__ldcg(acc_row + partner), inv, L->b_qkv ? __ldg(L->b_qkv + partner) : 0.0f);
    const float2 cs = __ldg(p.rope_table + (size_t)r * half + fi);
    return first ? val * cs.x - other * cs.y : val * cs.x + other * cs.y;
}

template <int HD>
__device__ void attention_item(const FusedParams& p, const LayerDesc* L, int item, uint8_t* attn, __nv_bfloat16* q_s,
                               float* new_s, int wt) {
    constexpr int BK = HD == 64 ? 32 : 16;       // keys per tile: 4 KB of K and of V either way
    constexpr int CH = HD / 8;                   // 16-byte chunks per row
    constexpr int TILE_BYTES = BK * HD * 2;
    constexpr int KS = HD / 16;                  // k-steps of Q K^T
    constexpr int NT = HD / 8;                   // n-tiles of P V
    constexpr int NS = BK / 8;                   // n-tiles of S
    constexpr int QP = HD + 8;                   // pitch of the staged q rows (bf16)
    const int warp = wt >> 5, lane = wt & 31;
    const int G = p.Hq / p.Hkv;
    const int sp = item % p.nsplit, pair = item / p.nsplit, kvh = pair % p.Hkv, r = pair / p.Hkv;
    const int Nqkv = (p.Hq + 2 * p.Hkv) * p.hd;
    const int qpos = __ldg(p.span_pos + r);
    const int hi = qpos;                                          // cached keys: positions below the new token's
    const int lo = L->window > 0 ? max(0, qpos - L->window + 1) : 0;
    int chunk = (hi - lo + p.nsplit - 1) / p.nsplit;
    chunk = ((chunk + BK - 1) / BK) * BK;
    const int klo = lo + sp * chunk, khi = min(hi, klo + chunk);
    const bool owner = sp == p.nsplit - 1;                        // this piece also takes the new token itself
    const int* bt = p.block_tables[L->group] + (size_t)r * p.max_pages;
    const float* acc_row = p.qkv_acc + (size_t)r * Nqkv;
    const float inv = 1.0f / sqrtf(__ldcg(p.ss1 + r) / (float)p.D + L->eps1);

    // q of the group's heads (bias, rotation) as bf16 rows in shared memory; the owner also makes the new token's k
    // and v, keeps them (rounded to bf16, as a later step will read them from the cache) and writes them to the cache.
    for (int i = wt; i < G * HD; i += WORKERS) {
        const int g = i / HD, d = i - g * HD;
        q_s[g * QP + d] = __float2bfloat16_rn(rotated_feature(p, L, acc_row, inv, r, (kvh * G + g) * HD + d, true));
    }
    if (owner) {
        const long long slot = __ldg(p.slot_mapping[L->group] + r);
        for (int i = wt; i < 2 * HD; i += WORKERS) {
            const bool is_v = i >= HD;
            const int d = is_v ? i - HD : i;
            const int n = (p.Hq + (is_v ? p.Hkv : 0) + kvh) * HD + d;
            const __nv_bfloat16 h = __float2bfloat16_rn(rotated_feature(p, L, acc_row, inv, r, n, !is_v));
            new_s[i] = __bfloat162float(h);
            if (slot >= 0) (is_v ? L->v_cache : L->k_cache)[((size_t)slot * p.Hkv + kvh) * HD + d] = h;
        }
    }
    worker_sync();

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
    const uint32_t wbase = smem_u32(attn) + warp * 4 * TILE_BYTES;      // per warp: K[2], V[2]
    const size_t row_stride = (size_t)p.Hkv * HD;
    auto slot_of = [&](int kb) -> long long {
        const int kpos = kb + lane;
        if (lane >= BK || kpos >= khi) return -1;
        return (long long)__ldg(bt + kpos / p.page_size) * p.page_size + (kpos % p.page_size);
    };
    auto issue = [&](int buf, long long slot) {
        const uint32_t kbase = wbase + buf * TILE_BYTES, vbase = wbase + (2 + buf) * TILE_BYTES;
#pragma unroll
        for (int it = 0; it < (BK * CH) / 32; ++it) {
            const int idx = it * 32 + lane;
            const int row = idx / CH, ch = idx % CH;
            const long long s = __shfl_sync(0xffffffffu, slot, row);
            const bool valid = s >= 0;
            const size_t off = (valid ? (size_t)s : 0) * row_stride + (size_t)kvh * HD + ch * 8;
            cp_async16(kv_tile_addr<HD>(kbase, row, ch), L->k_cache + off, valid);
            cp_async16(kv_tile_addr<HD>(vbase, row, ch), L->v_cache + off, valid);
        }
        cp_async_commit();
    };

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    const int kb_first = klo + warp * BK;
    int buf = 0;
    if (kb_first < khi) issue(0, slot_of(kb_first));
    for (int kb = kb_first; kb < khi; kb += ATTN_WARPS * BK) {
        const int kb_next = kb + ATTN_WARPS * BK;
        if (kb_next < khi) {
            issue(buf ^ 1, slot_of(kb_next));
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

    // Merge the warps through shared memory (the tile buffers are free now); the new token is a fifth entry.
    worker_sync();
    float* wacc = reinterpret_cast<float*>(attn);                       // [5][16][HD]
    float* wml = wacc + (ATTN_WARPS + 1) * 16 * HD;                     // [5][16][2]
    {
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
    }
    if (wt < 16) {      // the new token's score for each head of the group: q . k_new, keys and queries as bf16
        float sc = -INFINITY;
        if (owner && wt < G) {
            float dot = 0.0f;
            for (int d = 0; d < HD; ++d) dot = fmaf(__bfloat162float(q_s[wt * QP + d]), new_s[d], dot);
            sc = dot * p.scale_log2e;
        }
        wml[(ATTN_WARPS * 16 + wt) * 2] = sc;
        wml[(ATTN_WARPS * 16 + wt) * 2 + 1] = owner ? 1.0f : 0.0f;
    }
    worker_sync();
    const size_t base = ((size_t)(r * p.Hkv + kvh) * p.nsplit + sp) * G;
    for (int i = wt; i < G * HD; i += WORKERS) {
        const int g = i / HD, d = i - g * HD;
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w <= ATTN_WARPS; ++w) Mx = fmaxf(Mx, wml[(w * 16 + g) * 2]);
        float Ls = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w <= ATTN_WARPS; ++w) {
            const float mw = wml[(w * 16 + g) * 2];
            if (mw != -INFINITY) {
                const float e = fast_exp2(mw - Mx);
                Ls = fmaf(e, wml[(w * 16 + g) * 2 + 1], Ls);
                a = fmaf(e, w < ATTN_WARPS ? wacc[(size_t)(w * 16 + g) * HD + d] : new_s[HD + d], a);
            }
        }
        p.part_acc[(base + g) * HD + d] = a;
        if (d == 0) {
            p.part_ml[(base + g) * 2] = Mx;
            p.part_ml[(base + g) * 2 + 1] = Ls;
        }
    }
    worker_sync();            // the staged q, the new token and the merge area are free for the next item
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1) decode_layers_kernel(const FusedParams p) {
    constexpr uint32_t B_BYTES = BN * TILE_K * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    __shared__ __align__(8) uint64_t full_a[STAGES], full_b[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_s;
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
            mbar_init(&full_b[s], WORKERS);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], WORKERS);
        }
        abort_s = 0;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        // ---- weight tiles, in the order in which the block will use them, as far ahead as the ring allows ----------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int l = 0; l < p.num_layers && ok; ++l) {
                const LayerDesc* L = p.layers + l;
                for (int st = 0; st < 4 && ok; ++st) {
                    const StageInfo si = stage_info(p, L, st);
                    long long lo, hi;
                    stage_range(si, lo, hi);
                    for (long long i = lo; i < hi; ++i, ++it) {
                        const int nt = (int)(i / si.NKB), kb = (int)(i - (long long)nt * si.NKB), s = it % STAGES;
                        if (!mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag)) { ok = false; break; }
                        mbar_expect_tx(&full_a[s], A_BYTES);
                        tma_load_2d(a_tiles + s * A_BYTES, si.map, kb * TILE_K, nt * TILE_M, &full_a[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core instructions ------------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(TILE_M, BN);
            uint32_t it = 0, ua = 0;
            bool ok = true;
            for (int l = 0; l < p.num_layers && ok; ++l) {
                const LayerDesc* L = p.layers + l;
                for (int st = 0; st < 4 && ok; ++st) {
                    const StageInfo si = stage_info(p, L, st);
                    long long lo, hi;
                    stage_range(si, lo, hi);
                    for (long long i = lo; i < hi && ok;) {
                        const int kb0 = (int)(i % si.NKB);
                        const int n = (int)min((long long)(si.NKB - kb0), hi - i);
                        const int buf = ua & 1;
                        ok = mbar_wait(&acc_empty[buf], ((ua >> 1) & 1) ^ 1, abort_flag);
                        for (int k = 0; k < n && ok; ++k, ++it) {
                            const int s = it % STAGES;
                            ok = mbar_wait(&full_a[s], (it / STAGES) & 1, abort_flag) &&
                                 mbar_wait(&full_b[s], (it / STAGES) & 1, abort_flag);
                            if (!ok) break;
                            tc_fence_after();
                            const uint32_t a_addr = smem_u32(a_tiles + s * A_BYTES), b_addr = smem_u32(b_tiles + s * B_BYTES);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                umma_bf16(tmem_base + buf * BN, desc_kmajor(a_addr + j * 32), desc_kmajor(b_addr + j * 32),
                                          idesc, (k > 0 || j > 0) ? 1u : 0u);
                            umma_commit(&empty_bar[s]);
                        }
                        if (ok) umma_commit(&acc_full[buf]);
                        ++ua;
                        i += n;
                    }
                }
            }
        }
    } else {
        // ---- workers -------------------------------------------------------------------------------------------------
        const int wt = threadIdx.x - 64;
        const int quarter = warp & 3;
        const int Nqkv = (p.Hq + 2 * p.Hkv) * p.hd;
        uint32_t it = 0, ua = 0;
        unsigned epoch = 0;

        // Drain accumulator `u` (row tile nt of a stage with N outputs) into target [M, N] by atomic adds.
        auto drain = [&](uint32_t u, int nt, int N, float* target) {
            const int buf = u & 1;
            const bool ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (u >> 1) & 1, abort_flag));
            tc_fence_after();
            const int n = nt * TILE_M + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
            if (ok) {      // uniform over the warp: tcgen05.ld is a warp-wide instruction
#pragma unroll 1
                for (int c0 = 0; c0 < BN && c0 < p.M; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < p.M && n < N) red_add(target + (size_t)(c0 + j) * N + n, v[j]);
                }
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[buf]);
        };
        // One contraction stage: B operands for this block's units, accumulators drained one unit behind.
        auto gemm_stage = [&](const LayerDesc* L, int st, float* target) {
            const StageInfo si = stage_info(p, L, st);
            long long lo, hi;
            stage_range(si, lo, hi);
            int prev_nt = -1;
            uint32_t prev_u = 0;
            for (long long i = lo; i < hi;) {
                const int nt = (int)(i / si.NKB), kb0 = (int)(i - (long long)nt * si.NKB);
                const int n = (int)min((long long)(si.NKB - kb0), hi - i);
                for (int k = 0; k < n; ++k, ++it) {
                    const int s = it % STAGES, kb = kb0 + k;
                    uint8_t* tile = b_tiles + s * B_BYTES;
                    // the warp builds together (its lanes exchange sums of squares), so it goes ahead together
                    if (__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, abort_flag))) {
                        if (st == ST_QKV) build_b_norm(p, L->norm1_w, L->norm_w_bf16, kb, nt == 0 ? p.ss1 : nullptr, tile, wt);
                        else if (st == ST_GU) build_b_norm(p, L->norm2_w, L->norm_w_bf16, kb, nt == 0 ? p.ss2 : nullptr, tile, wt);
                        else if (st == ST_O) build_b_merge(p, kb, tile, wt);
                        else build_b_swiglu(p, L->eps2, kb, tile, wt);
                        fence_async_smem();
                    }
                    mbar_arrive(&full_b[s]);
                }
                if (prev_nt >= 0) drain(prev_u, prev_nt, si.N, target);
                prev_nt = nt;
                prev_u = ua++;
                i += n;
            }
            if (prev_nt >= 0) drain(prev_u, prev_nt, si.N, target);
        };
        auto zero_slice = [&](float* buf, long long count) {       // this block's part of a scratch array
            const long long lo = count * blockIdx.x / gridDim.x, hi = count * (blockIdx.x + 1) / gridDim.x;
            for (long long i = lo + wt; i < hi; i += WORKERS) buf[i] = 0.0f;
        };

        // Everything that is added into starts at zero, whatever an earlier launch left.
        zero_slice(p.qkv_acc, (long long)p.M * Nqkv);
        zero_slice(p.gu_acc, (long long)p.M * 2 * p.I);
        zero_slice(p.ss1, 64);
        zero_slice(p.ss2, 64);
        grid_barrier(p, epoch, abort_flag);

        for (int l = 0; l < p.num_layers; ++l) {
            const LayerDesc* L = p.layers + l;
            if (l > 0) {       // the last layer's feed-forward has read them; S4 of this layer adds into them again
                zero_slice(p.gu_acc, (long long)p.M * 2 * p.I);
                zero_slice(p.ss2, 64);
            }
            gemm_stage(L, ST_QKV, p.qkv_acc);
            grid_barrier(p, epoch, abort_flag);

            const int items = p.M * p.Hkv * p.nsplit;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {      // no waits inside: nothing to give up on
                if (p.hd == 64) attention_item<64>(p, L, item, attn, q_s, new_s, wt);
                else attention_item<128>(p, L, item, attn, q_s, new_s, wt);
            }
            grid_barrier(p, epoch, abort_flag);

            gemm_stage(L, ST_O, p.residual);
            grid_barrier(p, epoch, abort_flag);

            zero_slice(p.qkv_acc, (long long)p.M * Nqkv);     // S2 has read them; the next layer adds into them again
            zero_slice(p.ss1, 64);
            gemm_stage(L, ST_GU, p.gu_acc);
            grid_barrier(p, epoch, abort_flag);

            gemm_stage(L, ST_DOWN, p.residual);
            grid_barrier(p, epoch, abort_flag);
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

template <int BN>
int launch_fused(const FusedParams& p, cudaStream_t stream) {
    constexpr int STAGES = StagesFor<BN>::value;
    const size_t smem = fused_smem_bytes<BN>();
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_layers_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_layers_kernel<BN, STAGES>, p);
    if (e != cudaSuccess) return llb_fail("decode_layers: launch failed: %s", cudaGetErrorString(e));
    return llb_check_launch("decode_layers");
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
LLB_EXPORT int llb_decode_layers(const void* layers, int num_layers, float* residual, int M, int D, int Hq, int Hkv, int hd,
                                 int I, int rotary_dim, int interleaved, float scale, const float* rope_table,
                                 const int* span_pos, const int* bt0, const int* bt1, const int* bt2, const int* bt3,
                                 const int* sm0, const int* sm1, const int* sm2, const int* sm3, int max_pages,
                                 int page_size, int nsplit, float* scratch, long long scratch_floats, unsigned* sync,
                                 int* error_flag, cudaStream_t stream) {
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
    p.sync = sync; p.error_flag = error_flag;
    if (M <= 16) return launch_fused<16>(p, stream);
    if (M <= 32) return launch_fused<32>(p, stream);
    return launch_fused<64>(p, stream);
}
