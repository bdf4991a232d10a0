// Paged flash-attention for prompt portions on the 5th-generation tensor cores (sm_100a, bf16).
//
// A work item is 128 consecutive query rows of one span and one query head over a range of key tiles.
// Blocks are persistent: each walks through its share of the items with three roles, a loader warp, a warp
// that issues the tensor-core instructions, and eight softmax warps.  Keys and values come from the
// request's pages, 128 keys at a time: TMA copies each page of the tile (a box of page_size rows x 64
// elements) into a swizzled shared-memory tile, double buffered, ahead of use and across item boundaries.  Then
//     S = Q K^T          tcgen05.mma, both operands K-major, S in tensor memory (128 columns); issued for tile
//                        j+1 as soon as S of tile j has been read
//     softmax            two threads per query row (each half of the tile's keys) read S with tcgen05.ld; scale, mask by
//                        absolute position (and window) with selects, running max and sum in float
//     O_tile = P V       P (bf16) goes back to shared memory as the A operand; V is the B operand in
//                        MN-major form (its rows are keys), result in tensor memory
//     O = O * e^(m_old - m_new) + O_tile   in registers, float
// and finally O / l is written as bf16.  Formulas as src/kv_cache/paged_attention.cu:153-163 (scores,
// online softmax) with the same departures as the CUDA-core kernel of this library: -inf start, exact
// acc / l, the token's own key visible, every portion causal, page size a parameter.
//
// Head sizes 64 and 128; page sizes that divide 128 and are multiples of 8.  Other shapes use the
// CUDA-core kernel.  Every wait on an mbarrier is bounded in time; when one runs out the block raises
// the error flag, walks through the rest of its items without work, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "tcgen05_common.cuh"
#include "warp_mma.cuh"

namespace {

using namespace t5;
using wm::fast_exp2;

constexpr int BQ = 128;     // query rows per block = TMEM lanes
constexpr int BKV = 128;    // keys per tile
constexpr int NUM_THREADS = 320;   // 8 softmax warps (two threads per query row: each takes half of a tile's keys and
                                   // half of the output), the warp that issues tensor-core work, the loader warp
constexpr int MMA_WARP = 8, LOAD_WARP = 9;

// Masking is a select on the column index, never a branch: columns c_lo .. c_hi of the tile are this row's
// visible keys (causal, the span's end, the window's start; c_hi < c_lo when none is).
__device__ __forceinline__ float masked(float s, int col, int c_lo, int c_hi) {
    return (col >= c_lo && col <= c_hi) ? s : -INFINITY;
}
// Largest raw score of this thread's row among the visible keys of its two 32-column chunks of the tile.
template <bool MASKED>
__device__ __forceinline__ float row_max(uint32_t tmem_s, int c_begin, int c_lo, int c_hi) {
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll 1
    for (int c = c_begin; c < c_begin + 2; ++c) {
        float s[32];
        tmem_ld32(tmem_s + c * 32, s);
        if (MASKED) {
#pragma unroll
            for (int i = 0; i < 32; ++i) s[i] = masked(s[i], c * 32 + i, c_lo, c_hi);
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            m0 = fmaxf(m0, s[i]); m1 = fmaxf(m1, s[i + 1]); m2 = fmaxf(m2, s[i + 2]); m3 = fmaxf(m3, s[i + 3]);
        }
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}
// p = 2^(s*c - m) of this thread's 64 scores of the row, written as bf16 into the swizzled A-operand tiles; returns
// their sum (float, before rounding).  Row r, 16-byte chunk q of a 128-byte row lands at chunk q ^ (r & 7).
template <bool MASKED>
__device__ __forceinline__ float row_probs(uint32_t tmem_s, uint8_t* p_s, int r, int c_begin, float c_scale, float m_use,
                                           int c_lo, int c_hi) {
    float l0 = 0.0f, l1 = 0.0f;
#pragma unroll 1
    for (int c = c_begin; c < c_begin + 2; ++c) {
        float s[32];
        tmem_ld32(tmem_s + c * 32, s);
        if (MASKED) {
#pragma unroll
            for (int i = 0; i < 32; ++i) s[i] = masked(s[i], c * 32 + i, c_lo, c_hi);
        }
        uint8_t* prow = p_s + (c >> 1) * (128 * 128) + (uint32_t)r * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p0 = fast_exp2(fmaf(s[q * 8 + 2 * e], c_scale, -m_use));
                const float p1 = fast_exp2(fmaf(s[q * 8 + 2 * e + 1], c_scale, -m_use));
                l0 += p0;
                l1 += p1;
                const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                w[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
            *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
    return l0 + l1;
}

struct AttnTcParams {
    __nv_bfloat16* out;        // [T, Hq, HD]
    const int* tile_span;
    const int* tile_q0;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* block_table;    // [S, max_pages]
    int max_pages, page_size, Hq, Hkv, window, num_slots, num_items;
    float scale_log2e;         // scale * log2(e): scores are kept in base-2 units
    uint32_t dynamic_smem_bytes;
    // Optional cut of a tile's key range into work items, so that long rows do not set the kernel's time:
    // item i covers key tiles [tile_k0[i], tile_k0[i] + tile_nk[i]) of its query tile and, when tile_part[i] >= 0,
    // leaves its unnormalised (O, m, l) in part_o / part_ml for the merge kernel instead of writing the output.
    const int* tile_k0;
    const int* tile_nk;
    const int* tile_part;
    float* part_o;             // [parts, Hq, 128, HD]
    float* part_ml;            // [parts, Hq, 128, 2]  (m in base-2 units, l)
    int* error_flag;
};

// What one work item is: 128 query rows of one span and one head over a range of key tiles.
struct Item {
    int head, span, row0, nrows, pos0, hi, lo, kt0, ntiles, part;
};
__device__ __forceinline__ Item make_item(const AttnTcParams& p, int idx) {
    Item it;
    const int tile = idx / p.Hq;
    it.head = idx - tile * p.Hq;
    it.span = p.tile_span[tile];
    const int q0 = p.tile_q0[tile];
    it.row0 = p.span_row[it.span] + q0;
    it.nrows = min(BQ, p.span_len[it.span] - q0);
    it.pos0 = p.span_pos[it.span] + q0;
    it.hi = it.pos0 + it.nrows;                                    // keys [lo, hi) can be visible
    it.lo = p.window > 0 ? max(0, it.pos0 - p.window + 1) : 0;
    const int k_first = p.tile_k0 ? p.tile_k0[tile] : 0;
    it.kt0 = (it.lo / BKV) * BKV + k_first * BKV;
    const int all_tiles = (it.hi - (it.lo / BKV) * BKV + BKV - 1) / BKV - k_first;
    it.ntiles = max(0, p.tile_nk ? min(p.tile_nk[tile], all_tiles) : all_tiles);
    it.part = p.tile_part ? p.tile_part[tile] : -1;
    return it;
}

// Named barriers of the block (0 is __syncthreads).
constexpr int BAR_SOFTMAX = 1;     // the 256 softmax threads: the halves of a row have exchanged their maxima
constexpr int BAR_P_READY = 2;     // softmax threads and the MMA warp: S is read, P is in shared memory
constexpr int BAR_TILE_END = 3;    // softmax threads and the MMA warp: the tile's P V result is read
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// A persistent block: it takes one work item of every round of gridDim.x items (item = query tile x head, heads
// fastest, so that neighbouring blocks read the same keys) and keeps three roles busy:
//   warp 9   loader: Q of the next item and the key/value tiles, two stages ahead, across item boundaries
//   warp 8   issues the tensor-core instructions: S of tile j+1 right after P V of tile j
//   warps 0-7  softmax, two threads per query row
// The roles meet on mbarriers (data arrived, buffers free, tensor-core work done; every wait is bounded) and on
// named barriers among softmax and MMA warps.  After a wait has run out every role still walks through all its
// items and barriers, without copies, tensor-core work or stores, so that no barrier is left waiting.
template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, HD <= 64 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const AttnTcParams p) {
    constexpr int KB = HD / 64;                       // 64-element blocks along the head dimension
    constexpr uint32_t TILE_BYTES = 128 * 128;        // a [128 rows][64 elements] bf16 tile
    constexpr uint32_t TMEM_COLS = 256;               // S: columns 0..127, P V: columns 128..128+HD-1
    // Barriers live in static shared memory; the operand tiles in dynamic shared memory, aligned to
    // 1024 bytes for the swizzle.  The sizes are chosen so that two blocks of the head-64 kernel fit
    // in one SM, which leaves no room to spare: the fit is checked before anything is copied.
    __shared__ __align__(8) uint64_t bars[8];
    __shared__ uint32_t tmem_slot_s;
    __shared__ int abort_s;
    // The halves of a row agree on its maximum through this buffer.  The value is rounded up to bf16: any
    // common shift works for the softmax, and 512 bytes keep two blocks of the head-64 kernel within one SM.
    __shared__ __nv_bfloat16 xch[2][BQ];
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;                              // KB tiles
    uint8_t* k_s = q_s + KB * TILE_BYTES;             // 2 stages x KB tiles
    uint8_t* v_s = k_s + 2 * KB * TILE_BYTES;         // 2 stages x KB tiles
    uint8_t* p_s = v_s + 2 * KB * TILE_BYTES;         // 2 tiles (keys 0..63, 64..127)
    uint64_t* bar_q_full = &bars[0];
    uint64_t* bar_q_free = &bars[1];                  // the item's last S = Q K^T has been computed (a softmax thread arrives)
    uint64_t* bar_kv_full = &bars[2];                 // [2]
    uint64_t* bar_kv_free = &bars[4];                 // [2] the tile's P V has been computed (a softmax thread arrives)
    uint64_t* bar_s = &bars[6];
    uint64_t* bar_pv = &bars[7];
    uint32_t* tmem_slot = &tmem_slot_s;
    volatile int* abort_flag = &abort_s;
    if (p_s + 2 * TILE_BYTES > smem_raw + p.dynamic_smem_bytes) {     // uniform over the block
        if (threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 3);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) mbar_init(&bars[i], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: set-up is done; from here on global memory is touched, so the kernel before
    // this one must have completed.  The kernel after this one may start its set-up as blocks of this one leave.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int total = p.num_items;
    // The items come longest first.  Dealt round-robin, the blocks that got the longest items of one round would also
    // get the longest of the next; so every other round is dealt backwards, and a block's load stays near the mean.
    auto item_index = [&](int round) {
        return round * (int)gridDim.x + ((round & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
    };
    const int group = p.Hq / p.Hkv;
    constexpr uint32_t IDESC_S = idesc_bf16(BQ, BKV, 0);
    constexpr uint32_t IDESC_PV = idesc_bf16(BQ, HD, 1);
    constexpr int NUM_SOFTMAX = 256;

    if (warp == LOAD_WARP) {
        // ---- loader ------------------------------------------------------------------------------
        bool ok = true;
        uint32_t n_kv = 0, n_item = 0;
        for (int round = 0; round * (int)gridDim.x < total; ++round) {
            const int idx = item_index(round);
            if (idx >= total) continue;
            const Item it = make_item(p, idx);
            if (it.ntiles <= 0) continue;        // cannot happen with the lists the engine makes; every role skips it alike
            const int kvh = it.head / group;
            const int* bt = p.block_table + (size_t)it.span * p.max_pages;
            if (n_item > 0) ok = mbar_wait(bar_q_free, (n_item - 1) & 1, abort_flag) && ok;
            if (lane == 0 && ok) {
                mbar_expect_tx(bar_q_full, KB * TILE_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
                    tma_load_2d(q_s + kb * TILE_BYTES, &map_q, it.head * HD + kb * 64, it.row0, bar_q_full);
            }
            for (int j = 0; j < it.ntiles; ++j, ++n_kv) {
                const int st = n_kv & 1;
                const int kt = it.kt0 + j * BKV;
                // page numbers first: their latency then lies under the wait for the stage
                const int ppt = BKV / p.page_size;
                const int lp = kt / p.page_size + lane;
                // only pages that hold keys of [lo, hi): what lies beyond the request's own keys is never read
                const bool holds_keys = lp * p.page_size < it.hi && (lp + 1) * p.page_size > it.lo;
                const int page = (lane < ppt && lp < p.max_pages && holds_keys) ? bt[lp] : -1;
                if (n_kv >= 2) ok = mbar_wait(&bar_kv_free[st], ((n_kv >> 1) - 1) & 1, abort_flag) && ok;
                if (!ok) continue;
                if (lane == 0) mbar_expect_tx(&bar_kv_full[st], 2 * KB * TILE_BYTES);
                __syncwarp();
                if (lane < ppt) {
                    const int y = page >= 0 ? page * p.page_size : p.num_slots;   // out of range: the box is zero-filled
                    const uint32_t off = (uint32_t)lane * p.page_size * 128;
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb) {
                        tma_load_2d(k_s + (st * KB + kb) * TILE_BYTES + off, &map_k, kvh * HD + kb * 64, y, &bar_kv_full[st]);
                        tma_load_2d(v_s + (st * KB + kb) * TILE_BYTES + off, &map_v, kvh * HD + kb * 64, y, &bar_kv_full[st]);
                    }
                }
                __syncwarp();
            }
            ++n_item;
        }
    } else if (warp == MMA_WARP) {
        // ---- tensor-core instructions ----------------------------------------------------------------
        bool ok = true;
        uint32_t n_kv = 0, n_item = 0;
        // A tcgen05.commit is dear (the tensor pipe takes one about every 470 cycles, more than this kernel's
        // MMAs of a tile need), so there is one per tile: behind P V of tile j and S of tile j+1 together, plus one
        // behind the first S of an item.  The barriers that only say "this buffer may be overwritten" are arrived
        // at by a softmax thread once it has seen that commit.
        auto issue_s = [&](int st) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem_base, desc_kmajor(smem_u32(q_s + kb * TILE_BYTES) + k * 32),
                              desc_kmajor(smem_u32(k_s + (st * KB + kb) * TILE_BYTES) + k * 32), IDESC_S,
                              (kb > 0 || k > 0) ? 1u : 0u);
        };
        for (int round = 0; round * (int)gridDim.x < total; ++round) {
            const int idx = item_index(round);
            if (idx >= total) continue;
            const Item it = make_item(p, idx);
            if (it.ntiles <= 0) continue;
            ok = mbar_wait(bar_q_full, n_item & 1, abort_flag) && ok;
            for (int j = 0; j < it.ntiles; ++j, ++n_kv) {
                const int st = n_kv & 1;
                if (j == 0) {
                    ok = mbar_wait(&bar_kv_full[st], (n_kv >> 1) & 1, abort_flag) && ok;
                    if (lane == 0 && ok) {
                        issue_s(st);
                        umma_commit(bar_s);
                    }
                    __syncwarp();
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                named_barrier(BAR_P_READY, NUM_SOFTMAX + 32);
                if (lane == 0 && ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // O_tile[128 x HD] = P[128 x 128 keys] V[128 keys x HD]; 16 keys per instruction
#pragma unroll
                    for (int k = 0; k < BKV / 16; ++k)
                        umma_bf16(tmem_base + 128, desc_kmajor(smem_u32(p_s + (k >> 2) * TILE_BYTES) + (k & 3) * 32),
                                  desc_mnmajor(smem_u32(v_s + st * KB * TILE_BYTES) + k * 16 * 128, TILE_BYTES), IDESC_PV,
                                  k > 0 ? 1u : 0u);
                }
                __syncwarp();
                if (j + 1 < it.ntiles) {
                    // S of the next tile follows at once; it is complete when the softmax threads have read P V
                    const uint32_t n2 = n_kv + 1;
                    ok = mbar_wait(&bar_kv_full[n2 & 1], (n2 >> 1) & 1, abort_flag) && ok;
                    if (lane == 0 && ok) issue_s(n2 & 1);
                    __syncwarp();
                }
                if (lane == 0 && ok) umma_commit(bar_pv);     // P V of this tile and S of the next
                __syncwarp();
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                named_barrier(BAR_TILE_END, NUM_SOFTMAX + 32);
            }
            ++n_item;
        }
    } else {
        // ---- softmax ---------------------------------------------------------------------------------
        const int half = warp >> 2;                       // which half of the keys (and of the output dimensions)
        const uint32_t tmem_s = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t tmem_o = tmem_s + 128 + half * (HD / 2);
        const int r = threadIdx.x & (BQ - 1);       // query row of this thread = TMEM lane
        constexpr int HO = HD / 2;                  // output dimensions of this thread
        bool ok = true;
        uint32_t n_s = 0, n_item = 0;
        for (int round = 0; round * (int)gridDim.x < total; ++round) {
            const int idx = item_index(round);
            if (idx >= total) continue;
            const Item it = make_item(p, idx);
            if (it.ntiles <= 0) continue;
            const int qpos = it.pos0 + r;
            // visible keys of this row: positions vis_lo .. vis_hi
            const int vis_lo = p.window > 0 ? max(it.lo, qpos - p.window + 1) : it.lo;
            const int vis_hi = min(qpos, it.hi - 1);
            float o[HO];
#pragma unroll
            for (int d = 0; d < HO; ++d) o[d] = 0.0f;
            float m_run = -INFINITY, l_run = 0.0f;
            for (int j = 0; j < it.ntiles; ++j, ++n_s) {
                const int kt = it.kt0 + j * BKV;
                if (j == 0) {      // later tiles' S came with the commit behind the tile before them
                    ok = mbar_wait(bar_s, n_item & 1, abort_flag) && ok;
                    if (threadIdx.x == 0 && it.ntiles == 1) mbar_arrive(bar_q_free);     // the item's last S has read Q
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (kt + BKV > it.hi && kt + r >= it.hi) {
                    // The span's last page may hold rows that no token has written yet (what an earlier owner left
                    // there).  Their probabilities are exact zeros, but zero times anything must stay zero: the V
                    // rows of the keys from `hi` on are cleared before P V reads them.  (S is complete, so the tile's
                    // copies have landed; a row is 128 bytes in every 64-column tile, each half-thread clears 64.)
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb) {
                        uint4* vrow = reinterpret_cast<uint4*>(v_s + ((n_s & 1) * KB + kb) * TILE_BYTES + (uint32_t)r * 128 + half * 64);
#pragma unroll
                        for (int q = 0; q < 4; ++q) vrow[q] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                // Softmax of this thread's row over its 64 keys of the tile, in two passes over tensor memory
                // (maximum first, then the probabilities), 32 columns at a time.  Tiles that lie wholly below
                // the diagonal and inside the window of every row of the block skip the masking.
                const bool interior = (kt + BKV - 1 <= it.pos0) && (p.window <= 0 || (it.pos0 + BQ - 1) - kt < p.window);
                const int c_lo = vis_lo - kt, c_hi = vis_hi - kt;
                float m_tile;
                if (interior) m_tile = row_max<false>(tmem_s, 2 * half, c_lo, c_hi);
                else m_tile = row_max<true>(tmem_s, 2 * half, c_lo, c_hi);
                xch[half][r] = __float2bfloat16_ru(m_tile);      // rewritten only after the barriers further down
                named_barrier(BAR_SOFTMAX, NUM_SOFTMAX);
                m_tile = fmaxf(__bfloat162float(xch[0][r]), __bfloat162float(xch[1][r])) * p.scale_log2e;   // the scale is positive
                const float m_new = fmaxf(m_run, m_tile);
                const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;      // nothing visible yet: all p are 0
                const float corr = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_use);
                float l_tile;
                if (interior) l_tile = row_probs<false>(tmem_s, p_s, r, 2 * half, p.scale_log2e, m_use, c_lo, c_hi);
                else l_tile = row_probs<true>(tmem_s, p_s, r, 2 * half, p.scale_log2e, m_use, c_lo, c_hi);
                l_run = l_run * corr + l_tile;
                m_run = m_new;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // P is read by the tensor core
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                named_barrier(BAR_P_READY, NUM_SOFTMAX + 32);
                ok = mbar_wait(bar_pv, n_s & 1, abort_flag) && ok;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (threadIdx.x == 0) {
                    mbar_arrive(&bar_kv_free[n_s & 1]);                       // this tile's K and V have been read
                    if (j + 2 == it.ntiles) mbar_arrive(bar_q_free);           // and so has Q, by the item's last S
                }
#pragma unroll
                for (int c = 0; c < HO / 32; ++c) {
                    float t[32];
                    tmem_ld32(tmem_o + c * 32, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * corr + t[i];
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                named_barrier(BAR_TILE_END, NUM_SOFTMAX + 32);   // S's successor may be read, the P V columns overwritten
            }

            // The halves of a row add up their sums; each writes its half of the dimensions.  The P tile is idle:
            // its last reader (the tile's P V) has completed, and the next item's P is written only after a
            // barrier of all softmax threads.
            float* lx = reinterpret_cast<float*>(p_s);
            lx[half * BQ + r] = l_run;
            named_barrier(BAR_SOFTMAX, NUM_SOFTMAX);
            const float l_row = lx[r] + lx[BQ + r];
            if (ok && r < it.nrows && it.part >= 0) {
                float* po = p.part_o + (((size_t)it.part * p.Hq + it.head) * BQ + r) * HD + half * HO;
#pragma unroll
                for (int d = 0; d < HO; d += 4)
                    *reinterpret_cast<float4*>(po + d) = make_float4(o[d], o[d + 1], o[d + 2], o[d + 3]);
                if (half == 0) {
                    float* pm = p.part_ml + (((size_t)it.part * p.Hq + it.head) * BQ + r) * 2;
                    pm[0] = m_run;
                    pm[1] = l_row;
                }
            } else if (ok && r < it.nrows) {
                const float inv = 1.0f / l_row;
                __nv_bfloat16* dst = p.out + ((size_t)(it.row0 + r) * p.Hq + it.head) * HD + half * HO;
#pragma unroll
                for (int d = 0; d < HO; d += 8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(o[d + 2 * e] * inv, o[d + 2 * e + 1] * inv);
                        w[e] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(dst + d) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            ++n_item;
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0 && p.error_flag) atomicExch(p.error_flag, 2);
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Merge of the items of one query tile: out = sum_c 2^(m_c - M) O_c / sum_c 2^(m_c - M) l_c.
struct MergeParams {
    __nv_bfloat16* out;
    const int* merge_span;     // [NM]
    const int* merge_q0;
    const int* merge_first;    // first part of the tile
    const int* merge_count;    // number of parts
    const int* span_row;
    const int* span_len;
    const float* part_o;
    const float* part_ml;
    int Hq, HD;
};

__global__ void __launch_bounds__(256) attention_tcgen05_merge_kernel(MergeParams p) {
    // A group of HD/4 threads takes one row (four dimensions each, so a row's loads are contiguous); the
    // blocks of grid.z share the tile's rows.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int mt = blockIdx.x, head = blockIdx.y;
    const int span = p.merge_span[mt], q0 = p.merge_q0[mt];
    const int nrows = min(BQ, p.span_len[span] - q0);
    const int first = p.merge_first[mt], count = p.merge_count[mt];
    const int HD = p.HD;
    const int tpr = HD / 4;                              // threads per row
    const int d = (threadIdx.x % tpr) * 4;
    const int rows_per_block = blockDim.x / tpr;
    for (int r = blockIdx.z * rows_per_block + threadIdx.x / tpr; r < nrows; r += gridDim.z * rows_per_block) {
        float M = -INFINITY;
        for (int c = 0; c < count; ++c) M = fmaxf(M, p.part_ml[(((size_t)(first + c) * p.Hq + head) * BQ + r) * 2]);
        float L = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int c = 0; c < count; ++c) {
            const size_t base = ((size_t)(first + c) * p.Hq + head) * BQ + r;
            const float m = p.part_ml[base * 2];
            if (m == -INFINITY) continue;
            const float w = fast_exp2(m - M);
            L += w * p.part_ml[base * 2 + 1];
            const float4 a = *reinterpret_cast<const float4*>(p.part_o + base * HD + d);
            acc.x += w * a.x; acc.y += w * a.y; acc.z += w * a.z; acc.w += w * a.w;
        }
        const float inv = 1.0f / L;
        __nv_bfloat16* dst = p.out + ((size_t)(p.span_row[span] + q0 + r) * p.Hq + head) * HD + d;
        const __nv_bfloat162 h0 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        const __nv_bfloat162 h1 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<const uint32_t*>(&h0),
                                                    *reinterpret_cast<const uint32_t*>(&h1));
    }
}

// ---------------------------------------------------------------------------------------------
// A map over a row-major bf16 matrix [rows, cols] with boxes of box_rows x 64 and the 128-byte swizzle.
int make_map(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
    return make_map_bf16(ptr, rows, cols, box_rows, out);
}

template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p, int num_tiles,
           cudaStream_t stream) {
    constexpr int KB = HD / 64;
    // 584 bytes of static shared memory (barriers, the halves' exchange) precede the tiles; the rest of the
    // kilobyte is what aligning the tiles to 1024 bytes can cost (checked in the kernel)
    constexpr size_t smem = (size_t)(KB + 4 * KB + 2) * 128 * 128 + 1024 - 592;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return llb_fail("attention_tcgen05: cannot opt in to %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
        configured = true;
    }
    static int num_sms = 0;
    if (num_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) {
            num_sms = 0;
            return llb_fail("attention_tcgen05: cannot ask the device for its number of SMs");
        }
    }
    AttnTcParams pp = p;
    pp.dynamic_smem_bytes = (uint32_t)smem;
    pp.num_items = num_tiles * p.Hq;
    const int resident = (HD <= 64 ? 2 : 1) * num_sms;       // persistent blocks: as many as stay on the device
    const int grid = pp.num_items < resident ? pp.num_items : resident;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_tcgen05_kernel<HD>, mq, mk, mv, pp);
    if (e != cudaSuccess) return llb_fail("attention_tcgen05: launch failed: %s", cudaGetErrorString(e));
    return llb_check_launch("attention_tcgen05");
}

}  // namespace

// Whether the tensor-core kernel takes this shape (else the CUDA-core kernel is the one to call).
LLB_EXPORT int llb_attention_tcgen05_supports(int hd, int page_size) {
    return (hd == 64 || hd == 128) && page_size >= 8 && page_size <= 128 && page_size % 8 == 0 && 128 % page_size == 0;
}

// q, out [T, Hq, hd] bf16; k_cache, v_cache [num_slots, Hkv, hd] bf16 with slot = page*page_size + offset;
// tiles of 128 query rows: tile_span, tile_q0 [num_tiles]; span_row, span_len, span_pos [S];
// block_table [S, max_pages].  window <= 0: every earlier key is visible.  tile_k0 / tile_nk / tile_part (or all
// null) cut tiles into items over ranges of 128-key tiles; items with tile_part >= 0 write partial results to
// part_scratch (num_parts * Hq * 128 * (hd + 2) floats) for llb_attention_tcgen05_merge.
LLB_EXPORT int llb_paged_attention_tcgen05(const void* q, const void* k_cache, const void* v_cache, void* out, int T,
                                           const int* tile_span, const int* tile_q0, int num_tiles,
                                           const int* span_row, const int* span_len, const int* span_pos,
                                           const int* block_table, int max_pages, int page_size, int num_slots,
                                           int Hq, int Hkv, int hd, int window, float scale, const int* tile_k0,
                                           const int* tile_nk, const int* tile_part, float* part_scratch,
                                           int num_parts, int* error_flag, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    LLB_REQUIRE(tile_part == nullptr || (tile_k0 && tile_nk && (num_parts == 0 || part_scratch)),
                "attention_tcgen05: a cut key range needs tile_k0, tile_nk, tile_part and scratch");
    LLB_REQUIRE(llb_attention_tcgen05_supports(hd, page_size),
                "attention_tcgen05: head_dim %d with page size %d is not supported (head 64 or 128; page size a "
                "multiple of 8 that divides 128)", hd, page_size);
    LLB_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Hq <= 65535 && (long long)num_tiles * Hq < (1ll << 30), "attention_tcgen05: bad head counts %d/%d", Hq, Hkv);
    LLB_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0) &&
                ((uintptr_t)out % 16 == 0), "attention_tcgen05: tensors must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = make_map(q, T, (long long)Hq * hd, BQ, &mq))) return rc;
    if ((rc = make_map(k_cache, num_slots, (long long)Hkv * hd, page_size, &mk))) return rc;
    if ((rc = make_map(v_cache, num_slots, (long long)Hkv * hd, page_size, &mv))) return rc;
    AttnTcParams p;
    p.out = (__nv_bfloat16*)out;
    p.tile_span = tile_span; p.tile_q0 = tile_q0; p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos;
    p.block_table = block_table; p.max_pages = max_pages; p.page_size = page_size; p.Hq = Hq; p.Hkv = Hkv;
    p.window = window; p.num_slots = num_slots; p.scale_log2e = scale * 1.4426950408889634f; p.error_flag = error_flag;
    p.tile_k0 = tile_k0; p.tile_nk = tile_nk; p.tile_part = tile_part;
    p.part_o = part_scratch;
    p.part_ml = part_scratch ? part_scratch + (size_t)num_parts * Hq * BQ * hd : nullptr;
    if (hd == 64) return launch<64>(mq, mk, mv, p, num_tiles, stream);
    return launch<128>(mq, mk, mv, p, num_tiles, stream);
}

// Merges the partial results of cut tiles: merge_span, merge_q0, merge_first, merge_count [num_merge] name each
// query tile, its first part and its number of parts.
LLB_EXPORT int llb_attention_tcgen05_merge(void* out, const int* merge_span, const int* merge_q0, const int* merge_first,
                                           const int* merge_count, int num_merge, const int* span_row,
                                           const int* span_len, const float* part_scratch, int num_parts, int Hq,
                                           int hd, cudaStream_t stream) {
    if (num_merge == 0) return 0;
    LLB_REQUIRE(num_merge > 0 && part_scratch && num_parts > 0 && Hq > 0 && Hq <= 65535 && hd % 8 == 0,
                "attention_tcgen05_merge: bad arguments");
    MergeParams p;
    p.out = (__nv_bfloat16*)out; p.merge_span = merge_span; p.merge_q0 = merge_q0; p.merge_first = merge_first;
    p.merge_count = merge_count; p.span_row = span_row; p.span_len = span_len; p.part_o = part_scratch;
    p.part_ml = part_scratch + (size_t)num_parts * Hq * BQ * hd; p.Hq = Hq; p.HD = hd;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_merge, Hq, BQ / (256 / (hd / 4)));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_tcgen05_merge_kernel, p);
    if (e != cudaSuccess) return llb_fail("attention_tcgen05_merge: launch failed: %s", cudaGetErrorString(e));
    return llb_check_launch("attention_tcgen05_merge");
}
