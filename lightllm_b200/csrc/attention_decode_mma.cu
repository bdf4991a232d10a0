// Split-KV paged attention for decode (one query row per request) on tensor cores, bf16.
//
// The G query heads that share a kv head (G <= 16) are the 16 rows of a warp-level MMA tile
// (mma.sync m16n8k16), so a 32-key tile of K and V costs a few dozen instructions instead of the
// thousands the CUDA-core kernel spends on it.  Each warp streams its own key tiles: cp.async copies
// the page rows into the warp's shared-memory buffers (two or three, so the next tiles are in flight
// while this one is computed; tiles of 32 or 16 keys, see Shape below), ldmatrix reads them as MMA fragments (K as is, V transposed), scores
// and the online softmax stay in registers in float (src/kv_cache/paged_attention.cu:153-163, with
// this library's departures: -inf start, exact acc / l, the token's own key visible).  The four warps
// of a block are merged through shared memory.  With 2 to 16 splits the blocks of one (request, kv head)
// form a thread-block cluster and merge their partial (acc, m, l) through distributed shared memory, in
// the same kernel; with more splits the partials go to scratch and a second kernel merges them
// (paged_attention.cu:476-532 does the same for 4 fixed splits).
//
// Both kernels are programmatic dependent launches: everything that does not depend on the previous
// kernel (block tables, positions, ranges) is read before griddepcontrol.wait.
#include <math.h>

#include "common.cuh"
#include "warp_mma.cuh"

namespace {

using namespace wm;

constexpr int NWARPS = 4;
constexpr int MERGE_MAX_SPLITS = 256;
constexpr int CLUSTER_MAX_SPLITS = 16;      // beyond the portable 8 the kernel opts in to larger clusters

struct DecodeParams {
    const __nv_bfloat16* q;        // [T, Hq, HD]
    const __nv_bfloat16* k_cache;  // [slots, Hkv, HD]
    const __nv_bfloat16* v_cache;
    __nv_bfloat16* out;            // [T, Hq, HD]
    const int* tile_span;
    const int* tile_q0;
    const int* span_row;
    const int* span_pos;
    const int* block_table;
    int max_pages, page_size, Hq, Hkv, window, nsplit;
    float scale_log2e;
    float* part_acc;               // [tiles, Hkv, nsplit, G, HD]
    float* part_ml;                // [tiles, Hkv, nsplit, G, 2]   (m in base-2 units, l)
};

// Distributed shared memory: the float at `local_addr` (a shared-memory address of this block) in the block of
// rank `rank` of the cluster.
__device__ __forceinline__ float ld_cluster_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
// Every thread of every block of the cluster arrives and waits (a hardware barrier: it has no time limit, so no
// block may leave the kernel or skip it on any path).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Shared memory tile [32 keys][HD] bf16; the 16-byte chunk c of row r sits at chunk c ^ (r & 7), so that
// the eight rows an ldmatrix touches fall into different banks.
template <int HD>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    return base + (uint32_t)row * (HD * 2) + (uint32_t)((chunk ^ (row & 7)) * 16);
}

// BK keys a tile (16 or 32), NST tile buffers a warp: NST - 1 tiles are in flight while one is computed.
template <int HD, bool CLUSTER, int BK, int NST>
__global__ void __launch_bounds__(NWARPS * 32) paged_decode_mma_kernel(DecodeParams p) {
    static_assert((BK == 16 || BK == 32) && NST >= 2 && NST <= 8, "tile shape");
    constexpr int CH = HD / 8;                 // 16-byte chunks per row
    constexpr int TILE_BYTES = BK * HD * 2;
    constexpr int NK = BK / 8;                 // n-tiles of S (8 keys each)
    constexpr int KJ = BK / 16;                // k-steps of P V (16 keys each)
    constexpr int KS = HD / 16;                // k-steps of Q K^T
    constexpr int NT = HD / 8;                 // n-tiles of P V
    extern __shared__ __align__(128) uint8_t smem[];
    // per warp: K[NST], V[NST]; afterwards reused for the merge of the warps
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t wbase = smem_addr(smem) + warp * 2 * NST * TILE_BYTES;
    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = p.Hq / p.Hkv;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int span = p.tile_span[tile];
    const int q0 = p.tile_q0[tile];
    const int row0 = p.span_row[span] + q0;
    const int qpos = p.span_pos[span] + q0;
    const int* bt = p.block_table + (size_t)span * p.max_pages;
    const int hi = qpos + 1;
    const int lo = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
    int klo = lo, khi = hi;
    if (p.nsplit > 1) {
        int chunk = (hi - lo + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + BK - 1) / BK) * BK;
        klo = lo + split * chunk;
        khi = min(hi, klo + chunk);
    }
    const size_t row_stride = (size_t)p.Hkv * HD;
    // cache row of this lane's key in a tile that starts at kb (only block tables are read: no dependency)
    // (an int: a row of a head is 128 bytes or more, so a plane of 2^31 rows would not fit the device's memory)
    auto slot_of = [&](int kb) -> int {
        const int kpos = kb + lane;
        if (lane >= BK || kpos >= khi) return -1;
        return bt[kpos / p.page_size] * p.page_size + (kpos % p.page_size);
    };
    const int kb_first = klo + warp * BK;
    // the cache rows of the tiles that go out before the first one is awaited
    int slot_ahead[NST - 1];
#pragma unroll
    for (int a = 0; a < NST - 1; ++a) slot_ahead[a] = slot_of(kb_first + a * NWARPS * BK);
    // ... and of the tile that goes out in the first iteration: every later one is looked up an iteration before it
    // is needed, so that the block table's latency is not part of an iteration
    int slot_q = slot_of(kb_first + (NST - 1) * NWARPS * BK);

    asm volatile("griddepcontrol.wait;" ::: "memory");

    // Q fragments: rows = heads of the group (zero beyond G), K-steps over the head dimension.
    uint32_t qf[KS][4];
    {
        const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
        const __nv_bfloat16* qb = p.q + ((size_t)row0 * p.Hq + kvh * G) * HD;
#pragma unroll
        for (int s = 0; s < KS; ++s) {
            qf[s][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(qb + r0 * HD + s * 16 + c) : 0u;
            qf[s][1] = r1 < G ? *reinterpret_cast<const uint32_t*>(qb + r1 * HD + s * 16 + c) : 0u;
            qf[s][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(qb + r0 * HD + s * 16 + 8 + c) : 0u;
            qf[s][3] = r1 < G ? *reinterpret_cast<const uint32_t*>(qb + r1 * HD + s * 16 + 8 + c) : 0u;
        }
    }
    // Issue the copies of one tile into buffer `buf`: BK rows x CH chunks of K and of V (nothing for a tile beyond
    // the range: `slot` is -1 in every lane), as one group.
    auto issue = [&](int buf, int slot, bool in_range) {
        const uint32_t kbase = wbase + buf * TILE_BYTES, vbase = wbase + (NST + buf) * TILE_BYTES;
#pragma unroll
        for (int it = 0; in_range && it < BK * CH / 32; ++it) {
            const int idx = it * 32 + lane;
            const int row = idx / CH, ch = idx % CH;
            const int s = __shfl_sync(0xffffffffu, slot, row);
            const bool valid = s >= 0;
            const size_t off = (size_t)(valid ? s : 0) * row_stride + (size_t)(kvh * HD + ch * 8);
            cp_async16(tile_addr<HD>(kbase, row, ch), p.k_cache + off, valid);
            cp_async16(tile_addr<HD>(vbase, row, ch), p.v_cache + off, valid);
        }
        cp_async_commit();
    };

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    int buf = 0;
#pragma unroll
    for (int a = 0; a < NST - 1; ++a) issue(a, slot_ahead[a], kb_first + a * NWARPS * BK < khi);
    for (int kb = kb_first; kb < khi; kb += NWARPS * BK) {
        // the tile NST - 1 ahead goes into the buffer that the last iteration read; then all but the newest NST - 1
        // groups are complete, this tile's among them
        const int kb_ahead = kb + (NST - 1) * NWARPS * BK;
        issue(buf == 0 ? NST - 1 : buf - 1, slot_q, kb_ahead < khi);
        slot_q = slot_of(kb_ahead + NWARPS * BK);
        cp_async_wait<NST - 1>();
        __syncwarp();
        const uint32_t kbase = wbase + buf * TILE_BYTES, vbase = wbase + (NST + buf) * TILE_BYTES;

        // S[16 x BK] = Q K^T: n-tiles of 8 keys.
        float s[NK][4];
#pragma unroll
        for (int i = 0; i < NK; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KS; ks += 2) {
#pragma unroll
            for (int i = 0; i < NK; ++i) {
                // matrices: keys 8i..8i+7 x dims [16ks, +8), [16ks+8, +8), [16ks+16, +8), [16ks+24, +8)
                uint32_t b[4];
                ldmatrix_x4(tile_addr<HD>(kbase, i * 8 + (lane & 7), ks * 2 + (lane >> 3)), b);
                mma_bf16(s[i], qf[ks], b[0], b[1]);
                mma_bf16(s[i], qf[ks + 1], b[2], b[3]);
            }
        }
        // Online softmax for rows r0 = lane / 4 (values [0], [1]) and r0 + 8 (values [2], [3]).
        const int c0 = (lane & 3) * 2;
        float mt[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < NK; ++i) {
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
        uint32_t pf[KJ][4];     // P as A fragments for the k-steps of 16 keys
#pragma unroll
        for (int i = 0; i < NK; ++i) {
            const float p0 = fast_exp2(s[i][0] - m_run[0]), p1 = fast_exp2(s[i][1] - m_run[0]);
            const float p2 = fast_exp2(s[i][2] - m_run[1]), p3 = fast_exp2(s[i][3] - m_run[1]);
            lt[0] += p0 + p1;
            lt[1] += p2 + p3;
            // n-tiles 2j and 2j+1 of S are the k-halves of A for k-step j: a0,a1 from tile 2j; a2,a3 from 2j+1
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
        // O[16 x HD] += P[16 x 32] V[32 x HD]: V fragments come transposed out of shared memory.
#pragma unroll
        for (int j = 0; j < KJ; ++j) {             // k-step: keys 16j .. 16j+15
#pragma unroll
            for (int i = 0; i < NT; i += 2) {      // two n-tiles (16 dims) per ldmatrix.x4
                // matrices: (keys 16j..+7, dims 8i..), (keys 16j+8..+15, dims 8i..), (keys 16j..+7, dims 8i+8..), (keys 16j+8.., dims 8i+8..)
                uint32_t b[4];
                const int mat = lane >> 3;
                ldmatrix_x4_trans(tile_addr<HD>(vbase, j * 16 + (mat & 1) * 8 + (lane & 7), i + (mat >> 1)), b);
                mma_bf16(o[i], pf[j], b[0], b[1]);
                mma_bf16(o[i + 1], pf[j], b[2], b[3]);
            }
        }
        buf = buf + 1 == NST ? 0 : buf + 1;
        __syncwarp();
    }
    cp_async_wait<0>();         // the empty groups of the tiles beyond the range

    // Merge the four warps through shared memory (the tile buffers are free now).
    __syncthreads();
    float* wacc = reinterpret_cast<float*>(smem);                  // [NWARPS][16][HD]
    float* wml = wacc + NWARPS * 16 * HD;                           // [NWARPS][16][2]
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
    __syncthreads();
    const size_t base = (((size_t)tile * p.Hkv + kvh) * p.nsplit + split) * G;
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int g = i / HD, d = i - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, wml[(w * 16 + g) * 2]);
        float L = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float mw = wml[(w * 16 + g) * 2];
            if (mw != -INFINITY) {
                const float e = fast_exp2(mw - M);
                L += e * wml[(w * 16 + g) * 2 + 1];
                a += e * wacc[(size_t)(w * 16 + g) * HD + d];
            }
        }
        if (CLUSTER) {
            float* pacc = wml + NWARPS * 16 * 2;      // [16][HD], then (m, l) [16][2]
            pacc[g * HD + d] = a;
            if (d == 0) {
                pacc[16 * HD + g * 2] = M;
                pacc[16 * HD + g * 2 + 1] = L;
            }
        } else if (p.nsplit == 1) {
            p.out[((size_t)row0 * p.Hq + kvh * G + g) * HD + d] = __float2bfloat16_rn(a / L);
        } else {
            p.part_acc[(base + g) * HD + d] = a;
            if (d == 0) {
                p.part_ml[(base + g) * 2] = M;
                p.part_ml[(base + g) * 2 + 1] = L;
            }
        }
    }
    if (CLUSTER) {
        // The splits of this (request, kv head) are the blocks of one cluster (rank = split).  Each block takes a
        // share of the outputs and reads every block's partial through distributed shared memory:
        // out = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s.
        cluster_sync_all();
        const uint32_t pacc_addr = smem_addr(wml + NWARPS * 16 * 2);
        const uint32_t pml_addr = pacc_addr + 16 * HD * 4;
        for (int i = split * blockDim.x + threadIdx.x; i < G * HD; i += p.nsplit * blockDim.x) {
            const int g = i / HD, d = i - g * HD;
            float M = -INFINITY;
            for (int sp = 0; sp < p.nsplit; ++sp) M = fmaxf(M, ld_cluster_f32(pml_addr + g * 8, sp));
            float L = 0.0f, a = 0.0f;
            for (int sp = 0; sp < p.nsplit; ++sp) {
                const float ms = ld_cluster_f32(pml_addr + g * 8, sp);
                if (ms != -INFINITY) {
                    const float e = fast_exp2(ms - M);
                    L += e * ld_cluster_f32(pml_addr + g * 8 + 4, sp);
                    a += e * ld_cluster_f32(pacc_addr + (g * HD + d) * 4, sp);
                }
            }
            p.out[((size_t)row0 * p.Hq + kvh * G + g) * HD + d] = __float2bfloat16_rn(a / L);
        }
        cluster_sync_all();        // no block leaves while another may still read its shared memory
    }
}

// out = sum_s 2^(m_s - M) acc_s / sum_s 2^(m_s - M) l_s; one warp per (tile, head).
__global__ void __launch_bounds__(32) decode_merge_kernel(DecodeParams p, int HD) {
    __shared__ float wsm[MERGE_MAX_SPLITS];
    const int tile = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int G = p.Hq / p.Hkv;
    const int kvh = head / G, g = head - kvh * G;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int span = p.tile_span[tile];
    const int row0 = p.span_row[span] + p.tile_q0[tile];
    const size_t base0 = ((size_t)tile * p.Hkv + kvh) * p.nsplit;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float M = -INFINITY;
    for (int s = lane; s < p.nsplit; s += 32) M = fmaxf(M, p.part_ml[((base0 + s) * G + g) * 2]);
    M = llb_warp_max(M);
    float L = 0.0f;
    for (int s = lane; s < p.nsplit; s += 32) {
        const size_t idx = (base0 + s) * G + g;
        const float m = p.part_ml[idx * 2];
        const float w = (m == -INFINITY) ? 0.0f : fast_exp2(m - M);
        wsm[s] = w;
        L += w * p.part_ml[idx * 2 + 1];
    }
    L = llb_warp_sum(L);
    __syncwarp();
    const float inv = 1.0f / L;
    for (int d = lane; d < HD; d += 32) {
        float a = 0.0f;
#pragma unroll 8
        for (int s = 0; s < p.nsplit; ++s) a = fmaf(wsm[s], p.part_acc[((base0 + s) * G + g) * HD + d], a);
        p.out[((size_t)row0 * p.Hq + head) * HD + d] = __float2bfloat16_rn(a * inv);
    }
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// Launch as a programmatic dependent launch whose grid.z is one thread-block cluster.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = grid.z;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// The tile shape of each head size.  What paces a warp is the issue of its own instructions (a tile of 16 keys of 128
// dimensions is some 300 of them, and a warp alone on its scheduler issues a dependent instruction every few cycles),
// not the bytes it has in flight: buffers for five tiles ahead with one block an SM measured slower than two buffers,
// and what helps is more warps an SM.  Measured over 64 requests of 8,192 keys, 4 kv heads of 128 (1.07 GB): 242 us
// with tiles of 32 keys, two buffers and one block an SM; 190 us (5.6 TB/s) with tiles of 16 keys, three buffers and
// two blocks an SM.  Heads of 64 hold three blocks an SM with tiles of 32 keys already; other shapes measured the same
// within 2 us there.
template <int HD> struct Shape;
template <> struct Shape<64> { static constexpr int BK = 32, NST = 2; };
template <> struct Shape<128> { static constexpr int BK = 16, NST = 3; };

template <int HD, int BK, int NST>
struct Launcher {
    static constexpr size_t smem = (size_t)NWARPS * 2 * NST * BK * HD * 2;     // also covers the merges: 4 x 16 x HD floats
                                                                               // + m, l, and the block's own 16 x HD + m, l
    static_assert(smem >= (size_t)(NWARPS + 1) * (16 * HD * 4 + 16 * 2 * 4), "merge area does not fit");
    static int configure() {
        static bool configured = false;
        if (configured) return 0;
        cudaError_t e = cudaSuccess;
        if (smem > 48 * 1024) {
            e = cudaFuncSetAttribute(paged_decode_mma_kernel<HD, false, BK, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(paged_decode_mma_kernel<HD, true, BK, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        }
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(paged_decode_mma_kernel<HD, true, BK, NST>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return llb_fail("decode attention: cannot set the kernel's attributes (%zu bytes of shared "
                                              "memory, clusters of %d): %s", smem, CLUSTER_MAX_SPLITS, cudaGetErrorString(e));
        configured = true;
        return 0;
    }
    // Blocks of this kernel that one SM holds at a time: its shared memory (228 KB, 1 KB of each block the system's) is what
    // limits them (the kernels take 128 to 168 registers a thread, which allows three blocks of 128 threads or more).
    static int resident() { return (int)((228 * 1024) / (smem + 1024)); }
    static int launch(const DecodeParams& p, int num_tiles, cudaStream_t stream) {
        int rc = configure();
        if (rc) return rc;
        const bool cluster = p.nsplit > 1 && p.nsplit <= CLUSTER_MAX_SPLITS;
        cudaError_t e;
        if (cluster)
            e = launch_pdl_cluster(paged_decode_mma_kernel<HD, true, BK, NST>, dim3(num_tiles, p.Hkv, p.nsplit), dim3(NWARPS * 32),
                                   smem, stream, p);
        else
            e = launch_pdl(paged_decode_mma_kernel<HD, false, BK, NST>, dim3(num_tiles, p.Hkv, p.nsplit), dim3(NWARPS * 32), smem,
                           stream, p);
        if (e != cudaSuccess) return llb_fail("decode attention: launch failed: %s", cudaGetErrorString(e));
        rc = llb_check_launch("paged_decode_mma");
        if (rc) return rc;
        if (p.nsplit > 1 && !cluster) {
            e = launch_pdl(decode_merge_kernel, dim3(num_tiles, p.Hq), dim3(32), 0, stream, p, HD);
            if (e != cudaSuccess) return llb_fail("decode merge: launch failed: %s", cudaGetErrorString(e));
            rc = llb_check_launch("decode_merge");
        }
        return rc;
    }
};

template <int HD>
int launch(const DecodeParams& p, int num_tiles, cudaStream_t stream) {
    return Launcher<HD, Shape<HD>::BK, Shape<HD>::NST>::launch(p, num_tiles, stream);
}
template <int HD>
int resident() {
    return Launcher<HD, Shape<HD>::BK, Shape<HD>::NST>::resident();
}

}  // namespace

// Whether this kernel takes the shape (else the CUDA-core kernel of attention_simt.cu is the one to call).
LLB_EXPORT int llb_paged_decode_mma_supports(int Hq, int Hkv, int hd) {
    return Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 16 && (hd == 64 || hd == 128);
}

// Blocks of the kernel that an SM holds at a time for this head size (what a planner divides by when it chooses the
// split count), or a negative code.
LLB_EXPORT int llb_paged_decode_mma_resident(int hd) {
    if (hd == 64) return resident<64>();
    if (hd == 128) return resident<128>();
    return llb_fail("decode attention: head size %d is not supported", hd);
}

// The largest split count that is merged inside the attention kernel, through a thread-block cluster.
LLB_EXPORT int llb_paged_decode_mma_cluster_splits() { return CLUSTER_MAX_SPLITS; }

// One query row per tile: q, out [T, Hq, hd] bf16 (row = span_row[tile_span[t]] + tile_q0[t], position
// span_pos + tile_q0); caches [slots, Hkv, hd] bf16; block_table [S, max_pages].  scratch: num_tiles * Hq *
// nsplit * (hd + 2) floats when nsplit > llb_paged_decode_mma_cluster_splits() (fewer splits merge inside the kernel).
LLB_EXPORT int llb_paged_decode_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                    const int* tile_span, const int* tile_q0, int num_tiles, const int* span_row,
                                    const int* span_pos, const int* block_table, int max_pages, int page_size,
                                    int Hq, int Hkv, int hd, int window, float scale, int nsplit, float* scratch,
                                    cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    LLB_REQUIRE(llb_paged_decode_mma_supports(Hq, Hkv, hd), "decode attention: %d/%d heads of size %d are not supported "
                "(groups of at most 16, head size 64 or 128)", Hq, Hkv, hd);
    LLB_REQUIRE(nsplit >= 1 && nsplit <= MERGE_MAX_SPLITS && (nsplit <= CLUSTER_MAX_SPLITS || scratch != nullptr),
                "decode attention: split count %d is outside 1..%d or scratch is missing", nsplit, MERGE_MAX_SPLITS);
    LLB_REQUIRE(page_size > 0 && max_pages > 0 && Hkv <= 65535, "decode attention: bad sizes");
    LLB_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0),
                "decode attention: tensors must be 16-byte aligned");
    DecodeParams p;
    p.q = (const __nv_bfloat16*)q; p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
    p.out = (__nv_bfloat16*)out; p.tile_span = tile_span; p.tile_q0 = tile_q0; p.span_row = span_row; p.span_pos = span_pos;
    p.block_table = block_table; p.max_pages = max_pages; p.page_size = page_size; p.Hq = Hq; p.Hkv = Hkv;
    p.window = window; p.nsplit = nsplit; p.scale_log2e = scale * 1.4426950408889634f;
    const int G = Hq / Hkv;
    p.part_acc = scratch;
    p.part_ml = scratch ? scratch + (size_t)num_tiles * Hkv * nsplit * G * hd : nullptr;
    if (hd == 64) return launch<64>(p, num_tiles, stream);
    return launch<128>(p, num_tiles, stream);
}
