// Paged attention over block tables on CUDA cores: any mix of spans (prompt portions of any
// length beside single decode tokens), causal by absolute position, optional window, any head
// size and group size.  All arithmetic is float; q, k, v may be float or bf16.
//
// Scores and softmax follow src/kv_cache/paged_attention.cu:153-163:
//     s = (q . k) * scale;  m' = max(m, s);  l = l*exp(m - m') + exp(s - m');
//     acc = acc*exp(m - m') + exp(s - m') * v;   out = acc / l
// with kv_head = q_head / (Hq / Hkv) (:115).  Differences from the reference: the running
// maximum starts at -inf and the result is exactly acc / l (the reference starts at -1e38 and
// divides by l + 1e-8, :130,169); a token's own key is visible (the reference's decode stops
// before it, src/engine/engine_server.cpp:1802); later portions of a prompt are causal too
// (engine_server.cpp:1755-1761 passes causal=false); the page size is a parameter (the
// reference fixes 16, paged_attention.cu:28).
//
// Work is cut into tiles of BQ query rows of one span; a block takes one tile and one kv head,
// i.e. BQ * G query vectors (G = Hq / Hkv) that share every key/value tile it stages in shared
// memory.  With nsplit > 1 the key range of a tile is cut into nsplit pieces whose partial
// (acc, m, l) go to scratch and are merged by a second kernel
// (as paged_attention.cu:323-460,476-532 does with a fixed 4 splits).
#include "common.cuh"

#include <math.h>

namespace {

constexpr int BK = 32;      // keys per staged tile = one per lane
constexpr int NWARPS = 4;

struct AttnParams {
    const void* q;
    const void* k_cache;
    const void* v_cache;
    void* out;
    const int* tile_span;
    const int* tile_q0;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* block_table;
    int max_pages, page_size, Hq, Hkv, hd, window, BQ, nsplit;
    float scale;
    float* part_acc;  // [tiles, Hkv, nsplit, BQ*G, hd]
    float* part_ml;   // [tiles, Hkv, nsplit, BQ*G, 2]
};

template <typename T>
__global__ void __launch_bounds__(NWARPS * 32) paged_attention_kernel(AttnParams p) {
    extern __shared__ float smem[];
    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = p.Hq / p.Hkv;
    const int hd = p.hd;
    const int nqv = p.BQ * G;
    const int kstride = hd | 1;
    float* Qs = smem;                       // [nqv][hd]
    float* Acc = Qs + (size_t)nqv * hd;     // [nqv][hd]
    float* Ms = Acc + (size_t)nqv * hd;     // [nqv]
    float* Ls = Ms + nqv;                   // [nqv]
    float* Ks = Ls + nqv;                   // [BK][kstride]
    float* Vs = Ks + BK * kstride;          // [BK][hd]
    float* Ps = Vs + BK * hd;               // [NWARPS][BK]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int span = p.tile_span[tile];
    const int q0 = p.tile_q0[tile];
    const int row0 = p.span_row[span] + q0;
    const int slen = p.span_len[span];
    const int pos0 = p.span_pos[span] + q0;        // position of the tile's first query
    const int nrows = min(p.BQ, slen - q0);        // valid query rows of this tile
    const int* bt = p.block_table + (size_t)span * p.max_pages;
    const T* q = (const T*)p.q;
    const T* kc = (const T*)p.k_cache;
    const T* vc = (const T*)p.v_cache;

    // Key range of the tile: [lo, hi); of this split: [klo, khi).
    const int hi = pos0 + nrows;
    int lo = 0;
    if (p.window > 0) lo = max(0, pos0 - p.window + 1);
    int klo = lo, khi = hi;
    if (p.nsplit > 1) {
        int chunk = (hi - lo + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + BK - 1) / BK) * BK;
        klo = lo + split * chunk;
        khi = min(hi, klo + chunk);
    }

    for (int i = threadIdx.x; i < nqv * hd; i += blockDim.x) {
        const int v = i / hd, d = i - v * hd;
        const int r = v / G, g = v - r * G;
        float val = 0.0f;
        if (r < nrows) val = llb_to_float(q[((size_t)(row0 + r) * p.Hq + kvh * G + g) * hd + d]);
        Qs[i] = val;
        Acc[i] = 0.0f;
    }
    for (int i = threadIdx.x; i < nqv; i += blockDim.x) {
        Ms[i] = -INFINITY;
        Ls[i] = 0.0f;
    }
    __syncthreads();

    for (int kb = klo; kb < khi; kb += BK) {
        // Stage BK keys and values of this kv head; rows past khi are zero.
        for (int j = warp; j < BK; j += NWARPS) {
            const int kpos = kb + j;
            if (kpos < khi) {
                const int page = bt[kpos / p.page_size];
                const size_t slot = (size_t)page * p.page_size + (kpos % p.page_size);
                const T* kr = kc + (slot * p.Hkv + kvh) * hd;
                const T* vr = vc + (slot * p.Hkv + kvh) * hd;
                for (int d = lane; d < hd; d += 32) {
                    Ks[j * kstride + d] = llb_to_float(kr[d]);
                    Vs[j * hd + d] = llb_to_float(vr[d]);
                }
            } else {
                for (int d = lane; d < hd; d += 32) {
                    Ks[j * kstride + d] = 0.0f;
                    Vs[j * hd + d] = 0.0f;
                }
            }
        }
        __syncthreads();

        const int kpos = kb + lane;
        for (int v = warp; v < nqv; v += NWARPS) {
            const int r = v / G;
            if (r >= nrows) continue;  // uniform over the warp
            const int qpos = pos0 + r;
            const bool visible = kpos < khi && kpos <= qpos && (p.window <= 0 || qpos - kpos < p.window);
            float s = -INFINITY;
            if (visible) {
                const float* qv = Qs + (size_t)v * hd;
                const float* kr = Ks + lane * kstride;
                float dot = 0.0f;
                for (int d = 0; d < hd; ++d) dot = fmaf(qv[d], kr[d], dot);
                s = dot * p.scale;
            }
            const float m_old = Ms[v];
            const float m_new = fmaxf(m_old, llb_warp_max(s));
            if (m_new == -INFINITY) continue;  // nothing visible yet; uniform over the warp
            const float pr = visible ? expf(s - m_new) : 0.0f;
            const float corr = (m_old == -INFINITY) ? 0.0f : expf(m_old - m_new);
            const float l_new = Ls[v] * corr + llb_warp_sum(pr);
            Ps[warp * BK + lane] = pr;
            __syncwarp();
            for (int d = lane; d < hd; d += 32) {
                float a = Acc[(size_t)v * hd + d] * corr;
#pragma unroll 8
                for (int j = 0; j < BK; ++j) a = fmaf(Ps[warp * BK + j], Vs[j * hd + d], a);
                Acc[(size_t)v * hd + d] = a;
            }
            __syncwarp();
            if (lane == 0) {
                Ms[v] = m_new;
                Ls[v] = l_new;
            }
            __syncwarp();
        }
        __syncthreads();
    }

    if (p.nsplit == 1) {
        T* out = (T*)p.out;
        for (int v = warp; v < nqv; v += NWARPS) {
            const int r = v / G, g = v - r * G;
            if (r >= nrows) continue;
            const float inv = 1.0f / Ls[v];
            T* o = out + ((size_t)(row0 + r) * p.Hq + kvh * G + g) * hd;
            for (int d = lane; d < hd; d += 32) o[d] = llb_from_float<T>(Acc[(size_t)v * hd + d] * inv);
        }
    } else {
        const size_t base = (((size_t)tile * p.Hkv + kvh) * p.nsplit + split) * nqv;
        for (int v = warp; v < nqv; v += NWARPS) {
            float* pa = p.part_acc + (base + v) * hd;
            for (int d = lane; d < hd; d += 32) pa[d] = Acc[(size_t)v * hd + d];
            if (lane == 0) {
                p.part_ml[(base + v) * 2 + 0] = Ms[v];
                p.part_ml[(base + v) * 2 + 1] = Ls[v];
            }
        }
    }
}

// Merge of the split partials: out = sum_s e^{m_s - M} acc_s / sum_s e^{m_s - M} l_s.
// One warp per (tile, head): the lanes first share the splits (weights w_s = e^{m_s - M} / L go to
// shared memory), then the output dimensions, reading every split's row with independent loads.
constexpr int MERGE_MAX_SPLITS = 256;
template <typename T>
__global__ void __launch_bounds__(32) attention_merge_kernel(AttnParams p) {
    __shared__ float wsm[MERGE_MAX_SPLITS];
    const int tile = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const int G = p.Hq / p.Hkv;
    const int kvh = head / G, g = head - kvh * G;
    const int nqv = p.BQ * G;
    const int span = p.tile_span[tile];
    const int q0 = p.tile_q0[tile];
    const int nrows = min(p.BQ, p.span_len[span] - q0);
    const int row0 = p.span_row[span] + q0;
    T* out = (T*)p.out;
    const size_t base0 = ((size_t)tile * p.Hkv + kvh) * p.nsplit;
    for (int r = 0; r < nrows; ++r) {
        const int v = r * G + g;
        float M = -INFINITY;
        for (int s = lane; s < p.nsplit; s += 32) M = fmaxf(M, p.part_ml[((base0 + s) * nqv + v) * 2]);
        M = llb_warp_max(M);
        float L = 0.0f;
        for (int s = lane; s < p.nsplit; s += 32) {
            const size_t idx = (base0 + s) * nqv + v;
            const float m = p.part_ml[idx * 2];
            const float w = (m == -INFINITY) ? 0.0f : expf(m - M);
            wsm[s] = w;
            L += w * p.part_ml[idx * 2 + 1];
        }
        L = llb_warp_sum(L);
        __syncwarp();
        const float inv = 1.0f / L;
        for (int d = lane; d < p.hd; d += 32) {
            float a = 0.0f;
#pragma unroll 8
            for (int s = 0; s < p.nsplit; ++s) a = fmaf(wsm[s], p.part_acc[((base0 + s) * nqv + v) * p.hd + d], a);
            out[((size_t)(row0 + r) * p.Hq + head) * p.hd + d] = llb_from_float<T>(a * inv);
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------
// Decode: one query row per tile (BQ == 1).  No block-wide barrier inside the key loop: each warp
// streams its own 32-key tiles of the split (lane = key for the scores, lane = pair of dimensions for
// the values), reads keys with 16-byte loads straight from the pages, and keeps (m, l, acc) of the
// G heads of the group in registers.  The four warps are merged through shared memory at the end.
// ---------------------------------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
    static __device__ __forceinline__ void load2(const float* p, float& a, float& b) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        a = v.x; b = v.y;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x; f[2 * i + 1] = t.y;
        }
    }
    static __device__ __forceinline__ void load2(const __nv_bfloat16* p, float& a, float& b) {
        const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
        a = t.x; b = t.y;
    }
};

template <typename T, int GMAX, int NPMAX>
__global__ void __launch_bounds__(NWARPS * 32) paged_decode_kernel(AttnParams p) {
    extern __shared__ float smem[];
    constexpr int VEC = Vec16<T>::N;
    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int G = p.Hq / p.Hkv;
    const int hd = p.hd;
    float* Qs = smem;                                   // [G][hd]
    float* Ps = Qs + G * hd;                            // [NWARPS][GMAX][32]
    float* Wacc = Ps + NWARPS * GMAX * 32;              // [NWARPS][G][hd]
    float* Wml = Wacc + NWARPS * G * hd;                // [NWARPS][G][2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int span = p.tile_span[tile];
    const int q0 = p.tile_q0[tile];
    const int row0 = p.span_row[span] + q0;
    const int qpos = p.span_pos[span] + q0;
    const int* bt = p.block_table + (size_t)span * p.max_pages;
    const T* q = (const T*)p.q;
    const T* kc = (const T*)p.k_cache;
    const T* vc = (const T*)p.v_cache;

    const int hi = qpos + 1;
    const int lo = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
    int klo = lo, khi = hi;
    if (p.nsplit > 1) {
        int chunk = (hi - lo + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + BK - 1) / BK) * BK;
        klo = lo + split * chunk;
        khi = min(hi, klo + chunk);
    }
    for (int i = threadIdx.x; i < G * hd; i += blockDim.x)
        Qs[i] = llb_to_float(q[((size_t)row0 * p.Hq + kvh * G) * hd + i]);
    __syncthreads();

    float m[GMAX], l[GMAX], acc[GMAX][NPMAX][2];
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int n = 0; n < NPMAX; ++n) acc[g][n][0] = acc[g][n][1] = 0.0f;
    }
    float* myP = Ps + warp * GMAX * 32;
    const size_t row_stride = (size_t)p.Hkv * hd;

    for (int kb = klo + warp * BK; kb < khi; kb += NWARPS * BK) {
        const int kpos = kb + lane;
        const bool valid = kpos < khi;
        const int nkeys = min(BK, khi - kb);
        size_t slot = 0;
        if (valid) slot = (size_t)bt[kpos / p.page_size] * p.page_size + (kpos % p.page_size);
        // Values first (NPMAX == 1: all 32 rows of the tile are requested before any arithmetic, so the
        // memory system sees them at once); each lane owns two dimensions of every row.
        float v0r[NPMAX == 1 ? BK : 1], v1r[NPMAX == 1 ? BK : 1];
        if (NPMAX == 1) {
            const int d = 2 * lane;
#pragma unroll
            for (int j = 0; j < BK; ++j) {
                const size_t sj = __shfl_sync(0xffffffffu, slot, j);
                v0r[j] = v1r[j] = 0.0f;
                if (j < nkeys && d < hd) Vec16<T>::load2(vc + sj * row_stride + (size_t)kvh * hd + d, v0r[j], v1r[j]);
            }
        }
        float dot[GMAX];
#pragma unroll
        for (int g = 0; g < GMAX; ++g) dot[g] = 0.0f;
        if (valid) {
            const T* kr = kc + slot * row_stride + (size_t)kvh * hd;
#pragma unroll 8
            for (int c = 0; c < hd; c += VEC) {
                float kf[VEC];
                Vec16<T>::load(kr + c, kf);
#pragma unroll
                for (int g = 0; g < GMAX; ++g) {
                    if (g < G) {
                        const float* qv = Qs + g * hd + c;
#pragma unroll
                        for (int e = 0; e < VEC; ++e) dot[g] = fmaf(qv[e], kf[e], dot[g]);
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            if (g < G) {
                const float sc = valid ? dot[g] * p.scale : -INFINITY;
                const float m_new = fmaxf(m[g], llb_warp_max(sc));      // finite: the tile has a valid key
                const float pr = valid ? expf(sc - m_new) : 0.0f;
                const float corr = (m[g] == -INFINITY) ? 0.0f : expf(m[g] - m_new);
                l[g] = l[g] * corr + llb_warp_sum(pr);
                m[g] = m_new;
                myP[g * 32 + lane] = pr;
#pragma unroll
                for (int n = 0; n < NPMAX; ++n) {
                    acc[g][n][0] *= corr;
                    acc[g][n][1] *= corr;
                }
            }
        }
        __syncwarp();
        if (NPMAX == 1) {
#pragma unroll
            for (int j = 0; j < BK; ++j) {
#pragma unroll
                for (int g = 0; g < GMAX; ++g) {
                    if (g < G) {
                        const float pj = myP[g * 32 + j];      // 0 for keys past the end
                        acc[g][0][0] = fmaf(pj, v0r[j], acc[g][0][0]);
                        acc[g][0][1] = fmaf(pj, v1r[j], acc[g][0][1]);
                    }
                }
            }
        } else {
#pragma unroll 8
            for (int j = 0; j < nkeys; ++j) {
                const size_t sj = __shfl_sync(0xffffffffu, slot, j);
                const T* vr = vc + sj * row_stride + (size_t)kvh * hd;
#pragma unroll
                for (int n = 0; n < NPMAX; ++n) {
                    const int d = n * 64 + 2 * lane;
                    if (d < hd) {
                        float v0, v1;
                        Vec16<T>::load2(vr + d, v0, v1);
#pragma unroll
                        for (int g = 0; g < GMAX; ++g) {
                            if (g < G) {
                                const float pj = myP[g * 32 + j];
                                acc[g][n][0] = fmaf(pj, v0, acc[g][n][0]);
                                acc[g][n][1] = fmaf(pj, v1, acc[g][n][1]);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    }

    // Merge the four warps.
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
        if (g < G) {
#pragma unroll
            for (int n = 0; n < NPMAX; ++n) {
                const int d = n * 64 + 2 * lane;
                if (d < hd) {
                    Wacc[(warp * G + g) * hd + d] = acc[g][n][0];
                    Wacc[(warp * G + g) * hd + d + 1] = acc[g][n][1];
                }
            }
            if (lane == 0) {
                Wml[(warp * G + g) * 2] = m[g];
                Wml[(warp * G + g) * 2 + 1] = l[g];
            }
        }
    }
    __syncthreads();
    const size_t base = (((size_t)tile * p.Hkv + kvh) * p.nsplit + split) * G;
    for (int i = threadIdx.x; i < G * hd; i += blockDim.x) {
        const int g = i / hd, d = i - g * hd;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, Wml[(w * G + g) * 2]);
        float L = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float mw = Wml[(w * G + g) * 2];
            if (mw != -INFINITY) {
                const float e = expf(mw - M);
                L += e * Wml[(w * G + g) * 2 + 1];
                a += e * Wacc[(w * G + g) * hd + d];
            }
        }
        if (p.nsplit == 1) {
            ((T*)p.out)[((size_t)row0 * p.Hq + kvh * G + g) * hd + d] = llb_from_float<T>(a / L);
        } else {
            p.part_acc[(base + g) * hd + d] = a;
            if (d == 0) {
                p.part_ml[(base + g) * 2] = M;
                p.part_ml[(base + g) * 2 + 1] = L;
            }
        }
    }
}

size_t decode_smem_bytes(int G, int gmax, int hd) {
    return ((size_t)G * hd + (size_t)NWARPS * gmax * 32 + (size_t)NWARPS * G * hd + (size_t)NWARPS * G * 2) * sizeof(float);
}

template <typename T, int GMAX>
int launch_decode_np(const AttnParams& p, dim3 grid, size_t smem, cudaStream_t stream) {
    if (p.hd <= 64) paged_decode_kernel<T, GMAX, 1><<<grid, NWARPS * 32, smem, stream>>>(p);
    else if (p.hd <= 128) paged_decode_kernel<T, GMAX, 2><<<grid, NWARPS * 32, smem, stream>>>(p);
    else paged_decode_kernel<T, GMAX, 4><<<grid, NWARPS * 32, smem, stream>>>(p);
    return llb_check_launch("paged_decode");
}

// Whether the decode kernel takes this shape; else the general kernel runs it.
template <typename T>
bool decode_eligible(const AttnParams& p) {
    const int G = p.Hq / p.Hkv;
    const int gmax = G <= 1 ? 1 : G <= 2 ? 2 : G <= 4 ? 4 : G <= 8 ? 8 : 16;
    return p.BQ == 1 && G <= 16 && p.hd <= 256 && p.hd % 2 == 0 && (p.hd * sizeof(T)) % 16 == 0 &&
           ((uintptr_t)p.k_cache % 16 == 0) && ((uintptr_t)p.v_cache % 16 == 0) &&
           decode_smem_bytes(G, gmax, p.hd) <= 48 * 1024;
}

template <typename T>
int launch_decode(const AttnParams& p, int num_tiles, cudaStream_t stream) {
    const int G = p.Hq / p.Hkv;
    dim3 grid(num_tiles, p.Hkv, p.nsplit);
    if (G <= 1) return launch_decode_np<T, 1>(p, grid, decode_smem_bytes(G, 1, p.hd), stream);
    if (G <= 2) return launch_decode_np<T, 2>(p, grid, decode_smem_bytes(G, 2, p.hd), stream);
    if (G <= 4) return launch_decode_np<T, 4>(p, grid, decode_smem_bytes(G, 4, p.hd), stream);
    if (G <= 8) return launch_decode_np<T, 8>(p, grid, decode_smem_bytes(G, 8, p.hd), stream);
    return launch_decode_np<T, 16>(p, grid, decode_smem_bytes(G, 16, p.hd), stream);
}

size_t attention_smem_bytes(int BQ, int G, int hd) {
    const size_t nqv = (size_t)BQ * G;
    const size_t floats = 2 * nqv * hd + 2 * nqv + (size_t)BK * (hd | 1) + (size_t)BK * hd + NWARPS * BK;
    return floats * sizeof(float);
}

template <typename T>
int launch_attention(const AttnParams& p, int num_tiles, cudaStream_t stream) {
    const size_t smem = attention_smem_bytes(p.BQ, p.Hq / p.Hkv, p.hd);
    LLB_REQUIRE(smem <= 220 * 1024, "attention: BQ=%d with %d heads per group and head_dim %d needs %zu bytes of "
                "shared memory; use a smaller BQ", p.BQ, p.Hq / p.Hkv, p.hd, smem);
    static size_t configured = 0;  // largest opt-in so far for this instantiation
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(paged_attention_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return llb_fail("attention: cannot opt in to %zu bytes of shared memory: %s", smem,
                                              cudaGetErrorString(e));
        configured = smem;
    }
    int rc;
    if (decode_eligible<T>(p)) {
        rc = launch_decode<T>(p, num_tiles, stream);
    } else {
        dim3 grid(num_tiles, p.Hkv, p.nsplit);
        paged_attention_kernel<T><<<grid, NWARPS * 32, smem, stream>>>(p);
        rc = llb_check_launch("paged_attention");
    }
    if (rc) return rc;
    if (p.nsplit > 1) {
        dim3 mgrid(num_tiles, p.Hq);
        attention_merge_kernel<T><<<mgrid, 32, 0, stream>>>(p);
        rc = llb_check_launch("attention_merge");
    }
    return rc;
}

}  // namespace

// Shared memory one block needs for the given tile height; the caller picks BQ with it.
LLB_EXPORT long long llb_attention_smem_bytes(int BQ, int group, int hd) {
    return (long long)attention_smem_bytes(BQ, group, hd);
}

// Floats of scratch that nsplit > 1 needs: acc and (m, l).
LLB_EXPORT long long llb_attention_scratch_floats(int num_tiles, int Hq, int hd, int BQ, int nsplit) {
    return (long long)num_tiles * Hq * BQ * nsplit * (hd + 2);
}

// q, out [T, Hq, hd]; k_cache, v_cache [slots, Hkv, hd] with slot = page*page_size + offset;
// tile_span, tile_q0 [num_tiles]; span_row, span_len, span_pos [S]; block_table [S, max_pages].
// window <= 0 means every earlier key is visible.  scratch: llb_attention_scratch_floats floats
// when nsplit > 1, else unused.
LLB_EXPORT int llb_paged_attention(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype,
                                   const int* tile_span, const int* tile_q0, int num_tiles, const int* span_row,
                                   const int* span_len, const int* span_pos, const int* block_table,
                                   int max_pages, int page_size, int Hq, int Hkv, int hd, int window, float scale,
                                   int BQ, int nsplit, float* scratch, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    LLB_REQUIRE(num_tiles > 0 && Hq > 0 && Hkv > 0 && hd > 0 && page_size > 0 && max_pages > 0 && BQ > 0,
                "attention: bad sizes");
    LLB_REQUIRE(Hq % Hkv == 0, "attention: %d query heads are not a multiple of %d kv heads", Hq, Hkv);
    LLB_REQUIRE(nsplit >= 1 && nsplit <= MERGE_MAX_SPLITS && Hkv <= 65535,
                "attention: split count %d is outside 1..%d", nsplit, MERGE_MAX_SPLITS);
    LLB_REQUIRE(nsplit == 1 || scratch != nullptr, "attention: nsplit=%d needs scratch", nsplit);
    AttnParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
    p.tile_span = tile_span; p.tile_q0 = tile_q0;
    p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.block_table = block_table;
    p.max_pages = max_pages; p.page_size = page_size; p.Hq = Hq; p.Hkv = Hkv; p.hd = hd;
    p.window = window; p.BQ = BQ; p.nsplit = nsplit; p.scale = scale;
    p.part_acc = scratch;
    p.part_ml = scratch ? scratch + (size_t)num_tiles * Hq * BQ * nsplit * hd : nullptr;
    if (dtype == LLB_F32) return launch_attention<float>(p, num_tiles, stream);
    if (dtype == LLB_BF16) return launch_attention<__nv_bfloat16>(p, num_tiles, stream);
    return llb_fail("attention: unknown dtype %d", dtype);
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that cannot allocate: the scratch of the splits lives in this
// file.  See attention_noalloc.h for who needs this, the size limit and the rules of use.
// ---------------------------------------------------------------------------------------------
#include "attention_noalloc.h"

// In device code this name is the array.  In host code it is only a handle for the runtime's
// symbol functions, never an address to hand to a kernel.
static __device__ __align__(256) float g_noalloc_scratch[LLB_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_scratch_addr[NOALLOC_MAX_DEVICES] = {};   // device address of the array, per device

// Once per device, with that device current: ask the runtime where the array lives on it.
int noalloc_scratch(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return llb_fail("attention_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return llb_fail("attention_noalloc: device index %d is out of range", dev);
    if (g_noalloc_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return llb_fail("attention_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        g_noalloc_scratch_addr[dev] = (float*)p;
    }
    *out = g_noalloc_scratch_addr[dev];
    return 0;
}
}  // namespace

LLB_EXPORT long long llb_noalloc_scratch_floats(void) { return LLB_NOALLOC_SCRATCH_FLOATS; }

LLB_EXPORT int llb_paged_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                           int dtype, const int* tile_span, const int* tile_q0, int num_tiles,
                                           const int* span_row, const int* span_len, const int* span_pos,
                                           const int* block_table, int max_pages, int page_size, int Hq, int Hkv,
                                           int hd, int window, float scale, int BQ, int nsplit, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    LLB_REQUIRE(num_tiles > 0 && Hq > 0 && hd > 0 && BQ > 0 && nsplit >= 1, "attention_noalloc: bad sizes");
    // Without splits nothing is written to the scratch: such a call has no size limit and needs no address.
    float* scratch = nullptr;
    if (nsplit > 1) {
        const long long need = llb_attention_scratch_floats(num_tiles, Hq, hd, BQ, nsplit);
        LLB_REQUIRE(need <= (long long)LLB_NOALLOC_SCRATCH_FLOATS,
                    "attention_noalloc: %d tiles x %d heads x %d rows x %d splits x (head_dim %d + 2) needs %lld floats of "
                    "scratch; the built-in scratch holds %lld. Use fewer splits or the entry point that takes scratch",
                    num_tiles, Hq, BQ, nsplit, hd, need, (long long)LLB_NOALLOC_SCRATCH_FLOATS);
        int rc = noalloc_scratch(&scratch);
        if (rc) return rc;
    }
    return llb_paged_attention(q, k_cache, v_cache, out, dtype, tile_span, tile_q0, num_tiles, span_row, span_len,
                               span_pos, block_table, max_pages, page_size, Hq, Hkv, hd, window, scale, BQ, nsplit,
                               scratch, stream);
}
