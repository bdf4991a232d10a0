// The layers of a step run from C++ (see step_executor.h): one call issues every kernel of the run entries it is given,
// with the choices that the Python parts make (parts/linear.py, parts/attention.py, parts/mlp.py, parts/block.py):
// which contraction kernel a shape takes and how K is cut, which projection path a step takes, which attention kernels
// the step's plan names.  The host then spends a few microseconds a launch instead of a Python call chain.
#include "step_executor.h"

#include <stdint.h>

#include "common.cuh"

// ---- entry points of the kernel library that the executor calls (defined in their own files) -----------------------
extern "C" {
int llb_paged_decode_mma_cluster_splits();
int llb_paged_decode_mma(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_span,
                         const int* tile_q0, int num_tiles, const int* span_row, const int* span_pos,
                         const int* block_table, int max_pages, int page_size, int Hq, int Hkv, int hd, int window,
                         float scale, int nsplit, float* scratch, cudaStream_t stream);
int llb_paged_decode_mma_supports(int Hq, int Hkv, int hd);
long long llb_attention_scratch_floats(int num_tiles, int Hq, int hd, int BQ, int nsplit);
int llb_paged_attention(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype, const int* tile_span,
                        const int* tile_q0, int num_tiles, const int* span_row, const int* span_len, const int* span_pos,
                        const int* block_table, int max_pages, int page_size, int Hq, int Hkv, int hd, int window,
                        float scale, int BQ, int nsplit, float* scratch, cudaStream_t stream);
int llb_paged_attention_tcgen05(const void* q, const void* k_cache, const void* v_cache, void* out, int T,
                                const int* tile_span, const int* tile_q0, int num_tiles, const int* span_row,
                                const int* span_len, const int* span_pos, const int* block_table, int max_pages,
                                int page_size, int num_slots, int Hq, int Hkv, int hd, int window, float scale,
                                const int* tile_k0, const int* tile_nk, const int* tile_part, float* part_scratch,
                                int num_parts, int* error_flag, cudaStream_t stream);
int llb_attention_tcgen05_merge(void* out, const int* merge_span, const int* merge_q0, const int* merge_first,
                                const int* merge_count, int num_merge, const int* span_row, const int* span_len,
                                const float* part_scratch, int num_parts, int Hq, int hd, cudaStream_t stream);
int llb_gemm_decode_supports(int M, int N, int K, int norm, int epilogue, int hd);
int llb_gemm_decode(const void* W, const void* a_bf16, const float* x, const int* x_rows, const void* norm_w, int norm_w_bf16,
                    float eps, int norm, const float* bias, void* out, float* residual, int epilogue, int M, int N, int K,
                    int split_k, const int* slot_mapping, const float* rope_table, int rotary_dim, int interleaved, int Hq,
                    int Hkv, int hd, void* q_out, void* k_cache, void* v_cache, float* acc_scratch, long long scratch_floats,
                    int* counters, int* error_flag, cudaStream_t stream);
int llb_gemm_simt(const void* A, int a_dtype, const void* W, const void* bias, int w_dtype, void* out, float* residual,
                  int epilogue, int M, int N, int K, cudaStream_t stream);
int llb_gemm_tcgen05(const void* A, const void* W, const float* bias, void* out, float* residual, int epilogue, int M, int N,
                     int K, int split_k, float* partials, int* counters, int* error_flag, cudaStream_t stream);
long long llb_gemm_tcgen05_partial_floats(int M, int N, int split_k);
long long llb_gemm_tcgen05_counters(int M, int N, int split_k);
int llb_gemm_tcgen05_rope(const void* A, const void* W, const float* bias, int M, int N, int K, const float* rope_table,
                          const int* slot_mapping, void* q_out, void* k_cache, void* v_cache, int Hq, int Hkv, int hd,
                          int* error_flag, cudaStream_t stream);
int llb_rmsnorm(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype, const int* rows, int R, int D,
                float eps, cudaStream_t stream);
int llb_rope_kv_write(const void* qkv, int dtype, const int* positions, const int* slot_mapping, const float* inv_freq,
                      int rotary_dim, int interleaved, void* q_out, void* k_cache, void* v_cache, int T, int Hq, int Hkv,
                      int hd, int write_kv, cudaStream_t stream);
int llb_rope_table(const int* positions, const float* inv_freq, float* table, int T, int half, int transposed,
                   cudaStream_t stream);
}

namespace {

// The thresholds of the Python parts (parts/linear.py, parts/attention.py); a test runs both paths side by side.
constexpr int DECODE_ROWS = 64;             // steps of at most this many rows use the fused decode contraction
constexpr int FUSED_ROPE_MAX_ROWS = 16;     // up to here the projection's decode kernel rotates and writes the cache itself
constexpr int PREFILL_ROPE_MIN_ROWS = 16;   // beyond, the tensor-core projection does (heads of 64 or 128)
constexpr int DEPI_STORE_F32 = 1, DEPI_RESIDUAL = 2, DEPI_SWIGLU = 3, DEPI_ROPE_KV = 4;

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int imin(int a, int b) { return a < b ? a : b; }
inline int imax(int a, int b) { return a > b ? a : b; }

struct Exec {
    const LlbModelDesc& m;
    const LlbStepArgs& s;
    bool dry;                 // only count the workspace
    uint8_t* base;
    long long used = 0, peak = 0;
    int es;                   // bytes of an activation element
    bool bf16;
    // the rotary tables made for this step: by frequencies and orientation (token-major for the decode contraction,
    // pair-major for the tensor-core one)
    struct Table { int freqs; int transposed; float* data; };
    Table tables[8];
    int num_tables = 0;

    Exec(const LlbModelDesc& model, const LlbStepArgs& step, bool dry_)
        : m(model), s(step), dry(dry_), base((uint8_t*)step.workspace), es(model.act_dtype == LLB_BF16 ? 2 : 4),
          bf16(model.act_dtype == LLB_BF16) {}

    void* take(long long bytes) {
        bytes = (bytes + 255) & ~255ll;
        void* p = dry ? nullptr : (void*)(base + used);
        used += bytes;
        if (used > peak) peak = used;
        return p;
    }

    // ---- parts/linear.py ------------------------------------------------------------------------------------------
    int split_k_for(int N, int K) const { return imax(1, imin(ceil_div(K, 64), m.num_sms / ceil_div(N, 128))); }
    int split_k_fused(int M, int N, int K) const {
        const int tiles = ceil_div(N, 128);
        if (M > 16 || tiles * 4 > m.num_sms) return 1;
        return imax(1, imin(ceil_div(K, 64), m.num_sms / tiles));
    }
    int split_k_wide(int M, int N, int K) const {
        const int tiles = ceil_div(M, 128) * ceil_div(N, N > 128 ? 256 : 128);
        if (tiles * 2 > m.num_sms) return 1;
        return imax(1, imin(m.num_sms / tiles, ceil_div(K, 64) / 16));
    }
    bool decode_eligible(int M, int N, int K, int depi, int hd) const {
        return M <= DECODE_ROWS && bf16 && llb_gemm_decode_supports(M, N, K, 0, depi, hd);
    }
    float* splitk_for(int N, int split, int depi) const {      // the meeting place of a split fused epilogue, if it is large enough
        if (split > 1 && (depi == DEPI_SWIGLU || depi == DEPI_ROPE_KV) && s.splitk_scratch && s.splitk_tiles >= ceil_div(N, 128))
            return s.splitk_scratch;
        return nullptr;
    }

    // out = x W^T (+ bias) with the epilogue; x [M, K] in the activation dtype
    int linear(const void* x, const void* w, const float* bias, int epi, void* out, float* residual, int M, int N, int K) {
        const int depi = epi == LLB_EPI_STORE_F32 ? DEPI_STORE_F32 : epi == LLB_EPI_RESIDUAL ? DEPI_RESIDUAL
                         : epi == LLB_EPI_SWIGLU ? DEPI_SWIGLU : 0;
        if (depi && decode_eligible(M, N, K, depi, 0)) {
            int split = 1;
            if (epi == LLB_EPI_RESIDUAL) split = split_k_for(N, K);
            else if (epi == LLB_EPI_SWIGLU) split = split_k_fused(M, N, K);
            float* sc = splitk_for(N, split, depi);
            if (dry) return 0;
            return llb_gemm_decode(w, x, nullptr, nullptr, nullptr, 0, 0.0f, 0, bias, out, residual, depi, M, N, K, split, nullptr,
                                   nullptr, 0, 0, 0, 0, 0, nullptr, nullptr, nullptr, sc, sc ? s.splitk_floats : 0,
                                   sc ? s.splitk_counters : nullptr, s.error_flag, s.stream);
        }
        if (bf16 && K % 8 == 0) {
            int split = M > 128 ? split_k_wide(M, N, K) : (epi == LLB_EPI_RESIDUAL ? split_k_for(N, K) : 1);
            float* partials = nullptr;
            int* counters = nullptr;
            const long long mark = used;
            if (split > 1 && M > 128) {
                if (!s.meet_counters || llb_gemm_tcgen05_counters(M, N, split) > s.meet_counters_n) {
                    split = 1;
                } else {
                    counters = s.meet_counters;
                    partials = (float*)take(llb_gemm_tcgen05_partial_floats(M, N, split) * 4);
                }
            }
            int rc = 0;
            if (!dry) rc = llb_gemm_tcgen05(x, w, bias, out, residual, epi, M, N, K, split, partials, counters, s.error_flag, s.stream);
            used = mark;       // the kernels of the stream run in order: the next one may reuse the partials
            return rc;
        }
        if (dry) return 0;
        return llb_gemm_simt(x, m.act_dtype, w, bias, m.act_dtype, out, residual, epi, M, N, K, s.stream);
    }

    // ---- the step's rotary tables (parts/rotary.py: once per step and set of frequencies) ----------------------------------
    int ensure_table(const LlbAttentionDesc& a, bool transposed) {
        for (int i = 0; i < num_tables; ++i)
            if (tables[i].freqs == a.freqs && tables[i].transposed == (int)transposed) return 0;
        if (num_tables == 8) return llb_fail("step: more than 8 different rotary tables in one step");
        float* data = (float*)take((long long)s.T * a.rotary_dim * 4);
        tables[num_tables++] = Table{a.freqs, (int)transposed, data};
        if (dry) return 0;
        return llb_rope_table(s.positions, a.inv_freq, data, s.T, a.rotary_dim / 2, transposed ? 1 : 0, s.stream);
    }
    const float* table_of(const LlbAttentionDesc& a, bool transposed) const {
        for (int i = 0; i < num_tables; ++i)
            if (tables[i].freqs == a.freqs && tables[i].transposed == (int)transposed) return tables[i].data;
        return nullptr;
    }
    // Which way the projection of this layer goes (AttentionMixer.forward): 1 the decode contraction with rotation and
    // cache write in its epilogue, 2 the tensor-core contraction with them, 3 contraction and rotation apart.
    int projection_path(const LlbAttentionDesc& a) const {
        const int hd = a.head_dim, N = (a.num_heads + (a.writes ? 2 * a.num_kv_heads : 0)) * hd;
        const bool rotary = a.inv_freq != nullptr;
        if (rotary && bf16 && s.T <= FUSED_ROPE_MAX_ROWS && decode_eligible(s.T, N, m.hidden, DEPI_ROPE_KV, hd)) return 1;
        if (rotary && bf16 && s.T > PREFILL_ROPE_MIN_ROWS && a.writes && (hd == 64 || hd == 128) && m.hidden % 8 == 0 &&
            a.rotary_dim == hd && !a.interleaved)
            return 2;
        return 3;
    }

    // ---- parts/attention.py ---------------------------------------------------------------------------------------
    int attention(const LlbAttentionDesc& a, const void* x, float* residual) {
        const int T = s.T, D = m.hidden, hq = a.num_heads, hkv = a.num_kv_heads, hd = a.head_dim;
        const int Nq = hq * hd, Nqkv = (hq + 2 * hkv) * hd;
        const int N = a.writes ? Nqkv : Nq;                 // an entry that reads another's keys projects q only
        const int* slots = a.writes ? s.slot_mapping[a.group] : nullptr;
        void* kc = a.writes ? a.k_cache : nullptr;
        void* vc = a.writes ? a.v_cache : nullptr;
        void* q = take((long long)T * Nq * es);
        int rc = 0;
        const int path = projection_path(a);
        if (path == 1) {
            // few rows: projection, bias, rotation and cache write in the decode contraction
            const int split = split_k_fused(T, N, D);
            float* sc = splitk_for(N, split, DEPI_ROPE_KV);
            if (!dry)
                rc = llb_gemm_decode(a.w_qkv, x, nullptr, nullptr, nullptr, 0, 0.0f, 0, a.b_qkv, nullptr, nullptr, DEPI_ROPE_KV, T, N, D,
                                     split, slots, a.rotary_dim ? table_of(a, false) : nullptr, a.rotary_dim, a.interleaved, hq, hkv,
                                     hd, q, kc, vc, sc, sc ? s.splitk_floats : 0, sc ? s.splitk_counters : nullptr, s.error_flag,
                                     s.stream);
        } else if (path == 2) {
            // a long portion: the same in the epilogue of the tensor-core contraction
            if (!dry)
                rc = llb_gemm_tcgen05_rope(x, a.w_qkv, a.b_qkv, T, Nqkv, D, table_of(a, true), slots, q, kc, vc, hq, hkv, hd,
                                           s.error_flag, s.stream);
        } else {
            void* qkv = take((long long)T * N * es);
            rc = linear(x, a.w_qkv, a.b_qkv, LLB_EPI_STORE, qkv, nullptr, T, N, D);
            if (rc == 0 && !dry)
                rc = llb_rope_kv_write(qkv, m.act_dtype, s.positions, slots, a.inv_freq, a.rotary_dim, a.interleaved, q, kc, vc, T, hq,
                                       a.writes ? hkv : 0, hd, a.writes ? 1 : 0, s.stream);
        }
        if (rc) return rc;
        void* out = take((long long)T * Nq * es);
        if ((rc = attend(a, q, out))) return rc;
        return linear(out, a.w_o, a.b_o, LLB_EPI_RESIDUAL, nullptr, residual, T, D, Nq);
    }

    int simt(const LlbAttentionDesc& a, const void* q, void* out, const LlbTileList& t) {
        float* scratch = nullptr;
        if (t.nsplit > 1) scratch = (float*)take(llb_attention_scratch_floats(t.count, a.num_heads, a.head_dim, t.bq, t.nsplit) * 4);
        if (dry) return 0;
        return llb_paged_attention(q, a.k_cache, a.v_cache, out, m.act_dtype, t.span, t.q0, t.count, s.span_row, s.span_len,
                                   s.span_pos, s.block_tables[a.group], s.max_pages, s.page_size, a.num_heads, a.num_kv_heads,
                                   a.head_dim, a.window, a.scale, t.bq, t.nsplit, scratch, s.stream);
    }
    int decode_mma(const LlbAttentionDesc& a, const void* q, void* out, const LlbTileList& t, bool may_scratch) {
        float* scratch = nullptr;
        if (may_scratch && t.nsplit > llb_paged_decode_mma_cluster_splits())
            scratch = (float*)take(llb_attention_scratch_floats(t.count, a.num_heads, a.head_dim, 1, t.nsplit) * 4);
        if (dry) return 0;
        return llb_paged_decode_mma(q, a.k_cache, a.v_cache, out, t.span, t.q0, t.count, s.span_row, s.span_pos,
                                    s.block_tables[a.group], s.max_pages, s.page_size, a.num_heads, a.num_kv_heads, a.head_dim,
                                    a.window, a.scale, t.nsplit, scratch, s.stream);
    }
    int attend(const LlbAttentionDesc& a, const void* q, void* out) {
        const LlbAttentionPlan& p = s.plans[a.plan];
        if (p.kind == 0) return decode_mma(a, q, out, p.decode, true);
        if (p.kind == 1) return simt(a, q, out, p.decode);
        int rc = 0;
        if (p.items.count > 0) {
            float* parts = nullptr;
            if (p.num_parts > 0) parts = (float*)take((long long)p.num_parts * a.num_heads * 128 * (a.head_dim + 2) * 4);
            if (!dry) {
                rc = llb_paged_attention_tcgen05(q, a.k_cache, a.v_cache, out, s.T, p.items.span, p.items.q0, p.items.count,
                                                 s.span_row, s.span_len, s.span_pos, s.block_tables[a.group], s.max_pages,
                                                 s.page_size, (int)a.num_slots, a.num_heads, a.num_kv_heads, a.head_dim, a.window,
                                                 a.scale, p.item_k0, p.item_nk, p.item_part, parts, p.num_parts, s.error_flag,
                                                 s.stream);
                if (rc == 0 && p.num_parts > 0)
                    rc = llb_attention_tcgen05_merge(out, p.merge_span, p.merge_q0, p.merge_first, p.merge_count, p.num_merge,
                                                     s.span_row, s.span_len, parts, p.num_parts, a.num_heads, a.head_dim, s.stream);
            }
            if (rc) return rc;
        }
        if (p.decode.count > 0 && (rc = decode_mma(a, q, out, p.decode, false))) return rc;
        for (int i = 0; i < p.num_simt; ++i)
            if ((rc = simt(a, q, out, p.simt[i]))) return rc;
        return 0;
    }

    // ---- parts/block.py, parts/mlp.py: the run entries -------------------------------------------------------------
    int norm(const LlbNormDesc& n, const float* residual, void* out) {
        if (dry) return 0;
        return llb_rmsnorm(residual, LLB_F32, n.weight, n.weight_dtype, out, m.act_dtype, nullptr, s.T, m.hidden, n.eps, s.stream);
    }
    int run() {
        const int T = s.T, D = m.hidden;
        int rc;
        // the rotary tables that the layers of this call read, before anything else takes workspace
        for (int l = s.first_layer; l < s.last_layer; ++l) {
            const LlbAttentionDesc& a = m.layers[l].attn;
            if (a.plan < 0 || a.plan >= s.num_plans) return llb_fail("step: layer %d names plan %d of %d", l, a.plan, s.num_plans);
            if (a.group < 0 || a.group >= LLB_STEP_MAX_GROUPS) return llb_fail("step: layer %d names cache group %d", l, a.group);
            const int path = projection_path(a);
            if (path == 1 && a.rotary_dim && (rc = ensure_table(a, false))) return rc;
            if (path == 2 && (rc = ensure_table(a, true))) return rc;
        }
        const long long mark = used;
        for (int l = s.first_layer; l < s.last_layer; ++l) {
            const LlbLayerDesc& L = m.layers[l];
            used = mark;            // a layer's activations take the place of the layer before's
            void* x = take((long long)T * D * es);
            if ((rc = norm(L.norm1, s.residual, x))) return rc;
            if ((rc = attention(L.attn, x, s.residual))) return rc;
            used = mark;
            x = take((long long)T * D * es);
            if ((rc = norm(L.norm2, s.residual, x))) return rc;
            void* act = take((long long)T * L.mlp.intermediate * es);
            if ((rc = linear(x, L.mlp.w_gate_up, L.mlp.b_gate_up, LLB_EPI_SWIGLU, act, nullptr, T, 2 * L.mlp.intermediate, D))) return rc;
            if ((rc = linear(act, L.mlp.w_down, L.mlp.b_down, LLB_EPI_RESIDUAL, nullptr, s.residual, T, D, L.mlp.intermediate))) return rc;
            if (!dry && peak > s.workspace_bytes) return llb_fail("step: the workspace of %lld bytes is too small", s.workspace_bytes);
        }
        return 0;
    }
};

int check(const LlbModelDesc* model, const LlbStepArgs* step) {
    LLB_REQUIRE(model && step && model->layers, "step: null descriptor");
    LLB_REQUIRE(step->T > 0 && step->S > 0 && step->first_layer >= 0 && step->first_layer <= step->last_layer &&
                step->last_layer <= model->num_layers, "step: bad counts (T=%d, S=%d, layers %d..%d of %d)", step->T, step->S,
                step->first_layer, step->last_layer, model->num_layers);
    LLB_REQUIRE(model->act_dtype == LLB_F32 || model->act_dtype == LLB_BF16, "step: unknown dtype %d", model->act_dtype);
    return 0;
}

}  // namespace

LLB_EXPORT long long llb_step_workspace_need(const LlbModelDesc* model, const LlbStepArgs* step) {
    if (check(model, step)) return -1;
    Exec e(*model, *step, true);
    if (e.run()) return -1;
    return e.peak;
}

LLB_EXPORT int llb_step_layers(const LlbModelDesc* model, const LlbStepArgs* step) {
    int rc = check(model, step);
    if (rc) return rc;
    LLB_REQUIRE(step->residual && step->workspace && step->plans, "step: null buffer");
    {
        Exec need(*model, *step, true);
        if ((rc = need.run())) return rc;
        LLB_REQUIRE(need.peak <= step->workspace_bytes, "step: the workspace has %lld bytes, the step needs %lld",
                    step->workspace_bytes, need.peak);
    }
    Exec e(*model, *step, false);
    return e.run();
}

namespace {
int head(Exec& e, const LlbNormDesc* norm, const void* head_w, int vocab, const int* rows, int R, float* logits) {
    void* x = e.take((long long)R * e.m.hidden * e.es);
    int rc = 0;
    if (!e.dry)
        rc = llb_rmsnorm(e.s.residual, LLB_F32, norm->weight, norm->weight_dtype, x, e.m.act_dtype, rows, R, e.m.hidden, norm->eps,
                         e.s.stream);
    if (rc) return rc;
    return e.linear(x, head_w, nullptr, LLB_EPI_STORE_F32, logits, nullptr, R, vocab, e.m.hidden);
}
}  // namespace

LLB_EXPORT long long llb_step_head_workspace_need(const LlbModelDesc* model, const LlbStepArgs* step, int vocab, int R) {
    if (!model || !step || R < 0 || vocab <= 0) return -1;
    if (R == 0) return 0;
    Exec e(*model, *step, true);
    if (head(e, nullptr, nullptr, vocab, nullptr, R, nullptr)) return -1;
    return e.peak;
}

LLB_EXPORT int llb_step_head(const LlbModelDesc* model, const LlbStepArgs* step, const LlbNormDesc* norm, const void* head_w,
                             int vocab, const int* rows, int R, float* logits) {
    if (R == 0) return 0;
    LLB_REQUIRE(model && step && norm && head_w && rows && logits && step->residual && step->workspace, "head: null argument");
    LLB_REQUIRE(R > 0 && vocab > 0, "head: bad sizes (R=%d, vocab=%d)", R, vocab);
    LLB_REQUIRE(model->act_dtype == LLB_F32 || model->act_dtype == LLB_BF16, "head: unknown dtype %d", model->act_dtype);
    const long long need = llb_step_head_workspace_need(model, step, vocab, R);
    LLB_REQUIRE(need >= 0 && need <= step->workspace_bytes, "head: the workspace has %lld bytes, %d rows need %lld",
                step->workspace_bytes, R, need);
    Exec e(*model, *step, false);
    return head(e, norm, head_w, vocab, rows, R, logits);
}

LLB_EXPORT void llb_step_struct_sizes(int* out) {
    out[0] = (int)sizeof(LlbNormDesc);
    out[1] = (int)sizeof(LlbAttentionDesc);
    out[2] = (int)sizeof(LlbMlpDesc);
    out[3] = (int)sizeof(LlbLayerDesc);
    out[4] = (int)sizeof(LlbModelDesc);
    out[5] = (int)sizeof(LlbTileList);
    out[6] = (int)sizeof(LlbAttentionPlan);
    out[7] = (int)sizeof(LlbStepArgs);
}
