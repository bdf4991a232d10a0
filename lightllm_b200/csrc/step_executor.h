// The layers of a step, run from C++: what the Python parts do launch by launch (norm, q/k/v projection with position
// encoding and cache write, attention, output projection, norm, gated feed-forward), with the same choices of kernel,
// for a model whose layers are all of that common kind.  The reference's engine runs its layer loop in C++ as well
// (src/engine/engine_server.cpp:1530-1880); here the loop is data-driven: the model is an array of layer records that
// the Python model fills when it is bound, and a step is a record of the step's metadata and of the attention plans
// that the Python parts made for it.  Python mirrors these structs with ctypes (engine/native_step.py);
// llb_step_struct_sizes lets it check that the two sides agree.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLB_STEP_MAX_GROUPS 4      // cache groups a step can carry block tables for

typedef struct {
    const void* weight;            // [hidden]
    int weight_dtype;              // LLB_F32 / LLB_BF16
    float eps;
} LlbNormDesc;

typedef struct {
    const void* w_qkv;             // [(Hq + 2 Hkv) * hd, hidden], q rows first
    const float* b_qkv;            // [(Hq + 2 Hkv) * hd] or null
    const void* w_o;               // [hidden, Hq * hd]
    const float* b_o;              // [hidden] or null
    void* k_cache;                 // this run entry's planes: [slots, Hkv, hd]
    void* v_cache;
    const float* inv_freq;         // [rotary_dim / 2] or null (no rotation)
    long long num_slots;
    int writes;                    // this entry writes its keys and values (else it reads another entry's)
    int group;                     // cache group: which block table and slot mapping of the step
    int num_heads, num_kv_heads, head_dim, window;
    float scale;
    int rotary_dim, interleaved;
    int plan;                      // which of the step's attention plans this layer uses
    int freqs;                     // which set of rotary frequencies inv_freq is (layers with equal values share a number
                                   // and so the step's table)
    int pad_;
} LlbAttentionDesc;

typedef struct {
    const void* w_gate_up;         // [2 I, hidden], gate and up rows interleaved
    const float* b_gate_up;        // [2 I] or null
    const void* w_down;            // [hidden, I]
    const float* b_down;           // [hidden] or null
    int intermediate;
    int pad_;
} LlbMlpDesc;

typedef struct {
    LlbNormDesc norm1;
    LlbAttentionDesc attn;
    LlbNormDesc norm2;
    LlbMlpDesc mlp;
} LlbLayerDesc;

typedef struct {
    const LlbLayerDesc* layers;    // one per run entry
    int num_layers;
    int hidden;
    int act_dtype;                 // LLB_F32 / LLB_BF16: activations, weights and cache
    int num_sms;
} LlbModelDesc;

// One list of tiles of query rows: (span, first row) each.
typedef struct {
    const int* span;
    const int* q0;
    int count;
    int bq;                        // rows per tile (CUDA-core kernel)
    int nsplit;                    // pieces along the keys
    int pad_;
} LlbTileList;

// What the attention part decided for this step (AttentionMixer._plan).
typedef struct {
    int kind;                      // 0: all rows on the decode kernel, 1: all on the CUDA-core kernel, 2: mixed
    int num_simt;
    LlbTileList decode;            // kind 0 / 1: every request's row; kind 2: the single tokens (count 0: none)
    LlbTileList items;             // kind 2: items of the tensor-core kernel (count 0: none)
    const int* item_k0;            // cut of the items' key ranges (null: not cut)
    const int* item_nk;
    const int* item_part;
    const int* merge_span;
    const int* merge_q0;
    const int* merge_first;
    const int* merge_count;
    int num_parts, num_merge;
    LlbTileList simt[2];           // kind 2: what the CUDA-core kernel takes
} LlbAttentionPlan;

typedef struct {
    const int* token_ids;
    const int* positions;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* block_tables[LLB_STEP_MAX_GROUPS];
    const int* slot_mapping[LLB_STEP_MAX_GROUPS];
    float* residual;               // [T, hidden]: the stream the layers add into
    void* workspace;               // activations, tables and scratch of the step
    long long workspace_bytes;
    const LlbAttentionPlan* plans;
    float* splitk_scratch;         // the zeroed meeting place of the fused decode contractions (or null)
    long long splitk_floats;
    int* splitk_counters;
    int* meet_counters;            // the zeroed counters of wide split contractions (or null)
    int* error_flag;               // raised by kernels whose waits ran out
    cudaStream_t stream;
    int splitk_tiles, meet_counters_n;
    int T, S;
    int max_pages, page_size;
    int num_plans;
    int first_layer, last_layer;   // run entries [first, last)
    int pad_;
} LlbStepArgs;

// Runs the run entries [first_layer, last_layer) over the step.  0, or a negative code with llb_last_error().
int llb_step_layers(const LlbModelDesc* model, const LlbStepArgs* step);
// Bytes of workspace that this step needs (what llb_step_layers would carve out of step->workspace).
long long llb_step_workspace_need(const LlbModelDesc* model, const LlbStepArgs* step);
// The model's head over chosen rows of the stream: the norm of rows `rows` [R] of step->residual, then the contraction
// with head_w [vocab, hidden] into logits [R, vocab] (float), with the kernels that llb_step_layers would choose for a
// contraction of that shape.  It takes its activations from step->workspace (llb_step_head_workspace_need).
int llb_step_head(const LlbModelDesc* model, const LlbStepArgs* step, const LlbNormDesc* norm, const void* head_w, int vocab,
                  const int* rows, int R, float* logits);
long long llb_step_head_workspace_need(const LlbModelDesc* model, const LlbStepArgs* step, int vocab, int R);
// sizeof of the six structs above, in their order, for the binding to compare with its own.
void llb_step_struct_sizes(int* out);

#ifdef __cplusplus
}
#endif
