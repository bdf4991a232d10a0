// generate <model_dir> [token ids ... [/ token ids ...]]: the continuation of one or several prompts, from C++ alone.
//
// The reference's command lines are C++ programs over its engine (tests/test_generate.cpp:148-149,284-290: the prompt
// 576 8319 315 13466 374, 12 new tokens, temperature 0.8, top-k 40, top-p 0.9; tools/bench_server.cpp:158-245).  This
// one is the same over this engine's kernel library: it reads config.json and model.safetensors, lays the weights out
// as the library's step executor wants them (q/k/v rows in one matrix, gate and up rows interleaved), keeps keys and
// values in pages with a block table per request, and runs steps of (prompt portions under a token budget beside one
// token of every decoding request) through llb_embedding, llb_step_layers, llb_step_head and the samplers.  No Python,
// no torch.  It takes what the step executor takes on its tensor-core paths: bfloat16 weights, one cache group (no
// layer with a window), heads that the attention kernels support; anything else it refuses with a message that names
// the Python entry point, which runs every configuration.
//
// Options (names and defaults of python -m lightllm_b200.cli.generate): --max-new-tokens 12, --temperature 0.8,
// --top-k 40, --top-p 0.9, --min-p 0, --seed 42, --eos-token-id (default: config.json's), --max-seq-len 2048,
// --max-batch-tokens 2048; --timing prints times, --no-graphs issues every step launch by launch.  Temperature 0 is greedy.  Sampling draws its uniforms from a generator of its own
// (splitmix64 of seed, request and step), so sampled tokens repeat for a seed but are not the Python entry point's.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "../step_executor.h"
#include "json.h"

extern "C" {
int llb_abi_version();
const char* llb_last_error();
int llb_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int D, int V, int* err, cudaStream_t stream);
int llb_step_head(const LlbModelDesc* model, const LlbStepArgs* step, const LlbNormDesc* norm, const void* head_w, int vocab,
                  const int* rows, int R, float* logits);
long long llb_step_head_workspace_need(const LlbModelDesc* model, const LlbStepArgs* step, int vocab, int R);
int llb_argmax(const float* logits, int R, int V, long long stride, int* out, int* scratch, int scratch_rows, cudaStream_t stream);
int llb_sample(const float* logits, int R, int V, long long stride, const float* temperature, const int* top_k, const float* top_p,
               const float* min_p, const float* uniform, int* out, cudaStream_t stream);
int llb_paged_decode_mma_supports(int Hq, int Hkv, int hd);
int llb_paged_decode_mma_cluster_splits();
int llb_paged_decode_mma_resident(int hd);
int llb_attention_tcgen05_supports(int hd, int page_size);
}

namespace {

constexpr int F32 = 0, BF16 = 1;                 // the library's dtype codes
constexpr int PAGE = 16;                         // tokens of a cache page
constexpr int EXPECTED_ABI = 21;
constexpr int DECODE_ROWS = 64;                  // rows that the fused decode contractions take (their meeting place is sized for it)
constexpr int CLUSTER_MERGE_MAX_KEYS = 8192;     // up to here the decode attention merges its pieces inside a cluster

[[noreturn]] void die(const std::string& what) {
    std::fprintf(stderr, "generate: %s\n", what.c_str());
    std::exit(1);
}
void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) die(std::string(what) + ": " + cudaGetErrorString(e));
}
void lib_ok(int rc, const char* what) {
    if (rc != 0) die(std::string(what) + ": " + llb_last_error());
}
inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---- files ----------------------------------------------------------------------------------------------------------
struct MappedFile {
    const uint8_t* data = nullptr;
    size_t size = 0;
    explicit MappedFile(const std::string& path) {
        const int fd = ::open(path.c_str(), O_RDONLY);
        if (fd < 0) die(path + ": cannot be opened");
        struct stat st;
        if (fstat(fd, &st) != 0 || st.st_size <= 0) die(path + ": cannot be read");
        size = (size_t)st.st_size;
        void* p = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        ::close(fd);
        if (p == MAP_FAILED) die(path + ": cannot be mapped");
        data = (const uint8_t*)p;
    }
    ~MappedFile() { if (data) munmap((void*)data, size); }
    MappedFile(const MappedFile&) = delete;
};

struct Tensor {
    std::string dtype;
    std::vector<long long> shape;
    const uint8_t* data = nullptr;
    size_t bytes = 0;
    long long numel() const { long long n = 1; for (long long d : shape) n *= d; return n; }
};

// model.safetensors: 8 bytes of header length, a JSON header {name: {dtype, shape, data_offsets}}, then the data.
struct SafeTensors {
    MappedFile file;
    std::map<std::string, Tensor> tensors;
    std::set<std::string> used;
    explicit SafeTensors(const std::string& path) : file(path) {
        if (file.size < 8) die(path + ": too short for a safetensors file");
        uint64_t n = 0;
        std::memcpy(&n, file.data, 8);
        if (n > file.size - 8) die(path + ": the header is longer than the file");
        llb::Json head;
        try {
            head = llb::JsonParser((const char*)file.data + 8, (size_t)n, path).parse();
        } catch (const std::exception& e) { die(e.what()); }
        if (head.kind != llb::Json::Object) die(path + ": the header is not an object");
        const uint8_t* base = file.data + 8 + n;
        const size_t room = file.size - 8 - (size_t)n;
        for (const auto& m : head.members) {
            if (m.first == "__metadata__") continue;
            const llb::Json *dt = m.second.find("dtype"), *sh = m.second.find("shape"), *off = m.second.find("data_offsets");
            if (!dt || dt->kind != llb::Json::String || !sh || sh->kind != llb::Json::Array || !off || off->kind != llb::Json::Array ||
                off->items.size() != 2)
                die(path + ": bad entry for tensor '" + m.first + "'");
            Tensor t;
            t.dtype = dt->text;
            for (const auto& d : sh->items) t.shape.push_back((long long)d.number);
            const size_t b = (size_t)off->items[0].number, e = (size_t)off->items[1].number;
            const size_t es = t.dtype == "BF16" || t.dtype == "F16" ? 2 : t.dtype == "F32" || t.dtype == "I32" ? 4 : 0;
            if (b > e || e > room || (es && (e - b) != (size_t)t.numel() * es))
                die(path + ": tensor '" + m.first + "' has offsets that do not fit its shape or the file");
            t.data = base + b;
            t.bytes = e - b;
            tensors.emplace(m.first, std::move(t));
        }
    }
};

// ---- configuration: the keys of Qwen2ForCausalLM's config.json ----------------------------------------------------
struct Config {
    int vocab = 0, hidden = 0, intermediate = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0, max_positions = 0;
    double eps = 1e-6, theta = 10000.0;
    bool tie = false;
    std::vector<int> eos;
};

long long want_int(const llb::Json& j, const std::string& key, const std::string& where, long long fallback = -1) {
    const llb::Json* v = j.find(key);
    if (!v || v->kind == llb::Json::Null) {
        if (fallback >= 0) return fallback;
        die(where + ": required key '" + key + "' is missing");
    }
    if (v->kind != llb::Json::Number || v->number != std::floor(v->number)) die(where + ": key '" + key + "' must be an integer");
    if (v->number < 1) die(where + ": key '" + key + "' must be >= 1");
    return (long long)v->number;
}
double want_real(const llb::Json& j, const std::string& key, const std::string& where, double fallback) {
    const llb::Json* v = j.find(key);
    if (!v || v->kind == llb::Json::Null) return fallback;
    if (v->kind != llb::Json::Number || !(v->number > 0)) die(where + ": key '" + key + "' must be a number > 0");
    return v->number;
}
bool want_bool(const llb::Json& j, const std::string& key, const std::string& where, bool fallback) {
    const llb::Json* v = j.find(key);
    if (!v || v->kind == llb::Json::Null) return fallback;
    if (v->kind != llb::Json::Bool) die(where + ": key '" + key + "' must be true or false");
    return v->boolean;
}

Config read_config(const std::string& dir) {
    const std::string path = dir + "/config.json";
    MappedFile f(path);
    llb::Json j;
    try {
        j = llb::JsonParser((const char*)f.data, f.size, path).parse();
    } catch (const std::exception& e) { die(e.what()); }
    if (j.kind != llb::Json::Object) die(path + ": top level must be an object");
    const llb::Json* archs = j.find("architectures");
    if (!archs || archs->kind != llb::Json::Array || archs->items.empty() || archs->items[0].kind != llb::Json::String)
        die(path + ": required key 'architectures' must be a non-empty list of names");
    if (archs->items[0].text != "Qwen2ForCausalLM")
        die(path + ": architecture '" + archs->items[0].text + "' is not one this program runs (Qwen2ForCausalLM); "
            "python -m lightllm_b200.cli.generate runs every registered architecture");
    Config c;
    c.hidden = (int)want_int(j, "hidden_size", path);
    c.heads = (int)want_int(j, "num_attention_heads", path);
    c.kv_heads = (int)want_int(j, "num_key_value_heads", path, c.heads);
    const llb::Json* hd = j.find("head_dim");
    if (hd && hd->kind != llb::Json::Null) c.head_dim = (int)want_int(j, "head_dim", path);
    else {
        if (c.hidden % c.heads) die(path + ": 'hidden_size' is not a multiple of 'num_attention_heads' and no 'head_dim' is given");
        c.head_dim = c.hidden / c.heads;
    }
    if (c.heads % c.kv_heads) die(path + ": 'num_attention_heads' is not a multiple of 'num_key_value_heads'");
    if (c.head_dim % 2) die(path + ": 'head_dim' must be even for rotary positions");
    const llb::Json* act = j.find("hidden_act");
    if (act && act->kind != llb::Json::Null && (act->kind != llb::Json::String || act->text != "silu"))
        die(path + ": 'hidden_act' must be 'silu'");
    const llb::Json* scaling = j.find("rope_scaling");
    if (scaling && scaling->kind != llb::Json::Null && !(scaling->kind == llb::Json::Object && scaling->members.empty()))
        die(path + ": 'rope_scaling' is not supported");
    c.layers = (int)want_int(j, "num_hidden_layers", path);
    c.vocab = (int)want_int(j, "vocab_size", path);
    c.intermediate = (int)want_int(j, "intermediate_size", path);
    c.max_positions = (int)want_int(j, "max_position_embeddings", path);
    c.eps = want_real(j, "rms_norm_eps", path, 1e-6);
    c.theta = want_real(j, "rope_theta", path, 10000.0);
    c.tie = want_bool(j, "tie_word_embeddings", path, false);
    if (want_bool(j, "use_sliding_window", path, false)) {
        const long long first = want_int(j, "max_window_layers", path, c.layers);
        if (first < c.layers)
            die(path + ": layers with a sliding window need a cache group of their own, which this program does not keep; "
                "use python -m lightllm_b200.cli.generate");
    }
    const llb::Json* eos = j.find("eos_token_id");
    if (eos && eos->kind == llb::Json::Number) c.eos.push_back((int)eos->number);
    if (eos && eos->kind == llb::Json::Array)
        for (const auto& e : eos->items)
            if (e.kind == llb::Json::Number) c.eos.push_back((int)e.number);
    return c;
}

// ---- device memory --------------------------------------------------------------------------------------------------
struct Device {
    std::vector<void*> owned;
    cudaStream_t stream = nullptr;
    void* alloc(size_t bytes, bool zero = false) {
        void* p = nullptr;
        cuda_ok(cudaMalloc(&p, bytes ? bytes : 16), "cudaMalloc");
        if (zero) cuda_ok(cudaMemset(p, 0, bytes ? bytes : 16), "cudaMemset");
        owned.push_back(p);
        return p;
    }
    void* upload(const void* host, size_t bytes) {
        void* p = alloc(bytes);
        cuda_ok(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice), "copy of a weight to the device");
        return p;
    }
    void release(void* p) {
        auto it = std::find(owned.begin(), owned.end(), p);
        if (it != owned.end()) { cudaFree(p); owned.erase(it); }
    }
    ~Device() { for (void* p : owned) cudaFree(p); }
};

// ---- weights --------------------------------------------------------------------------------------------------------
struct Weights {
    std::vector<LlbLayerDesc> layers;
    const void* embed = nullptr;
    int embed_dtype = BF16;
    const void* head = nullptr;
    LlbNormDesc final_norm{};
    size_t bytes = 0;
};

struct Loader {
    SafeTensors& st;
    Device* dev;                     // null: only check names, shapes and dtypes
    std::vector<std::string> missing, wrong;
    size_t bytes = 0;

    const Tensor* get(const std::string& name, std::initializer_list<long long> shape) {
        auto it = st.tensors.find(name);
        if (it == st.tensors.end()) { missing.push_back(name); return nullptr; }
        st.used.insert(name);
        const Tensor& t = it->second;
        if (t.shape != std::vector<long long>(shape)) {
            auto text = [](const std::vector<long long>& dims) {
                std::string out = "[";
                for (size_t i = 0; i < dims.size(); ++i) out += (i ? ", " : "") + std::to_string(dims[i]);
                return out + "]";
            };
            wrong.push_back(name + " has shape " + text(t.shape) + ", expected " + text(std::vector<long long>(shape)));
            return nullptr;
        }
        if (t.dtype != "BF16" && t.dtype != "F32") { wrong.push_back(name + " has dtype " + t.dtype); return nullptr; }
        return &t;
    }
    // a matrix of the contractions: bfloat16 as stored
    const Tensor* matrix(const std::string& name, long long rows, long long cols) {
        const Tensor* t = get(name, {rows, cols});
        if (t && t->dtype != "BF16") {
            wrong.push_back(name + " is stored in " + t->dtype + ": this program runs bfloat16 weights only "
                            "(python -m lightllm_b200.cli.generate keeps a tensor's stored precision)");
            return nullptr;
        }
        return t;
    }
    static void to_float(const Tensor& t, float* out) {
        const long long n = t.numel();
        if (t.dtype == "F32") { std::memcpy(out, t.data, (size_t)n * 4); return; }
        const uint16_t* h = (const uint16_t*)t.data;
        for (long long i = 0; i < n; ++i) {
            const uint32_t u = (uint32_t)h[i] << 16;
            std::memcpy(out + i, &u, 4);
        }
    }
    void* keep(const void* host, size_t n) {
        bytes += n;
        return dev ? dev->upload(host, n) : (void*)16;
    }
    LlbNormDesc norm(const std::string& name, long long hidden, double eps) {
        LlbNormDesc d{};
        d.eps = (float)eps;
        if (const Tensor* t = get(name, {hidden})) {
            d.weight = keep(t->data, t->bytes);
            d.weight_dtype = t->dtype == "BF16" ? BF16 : F32;
        }
        return d;
    }
};

// With dev == null nothing is copied: the file is only checked against the configuration (before a device is touched).
Weights load_weights(SafeTensors& st, const std::string& dir, const Config& c, Device* dev, const float* inv_freq_dev) {
    Loader ld{st, dev};
    st.used.clear();
    Weights w;
    const long long D = c.hidden, I = c.intermediate, hd = c.head_dim, Nq = (long long)c.heads * hd, Nkv = (long long)c.kv_heads * hd;
    if (const Tensor* t = ld.get("model.embed_tokens.weight", {c.vocab, D})) {
        w.embed = ld.keep(t->data, t->bytes);
        w.embed_dtype = t->dtype == "BF16" ? BF16 : F32;
        if (c.tie) {
            if (t->dtype != "BF16") ld.wrong.push_back("model.embed_tokens.weight is the head too and is stored in F32: bfloat16 only");
            w.head = w.embed;
        }
    }
    if (!c.tie)
        if (const Tensor* t = ld.matrix("lm_head.weight", c.vocab, D)) w.head = ld.keep(t->data, t->bytes);
    w.final_norm = ld.norm("model.norm.weight", D, c.eps);
    std::vector<uint8_t> qkv((size_t)(Nq + 2 * Nkv) * D * 2), gate_up((size_t)2 * I * D * 2);
    std::vector<float> bias((size_t)(Nq + 2 * Nkv));
    for (int l = 0; l < c.layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        LlbLayerDesc L{};
        L.norm1 = ld.norm(p + "input_layernorm.weight", D, c.eps);
        L.norm2 = ld.norm(p + "post_attention_layernorm.weight", D, c.eps);
        // q, k and v rows in one matrix, q first; their biases in float
        const Tensor *wq = ld.matrix(p + "self_attn.q_proj.weight", Nq, D), *wk = ld.matrix(p + "self_attn.k_proj.weight", Nkv, D),
                     *wv = ld.matrix(p + "self_attn.v_proj.weight", Nkv, D);
        const Tensor *bq = ld.get(p + "self_attn.q_proj.bias", {Nq}), *bk = ld.get(p + "self_attn.k_proj.bias", {Nkv}),
                     *bv = ld.get(p + "self_attn.v_proj.bias", {Nkv});
        if (wq && wk && wv) {
            if (dev) {
                std::memcpy(qkv.data(), wq->data, wq->bytes);
                std::memcpy(qkv.data() + wq->bytes, wk->data, wk->bytes);
                std::memcpy(qkv.data() + wq->bytes + wk->bytes, wv->data, wv->bytes);
            }
            L.attn.w_qkv = ld.keep(qkv.data(), qkv.size());
        }
        if (bq && bk && bv) {
            Loader::to_float(*bq, bias.data());
            Loader::to_float(*bk, bias.data() + Nq);
            Loader::to_float(*bv, bias.data() + Nq + Nkv);
            L.attn.b_qkv = (const float*)ld.keep(bias.data(), bias.size() * 4);
        }
        if (const Tensor* t = ld.matrix(p + "self_attn.o_proj.weight", D, Nq)) L.attn.w_o = ld.keep(t->data, t->bytes);
        L.attn.inv_freq = inv_freq_dev;
        L.attn.writes = 1;
        L.attn.group = 0;
        L.attn.num_heads = c.heads;
        L.attn.num_kv_heads = c.kv_heads;
        L.attn.head_dim = c.head_dim;
        L.attn.window = 0;
        L.attn.scale = (float)(1.0 / std::sqrt((double)c.head_dim));
        L.attn.rotary_dim = c.head_dim;
        L.attn.interleaved = 0;
        L.attn.plan = 0;
        L.attn.freqs = 0;
        // gate and up rows interleaved: row 2j is gate's row j, row 2j+1 is up's
        const Tensor *wg = ld.matrix(p + "mlp.gate_proj.weight", I, D), *wu = ld.matrix(p + "mlp.up_proj.weight", I, D);
        if (wg && wu) {
            const size_t row = (size_t)D * 2;
            for (long long j = 0; dev && j < I; ++j) {
                std::memcpy(gate_up.data() + (size_t)(2 * j) * row, wg->data + (size_t)j * row, row);
                std::memcpy(gate_up.data() + (size_t)(2 * j + 1) * row, wu->data + (size_t)j * row, row);
            }
            L.mlp.w_gate_up = ld.keep(gate_up.data(), gate_up.size());
        }
        if (const Tensor* t = ld.matrix(p + "mlp.down_proj.weight", D, I)) L.mlp.w_down = ld.keep(t->data, t->bytes);
        L.mlp.intermediate = c.intermediate;
        w.layers.push_back(L);
    }
    // one error that lists everything that is wrong with the file
    std::vector<std::string> unexpected;
    for (const auto& kv : st.tensors) {
        const std::string& n = kv.first;
        const bool ignored = n.size() >= 19 && n.compare(n.size() - 19, 19, "rotary_emb.inv_freq") == 0;
        if (!st.used.count(n) && !ignored && !(c.tie && n == "lm_head.weight")) unexpected.push_back(n);
    }
    if (!ld.missing.empty() || !ld.wrong.empty() || !unexpected.empty()) {
        std::string msg = dir + "/model.safetensors does not fit config.json:";
        auto list = [&msg](const char* title, const std::vector<std::string>& v) {
            if (v.empty()) return;
            msg += std::string("\n  ") + title + " (" + std::to_string(v.size()) + "):";
            for (size_t i = 0; i < v.size() && i < 12; ++i) msg += "\n    " + v[i];
            if (v.size() > 12) msg += "\n    ...";
        };
        list("missing tensors", ld.missing);
        list("unexpected tensors", unexpected);
        list("wrong shape or dtype", ld.wrong);
        die(msg);
    }
    w.bytes = ld.bytes;
    return w;
}

// ---- the attention kernel's work items (engine/batch.py: cut_attention_rows) ----------------------------------------
struct RowTile { int span, q0, ntiles; };
struct Item { int len, span, q0, k0, nk, part; };
struct Merge { int span, q0, first, count; };
struct Cut { std::vector<Item> items; std::vector<Merge> merges; int parts = 0; };

Cut cut_rows(const std::vector<RowTile>& rows, int chunk) {
    Cut c;
    for (const RowTile& r : rows) {
        if (r.ntiles <= chunk + 1) { c.items.push_back({r.ntiles, r.span, r.q0, 0, r.ntiles, -1}); continue; }
        const int n = ceil_div(r.ntiles, chunk);
        c.merges.push_back({r.span, r.q0, c.parts, n});
        for (int i = 0; i < n; ++i) {
            const int nk = std::min(chunk, r.ntiles - i * chunk);
            c.items.push_back({nk, r.span, r.q0, i * chunk, nk, c.parts + i});
        }
        c.parts += n;
    }
    std::stable_sort(c.items.begin(), c.items.end(), [](const Item& a, const Item& b) { return a.len > b.len; });
    return c;
}

// Key tiles of the busiest block when the kernel deals the items (times heads, heads fastest) to `slots` blocks: one
// item of every round of `slots` items, every other round backwards.
double busiest_block(const std::vector<Item>& items, int heads, int slots) {
    const long long n = (long long)items.size() * heads;
    const long long grid = std::min<long long>(n, std::max(1, slots));
    std::vector<double> load((size_t)grid, 0.0);
    for (long long i = 0; i < n; ++i) {
        const long long pos = i % grid, slot = ((i / grid) % 2 == 0) ? pos : grid - 1 - pos;
        load[(size_t)slot] += items[(size_t)(i / heads)].len;
    }
    return *std::max_element(load.begin(), load.end());
}

// The piece length with the least estimated time (the busiest block's key tiles, plus what merging partial results
// costs), among a few candidates around the share of key tiles that a block gets anyway.
Cut cut_attention_rows(const std::vector<RowTile>& rows, int heads, int slots) {
    constexpr double TILE_US = 2.56, MERGE_US = 10.2, PART_US = 0.026;
    int longest = 0;
    long long total = 0;
    for (const RowTile& r : rows) { longest = std::max(longest, r.ntiles); total += r.ntiles; }
    const double share = (double)total * heads / std::max(1, slots);
    std::set<int> candidates{longest};
    for (double f : {0.34, 0.5, 0.75, 1.0, 1.5, 2.0, 3.0}) candidates.insert(std::min(longest, std::max(4, (int)std::ceil(share * f))));
    double best_cost = 0;
    int best = -1;
    for (int c : candidates) {
        const Cut cut = cut_rows(rows, c);
        double cost = TILE_US * busiest_block(cut.items, heads, slots);
        if (cut.parts) cost += MERGE_US + PART_US * cut.parts * heads;
        if (best < 0 || cost < best_cost - 1e-9) { best_cost = cost; best = c; }
    }
    return cut_rows(rows, best);
}

// ---- requests and the cache's pages ---------------------------------------------------------------------------------
struct Request {
    std::vector<int> prompt, generated;
    std::vector<int> pages;
    int cached = 0;                  // tokens whose keys and values are in the cache
    const char* reason = nullptr;    // why it ended
    int length() const { return (int)prompt.size() + (int)generated.size(); }
};
struct Span { int request, count; bool want; };

uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

struct Options {
    std::string model_dir;
    std::vector<std::vector<int>> prompts;
    int max_new_tokens = 12, top_k = 40, max_seq_len = 2048, max_batch_tokens = 2048, eos = -1;
    double temperature = 0.8, top_p = 0.9, min_p = 0.0;
    long long seed = 42;
    bool timing = false, graphs = true;
};

Options parse_args(int argc, char** argv) {
    Options o;
    std::vector<int> cur;
    bool any_tokens = false;
    auto value = [&](int& i) -> std::string {
        if (i + 1 >= argc) die(std::string("option ") + argv[i] + " needs a value");
        return argv[++i];
    };
    auto number = [&](const std::string& s, const char* name) -> double {
        char* stop = nullptr;
        const double v = std::strtod(s.c_str(), &stop);
        if (stop == s.c_str() || *stop) die(std::string("option ") + name + ": '" + s + "' is not a number");
        return v;
    };
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--max-new-tokens") o.max_new_tokens = (int)number(value(i), "--max-new-tokens");
        else if (a == "--temperature") o.temperature = number(value(i), "--temperature");
        else if (a == "--top-k") o.top_k = (int)number(value(i), "--top-k");
        else if (a == "--top-p") o.top_p = number(value(i), "--top-p");
        else if (a == "--min-p") o.min_p = number(value(i), "--min-p");
        else if (a == "--seed") o.seed = (long long)number(value(i), "--seed");
        else if (a == "--eos-token-id") o.eos = (int)number(value(i), "--eos-token-id");
        else if (a == "--max-seq-len") o.max_seq_len = (int)number(value(i), "--max-seq-len");
        else if (a == "--max-batch-tokens") o.max_batch_tokens = (int)number(value(i), "--max-batch-tokens");
        else if (a == "--dtype") { if (value(i) != "bfloat16") die("--dtype: this program runs bfloat16 only; python -m lightllm_b200.cli.generate runs float32"); }
        else if (a == "--timing") o.timing = true;
        else if (a == "--no-graphs") o.graphs = false;
        else if (a == "-h" || a == "--help") {
            std::printf("usage: generate <model_dir> [token ids ... [/ token ids ...]] [--max-new-tokens N] [--temperature T] [--top-k K]\n"
                        "                [--top-p P] [--min-p P] [--seed S] [--eos-token-id ID] [--max-seq-len N] [--max-batch-tokens N]\n"
                        "                [--timing] [--no-graphs]\n");
            std::exit(0);
        } else if (a == "/") {
            if (cur.empty()) die("an empty prompt before '/'");
            o.prompts.push_back(cur);
            cur.clear();
        } else if (a.size() > 1 && a[0] == '-' && !(a[1] >= '0' && a[1] <= '9')) {
            die("unknown option " + a);
        } else if (o.model_dir.empty()) {
            o.model_dir = a;
        } else {
            cur.push_back((int)number(a, "token id"));
            any_tokens = true;
        }
    }
    if (o.model_dir.empty()) die("usage: generate <model_dir> [token ids ...] (see --help)");
    if (!cur.empty()) o.prompts.push_back(cur);
    else if (any_tokens) die("an empty prompt after '/'");
    if (o.prompts.empty()) o.prompts.push_back({576, 8319, 315, 13466, 374});
    if (o.max_new_tokens < 1) die("--max-new-tokens must be >= 1");
    if (o.max_seq_len < 2) die("--max-seq-len must be >= 2");
    if (o.max_batch_tokens < 1) die("--max-batch-tokens must be >= 1");
    if (o.temperature < 0) die("--temperature must be >= 0");
    return o;
}

// generate --cut-rows "<key tiles of row tile 0> <of row tile 1> ..." <heads> <slots>: prints how the attention kernel's
// items would be cut (the planner alone, for the test that compares it with the Python engine's).
int print_cut(int argc, char** argv) {
    if (argc != 5) die("usage: generate --cut-rows \"n0 n1 ...\" <heads> <slots>");
    std::vector<RowTile> rows;
    const char* c = argv[2];
    char* stop = nullptr;
    for (;;) {
        const long v = std::strtol(c, &stop, 10);
        if (stop == c) break;
        rows.push_back({0, 128 * (int)rows.size(), (int)v});
        c = stop;
    }
    if (rows.empty()) die("--cut-rows: no row tiles");
    const Cut cut = cut_attention_rows(rows, std::atoi(argv[3]), std::atoi(argv[4]));
    for (const Item& it : cut.items) std::printf("item %d %d %d %d %d %d\n", it.len, it.span, it.q0, it.k0, it.nk, it.part);
    for (const Merge& m : cut.merges) std::printf("merge %d %d %d %d\n", m.span, m.q0, m.first, m.count);
    std::printf("parts %d\n", cut.parts);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 2 && std::string(argv[1]) == "--cut-rows") return print_cut(argc, argv);
    const Options opt = parse_args(argc, argv);
    if (llb_abi_version() != EXPECTED_ABI)
        die("the kernel library has ABI " + std::to_string(llb_abi_version()) + ", this program was built for " + std::to_string(EXPECTED_ABI));
    {
        int sizes[8] = {0};
        llb_step_struct_sizes(sizes);
        const int mine[8] = {(int)sizeof(LlbNormDesc), (int)sizeof(LlbAttentionDesc), (int)sizeof(LlbMlpDesc), (int)sizeof(LlbLayerDesc),
                             (int)sizeof(LlbModelDesc), (int)sizeof(LlbTileList), (int)sizeof(LlbAttentionPlan), (int)sizeof(LlbStepArgs)};
        if (std::memcmp(sizes, mine, sizeof(mine)) != 0)
            die("the kernel library lays the step executor's records out differently");
    }
    const Config cfg = read_config(opt.model_dir);
    const int D = cfg.hidden, V = cfg.vocab, hd = cfg.head_dim;
    if (!llb_attention_tcgen05_supports(hd, PAGE) || !llb_paged_decode_mma_supports(cfg.heads, cfg.kv_heads, hd) || D % 8 != 0 ||
        (cfg.heads * hd) % 8 != 0 || cfg.intermediate % 8 != 0)
        die("heads of " + std::to_string(hd) + " (" + std::to_string(cfg.heads) + " over " + std::to_string(cfg.kv_heads) +
            ") or these widths are outside what the tensor-core kernels take; python -m lightllm_b200.cli.generate runs them "
            "on the other kernels");
    const int max_seq_len = std::min(opt.max_seq_len, cfg.max_positions);
    const int nreq = (int)opt.prompts.size();

    SafeTensors st(opt.model_dir + "/model.safetensors");
    load_weights(st, opt.model_dir, cfg, nullptr, nullptr);        // every fault of the file, before a device is touched

    int device_count = 0;
    if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_count == 0) die("no CUDA device");
    cuda_ok(cudaSetDevice(0), "cudaSetDevice");
    cudaDeviceProp prop;
    cuda_ok(cudaGetDeviceProperties(&prop, 0), "cudaGetDeviceProperties");
    if (prop.major != 10) die(std::string("the kernels are built for sm_100a; device 0 is ") + prop.name);
    const int sms = prop.multiProcessorCount;
    Device dev;
    cuda_ok(cudaStreamCreateWithFlags(&dev.stream, cudaStreamNonBlocking), "cudaStreamCreate");

    // requests
    std::vector<Request> reqs((size_t)nreq);
    long long pool_pages = 0;
    for (int r = 0; r < nreq; ++r) {
        for (int t : opt.prompts[(size_t)r]) reqs[(size_t)r].prompt.push_back(((t % V) + V) % V);
        const int n = (int)reqs[(size_t)r].prompt.size();
        if (n + 1 > max_seq_len) die("prompt " + std::to_string(r) + " has " + std::to_string(n) + " tokens; --max-seq-len is " + std::to_string(max_seq_len));
        pool_pages += ceil_div(std::min(n + opt.max_new_tokens, max_seq_len), PAGE);
    }
    const int max_pages = ceil_div(max_seq_len, PAGE);

    // rotary frequencies: 1 / theta^(2i / head_dim), computed in double and rounded to float
    std::vector<float> inv_freq((size_t)hd / 2);
    for (int i = 0; i < hd / 2; ++i) inv_freq[(size_t)i] = (float)(1.0 / std::pow(cfg.theta, (double)(2 * i) / hd));
    const float* inv_freq_dev = (const float*)dev.upload(inv_freq.data(), inv_freq.size() * 4);

    const auto t_load = std::chrono::steady_clock::now();
    Weights w = load_weights(st, opt.model_dir, cfg, &dev, inv_freq_dev);
    const long long slots = pool_pages * PAGE;
    const size_t plane = (size_t)slots * cfg.kv_heads * hd * 2;
    for (LlbLayerDesc& L : w.layers) {
        L.attn.k_cache = dev.alloc(plane, true);
        L.attn.v_cache = dev.alloc(plane, true);
        L.attn.num_slots = slots;
    }
    std::vector<int> free_pages;
    for (int p = (int)pool_pages - 1; p >= 0; --p) free_pages.push_back(p);
    LlbModelDesc model{};
    model.layers = w.layers.data();
    model.num_layers = cfg.layers;
    model.hidden = D;
    model.act_dtype = BF16;
    model.num_sms = sms;
    if (opt.timing)
        std::fprintf(stderr, "[generate] %.2f GB of weights and %.2f GB of cache on %s in %.1f s\n", w.bytes / 1e9,
                     2.0 * plane * cfg.layers / 1e9, prop.name,
                     std::chrono::duration<double>(std::chrono::steady_clock::now() - t_load).count());

    // buffers of a step
    const int max_T = opt.max_batch_tokens + nreq;
    float* residual = (float*)dev.alloc((size_t)max_T * D * 4);
    float* logits = (float*)dev.alloc((size_t)nreq * V * 4);
    const int Nqkv = (cfg.heads + 2 * cfg.kv_heads) * hd, widest = std::max(Nqkv, 2 * cfg.intermediate);
    const long long splitk_floats = (long long)DECODE_ROWS * widest;
    float* splitk = (float*)dev.alloc((size_t)splitk_floats * 4, true);
    const int splitk_tiles = ceil_div(widest, 128);
    int* splitk_counters = (int*)dev.alloc((size_t)splitk_tiles * 4, true);
    const int meet_n = 1 << 16;
    int* meet = (int*)dev.alloc((size_t)meet_n * 4, true);
    int* flags = (int*)dev.alloc(2 * 4, true);           // [0] raised by a kernel whose wait ran out, [1] by a token id out of range
    const int argmax_rows = 64;
    int* argmax_scratch = (int*)dev.alloc((size_t)3 * argmax_rows * 4, true);
    // the step's integers: one pinned array, one copy
    const size_t row_tiles_max = (size_t)ceil_div(max_T, 128) + (size_t)nreq;
    const size_t items_max = row_tiles_max * ((size_t)ceil_div(ceil_div(max_seq_len, 128), 4) + 1);      // pieces have 4 key tiles or more
    const size_t meta_words = (size_t)max_T * 3 + (size_t)nreq * (8 + max_pages + 32) + items_max * 5 + row_tiles_max * 4 + 256;
    int* meta_host = nullptr;
    cuda_ok(cudaMallocHost((void**)&meta_host, meta_words * 4), "cudaMallocHost");
    int* meta_dev = (int*)dev.alloc(meta_words * 4);
    float* samp_host = nullptr;                           // per wanted row: temperature, top_p, min_p, uniform; then top_k
    cuda_ok(cudaMallocHost((void**)&samp_host, (size_t)nreq * 5 * 4), "cudaMallocHost");
    float* samp_dev = (float*)dev.alloc((size_t)nreq * 5 * 4);
    int* out_dev = (int*)dev.alloc((size_t)(nreq + 2) * 4);
    int* out_host = nullptr;
    cuda_ok(cudaMallocHost((void**)&out_host, (size_t)(nreq + 2) * 4), "cudaMallocHost");
    void* workspace = nullptr;
    long long workspace_bytes = 0;

    cuda_ok(cudaDeviceSynchronize(), "setting up the device");      // the uploads and clears above ran on the default stream

    std::set<int> eos(cfg.eos.begin(), cfg.eos.end());
    if (opt.eos >= 0) eos = {opt.eos};
    const int cluster_splits = llb_paged_decode_mma_cluster_splits();
    const int blocks_per_sm = llb_paged_decode_mma_resident(hd);
    if (blocks_per_sm <= 0) die(std::string("decode attention: ") + llb_last_error());
    long long steps = 0, prompt_tokens = 0, new_tokens = 0, graph_steps = 0, decode_tokens = 0;
    std::map<std::pair<int, int>, cudaGraphExec_t> graphs;          // by (requests, block-table width) of a decoding step
    std::set<std::pair<int, int>> seen_shapes;
    double first_token_s = 0;
    const auto t0 = std::chrono::steady_clock::now();

    for (;;) {
        // ---- what this step runs: one token of every decoding request, then portions of prompts under the budget ----
        std::vector<Span> spans;
        int budget = opt.max_batch_tokens;
        for (int r = 0; r < nreq; ++r) {
            Request& q = reqs[(size_t)r];
            if (!q.reason && q.cached >= (int)q.prompt.size()) spans.push_back({r, 1, true});
        }
        for (int r = 0; r < nreq && budget > 0; ++r) {
            Request& q = reqs[(size_t)r];
            const int left = (int)q.prompt.size() - q.cached;
            if (q.reason || left <= 0) continue;
            const int n = std::min(left, budget);
            spans.push_back({r, n, n == left});
            budget -= n;
        }
        if (spans.empty()) break;
        const int S = (int)spans.size();
        int T = 0, max_context = 0, R = 0;
        bool decode_only = true;
        for (const Span& s : spans) {
            T += s.count;
            max_context = std::max(max_context, reqs[(size_t)s.request].cached + s.count);
            decode_only = decode_only && s.count == 1;
            R += s.want ? 1 : 0;
        }
        if (T > max_T) die("internal: a step of " + std::to_string(T) + " tokens");
        const int P = std::min(max_pages, ceil_div(ceil_div(max_context, PAGE), 32) * 32);

        // ---- the step's integers ------------------------------------------------------------------------------------
        size_t at = 0;
        auto take = [&](size_t n) -> size_t {
            const size_t here = at;
            at += (n + 3) & ~(size_t)3;                  // 16-byte steps
            if (at > meta_words) die("internal: the step's metadata outgrew its buffer");
            return here;
        };
        const size_t o_tok = take((size_t)T), o_pos = take((size_t)T), o_slot = take((size_t)T), o_row = take((size_t)S),
                     o_len = take((size_t)S), o_start = take((size_t)S), o_iota = take((size_t)S), o_zero = take((size_t)S),
                     o_want = take((size_t)std::max(R, 1)), o_bt = take((size_t)S * P);
        int row = 0, nw = 0;
        for (int i = 0; i < S; ++i) {
            const Span& s = spans[(size_t)i];
            Request& q = reqs[(size_t)s.request];
            const int start = q.cached;
            while ((int)q.pages.size() * PAGE < start + s.count) {
                if (free_pages.empty()) die("internal: the cache ran out of pages");
                q.pages.push_back(free_pages.back());
                free_pages.pop_back();
            }
            meta_host[o_row + i] = row;
            meta_host[o_len + i] = s.count;
            meta_host[o_start + i] = start;
            meta_host[o_iota + i] = i;
            meta_host[o_zero + i] = 0;
            for (int p = 0; p < P; ++p) meta_host[o_bt + (size_t)i * P + p] = p < (int)q.pages.size() ? q.pages[(size_t)p] : 0;
            for (int j = 0; j < s.count; ++j) {
                const int pos = start + j;
                const int tok = pos < (int)q.prompt.size() ? q.prompt[(size_t)pos] : q.generated[(size_t)(pos - (int)q.prompt.size())];
                meta_host[o_tok + row + j] = tok;
                meta_host[o_pos + row + j] = pos;
                meta_host[o_slot + row + j] = q.pages[(size_t)(pos / PAGE)] * PAGE + pos % PAGE;
            }
            if (s.want) meta_host[o_want + nw++] = row + s.count - 1;
            row += s.count;
        }

        // ---- the attention plan (parts/attention.py: AttentionMixer._plan) ------------------------------------------
        LlbAttentionPlan plan{};
        auto decode_splits = [&](int nspans) {
            const int bound = P * PAGE;
            int nsplit = std::max(1, std::min(std::max(1, ceil_div(2 * sms, (long long)nspans * cfg.kv_heads)), ceil_div(bound, 128)));
            if (bound <= CLUSTER_MERGE_MAX_KEYS) {
                const int resident = blocks_per_sm * sms / (nspans * cfg.kv_heads);
                nsplit = std::max(1, std::min(std::min(8, cluster_splits), std::min(resident, ceil_div(bound, 128))));
            }
            return nsplit;
        };
        if (decode_only) {
            plan.kind = 0;
            plan.decode = LlbTileList{meta_dev + o_iota, meta_dev + o_zero, S, 1, decode_splits(S), 0};
        } else {
            plan.kind = 2;
            std::vector<RowTile> rows;
            std::vector<int> single;
            for (int i = 0; i < S; ++i) {
                const int start = meta_host[o_start + i], len = spans[(size_t)i].count;
                if (len == 1) { single.push_back(i); continue; }
                for (int q0 = 0; q0 < len; q0 += 128) {
                    const int hi = q0 + 128 <= len ? start + q0 + 128 : start + len;
                    rows.push_back({i, q0, ceil_div(hi, 128)});
                }
            }
            if (!rows.empty()) {
                const Cut cut = cut_attention_rows(rows, cfg.heads, (hd <= 64 ? 2 : 1) * sms);
                const size_t n = cut.items.size();
                const size_t o_span = take(n), o_q0 = take(n), o_k0 = take(n), o_nk = take(n), o_part = take(n);
                for (size_t i = 0; i < n; ++i) {
                    const Item& it = cut.items[i];
                    meta_host[o_span + i] = it.span;
                    meta_host[o_q0 + i] = it.q0;
                    meta_host[o_k0 + i] = it.k0;
                    meta_host[o_nk + i] = it.nk;
                    meta_host[o_part + i] = it.part;
                }
                plan.items = LlbTileList{meta_dev + o_span, meta_dev + o_q0, (int)n, 128, 1, 0};
                plan.item_k0 = meta_dev + o_k0;
                plan.item_nk = meta_dev + o_nk;
                plan.item_part = meta_dev + o_part;
                plan.num_parts = cut.parts;
                plan.num_merge = (int)cut.merges.size();
                if (plan.num_merge) {
                    const size_t m = cut.merges.size();
                    const size_t o_ms = take(m), o_mq = take(m), o_mf = take(m), o_mc = take(m);
                    for (size_t i = 0; i < m; ++i) {
                        meta_host[o_ms + i] = cut.merges[i].span;
                        meta_host[o_mq + i] = cut.merges[i].q0;
                        meta_host[o_mf + i] = cut.merges[i].first;
                        meta_host[o_mc + i] = cut.merges[i].count;
                    }
                    plan.merge_span = meta_dev + o_ms;
                    plan.merge_q0 = meta_dev + o_mq;
                    plan.merge_first = meta_dev + o_mf;
                    plan.merge_count = meta_dev + o_mc;
                }
            }
            if (!single.empty()) {
                const size_t n = single.size();
                const size_t o_span = take(n), o_q0 = take(n);
                for (size_t i = 0; i < n; ++i) { meta_host[o_span + i] = single[i]; meta_host[o_q0 + i] = 0; }
                plan.decode = LlbTileList{meta_dev + o_span, meta_dev + o_q0, (int)n, 1, decode_splits((int)n), 0};
            }
        }
        cuda_ok(cudaMemcpyAsync(meta_dev, meta_host, at * 4, cudaMemcpyHostToDevice, dev.stream), "copy of the step's metadata");

        // ---- the step -----------------------------------------------------------------------------------------------
        LlbStepArgs step{};
        step.token_ids = meta_dev + o_tok;
        step.positions = meta_dev + o_pos;
        step.span_row = meta_dev + o_row;
        step.span_len = meta_dev + o_len;
        step.span_pos = meta_dev + o_start;
        step.block_tables[0] = meta_dev + o_bt;
        step.slot_mapping[0] = meta_dev + o_slot;
        step.residual = residual;
        step.plans = &plan;
        step.num_plans = 1;
        step.splitk_scratch = splitk;
        step.splitk_floats = splitk_floats;
        step.splitk_counters = splitk_counters;
        step.splitk_tiles = splitk_tiles;
        step.meet_counters = meet;
        step.meet_counters_n = meet_n;
        step.error_flag = flags;
        step.stream = dev.stream;
        step.T = T;
        step.S = S;
        step.max_pages = P;
        step.page_size = PAGE;
        step.first_layer = 0;
        step.last_layer = cfg.layers;
        const long long need = std::max(llb_step_workspace_need(&model, &step), llb_step_head_workspace_need(&model, &step, V, R));
        if (need < 0) die(std::string("the step cannot be laid out: ") + llb_last_error());
        if (need > workspace_bytes) {
            if (workspace) { cuda_ok(cudaStreamSynchronize(dev.stream), "synchronize"); dev.release(workspace); }
            for (auto& g : graphs) cudaGraphExecDestroy(g.second);          // they name the old workspace
            graphs.clear();
            workspace_bytes = need + need / 4 + (1 << 20);
            workspace = dev.alloc((size_t)workspace_bytes);
        }
        step.workspace = workspace;
        step.workspace_bytes = workspace_bytes;

        if (R > 0 && opt.temperature != 0.0) {
            float *temp = samp_host, *top_p = samp_host + nreq, *min_p = samp_host + 2 * nreq, *uni = samp_host + 3 * nreq;
            int* top_k = (int*)(samp_host + 4 * nreq);
            int k = 0;
            for (const Span& s : spans) {
                if (!s.want) continue;
                const Request& q = reqs[(size_t)s.request];
                temp[k] = (float)opt.temperature;
                top_p[k] = (float)opt.top_p;
                min_p[k] = (float)opt.min_p;
                top_k[k] = opt.top_k;
                const uint64_t bits = splitmix64(splitmix64((uint64_t)opt.seed) ^ splitmix64(((uint64_t)s.request << 32) | (uint64_t)q.generated.size()));
                uni[k] = (float)((bits >> 40) * (1.0 / 16777216.0));        // 24 bits: in [0, 1)
                ++k;
            }
            cuda_ok(cudaMemcpyAsync(samp_dev, samp_host, (size_t)nreq * 5 * 4, cudaMemcpyHostToDevice, dev.stream), "copy of the sampling parameters");
        }
        // every launch of the step: they read the step's integers and parameters from fixed places of the device
        auto issue = [&]() {
            lib_ok(llb_embedding(step.token_ids, w.embed, w.embed_dtype, residual, T, D, V, flags + 1, dev.stream), "embedding");
            lib_ok(llb_step_layers(&model, &step), "layers");
            if (R == 0) return;
            lib_ok(llb_step_head(&model, &step, &w.final_norm, w.head, V, meta_dev + o_want, R, logits), "head");
            if (opt.temperature == 0.0)
                lib_ok(llb_argmax(logits, R, V, V, out_dev, R <= argmax_rows ? argmax_scratch : nullptr, argmax_rows, dev.stream), "argmax");
            else
                lib_ok(llb_sample(logits, R, V, V, samp_dev, (const int*)(samp_dev + 4 * nreq), samp_dev + nreq, samp_dev + 2 * nreq,
                                  samp_dev + 3 * nreq, out_dev, dev.stream), "sample");
        };
        // A decoding step of a shape seen before (so many requests, so wide a block table) is replayed as a CUDA graph:
        // its launches depend on nothing else, and its arrays lie where they lay the first time.
        const std::pair<int, int> shape{S, P};
        if (decode_only && opt.graphs && seen_shapes.count(shape)) {
            auto it = graphs.find(shape);
            if (it == graphs.end()) {
                cudaGraph_t graph = nullptr;
                cudaGraphExec_t exec = nullptr;
                cuda_ok(cudaStreamBeginCapture(dev.stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
                issue();
                cuda_ok(cudaStreamEndCapture(dev.stream, &graph), "cudaStreamEndCapture");
                cuda_ok(cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate");
                cudaGraphDestroy(graph);
                it = graphs.emplace(shape, exec).first;
            }
            cuda_ok(cudaGraphLaunch(it->second, dev.stream), "cudaGraphLaunch");
            ++graph_steps;
        } else {
            issue();
            if (decode_only) seen_shapes.insert(shape);
        }
        if (R > 0) cuda_ok(cudaMemcpyAsync(out_host, out_dev, (size_t)R * 4, cudaMemcpyDeviceToHost, dev.stream), "copy of the tokens");
        cuda_ok(cudaMemcpyAsync(out_host + nreq, flags, 8, cudaMemcpyDeviceToHost, dev.stream), "copy of the error flags");
        cuda_ok(cudaStreamSynchronize(dev.stream), "the step");
        if (out_host[nreq] != 0) die("a kernel gave up waiting (code " + std::to_string(out_host[nreq]) + "); the step's results are not valid");
        if (out_host[nreq + 1] != 0) die("a token id was outside the vocabulary");
        ++steps;

        // ---- what the step brought ------------------------------------------------------------------------------------
        int k = 0;
        for (const Span& s : spans) {
            Request& q = reqs[(size_t)s.request];
            if (q.cached < (int)q.prompt.size()) prompt_tokens += s.count;
            else ++decode_tokens;
            q.cached += s.count;
            if (!s.want) continue;
            const int tok = out_host[k++];
            if (tok < 0 || tok >= V) die("the sampler returned token " + std::to_string(tok));
            q.generated.push_back(tok);
            ++new_tokens;
            if (first_token_s == 0) first_token_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (eos.count(tok)) q.reason = "eos";
            else if ((int)q.generated.size() >= opt.max_new_tokens) q.reason = "length";
            else if (q.length() >= max_seq_len) q.reason = "max_seq_len";
            if (q.reason) {                                  // its pages go back
                for (int p : q.pages) free_pages.push_back(p);
                q.pages.clear();
            }
        }
    }
    const double total_s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();

    for (int r = 0; r < nreq; ++r) {
        const Request& q = reqs[(size_t)r];
        std::printf("prompt:   ");
        for (int t : q.prompt) std::printf(" %d", t);
        std::printf("\ngenerated:");
        for (int t : q.generated) std::printf(" %d", t);
        std::printf(" (%s)\n", q.reason ? q.reason : "?");
    }
    if (opt.timing) {
        // the figures of the reference's serving benchmark, under its names (tools/bench_server.cpp:226-245)
        std::fprintf(stderr, "  %-30s %lld (%lld replayed as graphs)\n", "Total steps:", steps, graph_steps);
        std::fprintf(stderr, "  %-30s %lld\n", "Prefill tokens processed:", prompt_tokens);
        std::fprintf(stderr, "  %-30s %lld\n", "Decode steps:", decode_tokens);
        std::fprintf(stderr, "  %-30s %lld\n", "Tokens generated:", new_tokens);
        std::fprintf(stderr, "  %-30s %.1f ms\n", "First token after:", first_token_s * 1e3);
        std::fprintf(stderr, "  %-30s %.4f s\n", "Elapsed time:", total_s);
        std::fprintf(stderr, "  %-30s %.1f tok/s\n", "Generation throughput:", new_tokens / std::max(total_s, 1e-9));
        std::fprintf(stderr, "  %-30s %.1f steps/s\n", "Steps per second:", steps / std::max(total_s, 1e-9));
    }
    if ((long long)free_pages.size() != pool_pages) die("internal: " + std::to_string(pool_pages - (long long)free_pages.size()) + " pages were not given back");
    for (auto& g : graphs) cudaGraphExecDestroy(g.second);
    cudaFreeHost(meta_host);
    cudaFreeHost(samp_host);
    cudaFreeHost(out_host);
    cudaStreamDestroy(dev.stream);
    return 0;
}
