// Calls the reference's own CPU oracles on fixed inputs and prints inputs and results as JSON:
//   cpu_attention                  tests/test_paged_attention_v2.cu:111-156   (every query sees every key)
//   cpu_prefill_attention_causal   tests/test_paged_prefill.cu:164-215        (the last P positions, causal)
//   cpu_lm_head                    tests/test_lm_head.cu:50-61
// The oracles are `static` functions of the reference's test programs, so each program is included whole, inside a
// namespace of its own and with its `main` renamed; that `main` is never called and no CUDA call is made.
// The inputs come from the small generator below, in the order q, k, v per shape and then hidden, embed; the tests
// draw them again with the same generator, so the JSON holds the shapes and the oracles' results only.
// Built and run by make_golden.sh; the committed attention_golden.json is what the tests read.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <numeric>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "lightllm/kv_cache/block_allocator.h"
#include "lightllm/kv_cache/paged_attention.h"
#include "lightllm/ops/lm_head.h"
#include "lightllm/tensor.h"

namespace ref_decode {
#define main ref_main
#include "tests/test_paged_attention_v2.cu"
#undef main
}  // namespace ref_decode
namespace ref_prefill {
#define main ref_main
#include "tests/test_paged_prefill.cu"
#undef main
}  // namespace ref_prefill
namespace ref_head {
#define main ref_main
#include "tests/test_lm_head.cu"
#undef main
}  // namespace ref_head

static unsigned long long g_state = 88172645463325252ull;
static float next_float() {      // xorshift, uniform in [-1, 1)
    g_state ^= g_state << 13; g_state ^= g_state >> 7; g_state ^= g_state << 17;
    return (float)((g_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
}
static std::vector<float> draw(size_t n, float scale) {
    std::vector<float> v(n);
    for (auto& x : v) x = next_float() * scale;
    return v;
}
static void print_array(const char* name, const std::vector<float>& v, bool last = false) {
    printf("  \"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) printf("%s%.9g", i ? ", " : "", v[i]);
    printf("]%s\n", last ? "" : ",");
}

int main() {
    struct Shape { int T, Hq, Hkv, D, seq; };
    const Shape shapes[] = {{1, 8, 2, 16, 37}, {1, 4, 1, 32, 50}, {5, 4, 2, 16, 23}, {4, 3, 1, 8, 9}, {3, 2, 2, 8, 3}};
    printf("{\"attention\": [\n");
    const int n = sizeof(shapes) / sizeof(shapes[0]);
    for (int c = 0; c < n; ++c) {
        const Shape s = shapes[c];
        auto q = draw((size_t)s.T * s.Hq * s.D, 1.5f);
        auto k = draw((size_t)s.seq * s.Hkv * s.D, 1.5f);
        auto v = draw((size_t)s.seq * s.Hkv * s.D, 1.0f);
        auto all = ref_decode::cpu_attention(q.data(), s.T, s.Hq, s.D, k.data(), s.seq, s.Hkv, v.data());
        auto causal = ref_prefill::cpu_prefill_attention_causal(q.data(), s.T, s.Hq, s.D, k.data(), s.seq, s.Hkv, v.data());
        printf(" {\"T\": %d, \"Hq\": %d, \"Hkv\": %d, \"D\": %d, \"seq_len\": %d,\n", s.T, s.Hq, s.Hkv, s.D, s.seq);
        print_array("every_key", all); print_array("causal", causal, true);
        printf(" }%s\n", c + 1 < n ? "," : "");
    }
    printf("],\n\"lm_head\": {\n");
    const int D = 24, V = 37;
    auto hidden = draw(D, 1.0f), embed = draw((size_t)V * D, 0.5f);
    auto logits = ref_head::cpu_lm_head(hidden.data(), D, embed.data(), V);
    printf("  \"D\": %d, \"V\": %d,\n", D, V);
    print_array("logits", logits, true);
    printf("}}\n");
    return 0;
}
