// Runs the reference's own GPU operators that have no known defect on fixed inputs and prints their results as JSON:
//   rms_norm    src/ops/norm.cu:11-75         silu   src/ops/elementwise.cu:27-33,  embedding   src/ops/embedding.cu:9-30
// Inputs come from the generator of golden_attention.cu (same seed), in the order x, weight (norm); x (silu);
// table (embedding); the tests draw them again.  Needs a GPU: built and run once by make_golden_gpu.sh on a machine
// that has one; the committed ops_golden.json is what the tests read.
#include <cstdio>
#include <vector>

#include "lightllm/ops/elementwise.h"
#include "lightllm/ops/embedding.h"
#include "lightllm/ops/norm.h"
#include "lightllm/tensor.h"

using namespace lightllm;

static unsigned long long g_state = 88172645463325252ull;
static float next_float() {
    g_state ^= g_state << 13; g_state ^= g_state >> 7; g_state ^= g_state << 17;
    return (float)((g_state >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f;
}
static std::vector<float> draw(size_t n, float scale) {
    std::vector<float> v(n);
    for (auto& x : v) x = next_float() * scale;
    return v;
}
static Tensor to_gpu(const std::vector<int>& shape, const std::vector<float>& v) {
    Tensor t(shape, DType::F32, Device::CUDA);
    t.copy_from(v.data(), v.size() * sizeof(float));
    return t;
}
static void print_tensor(const char* name, const Tensor& t, bool last = false) {
    std::vector<float> v(t.numel());
    t.copy_to(v.data(), t.nbytes());
    printf("  \"%s\": [", name);
    for (size_t i = 0; i < v.size(); ++i) printf("%s%.9g", i ? ", " : "", v[i]);
    printf("]%s\n", last ? "" : ",");
}

int main() {
    const int R = 3, D = 40, N = 64, V = 11, E = 6;
    const float eps = 1e-5f;
    auto x = draw((size_t)R * D, 3.0f), w = draw(D, 1.0f);
    auto s = draw(N, 6.0f);
    auto table = draw((size_t)V * E, 1.0f);
    const std::vector<int> ids = {4, 0, 10, 4, 7};
    printf("{\"rows\": %d, \"width\": %d, \"eps\": %.9g, \"silu_n\": %d, \"vocab\": %d, \"embed_width\": %d, \"ids\": [4, 0, 10, 4, 7],\n",
           R, D, eps, N, V, E);
    print_tensor("rms_norm", ops::rms_norm(to_gpu({R, D}, x), to_gpu({D}, w), eps));
    print_tensor("silu", ops::silu(to_gpu({N}, s)));
    Tensor tid({(int)ids.size()}, DType::I32, Device::CUDA);
    tid.copy_from(ids.data(), ids.size() * sizeof(int));
    print_tensor("embedding", ops::embedding(tid, to_gpu({V, E}, table)), true);
    printf("}\n");
    return 0;
}
