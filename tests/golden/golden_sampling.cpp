// Drives the reference's sampler (src/ops/sampling.cpp) on a fixed row of logits and prints, for
// several parameter sets, how often each token was drawn over many seeds.
#include <cstdio>
#include <random>
#include <vector>

#include "lightllm/ops/sampling.h"

int main() {
    using namespace lightllm::ops;
    const int V = 24;
    std::vector<float> logits(V);
    for (int i = 0; i < V; ++i) logits[i] = 2.5f * std::sin(0.9f * i) + 0.1f * i - (i % 5 == 0 ? 1.5f : 0.0f);
    logits[7] = logits[3];  // a tie
    struct P { float t; int k; float p; float m; };
    const P sets[] = {{0.0f, 0, 1.0f, 0.0f}, {1.0f, 0, 1.0f, 0.0f}, {0.7f, 5, 1.0f, 0.0f}, {1.5f, 0, 0.8f, 0.0f},
                      {1.0f, 0, 1.0f, 0.1f}, {0.8f, 8, 0.9f, 0.05f}, {1.0f, 1, 1.0f, 0.0f}};
    const int draws = 40000;
    printf("{\"logits\": [");
    for (int i = 0; i < V; ++i) printf("%s%.9g", i ? ", " : "", logits[i]);
    printf("], \"draws\": %d, \"cases\": [\n", draws);
    int n = sizeof(sets) / sizeof(sets[0]);
    for (int c = 0; c < n; ++c) {
        SamplingParams sp;
        sp.temperature = sets[c].t; sp.top_k = sets[c].k; sp.top_p = sets[c].p; sp.min_p = sets[c].m;
        std::vector<int> hist(V, 0);
        std::mt19937 rng(1234 + c);
        for (int d = 0; d < draws; ++d) hist[sample(logits.data(), V, sp, rng, nullptr)]++;
        printf(" {\"temperature\": %.9g, \"top_k\": %d, \"top_p\": %.9g, \"min_p\": %.9g, \"hist\": [", sets[c].t,
               sets[c].k, sets[c].p, sets[c].m);
        for (int i = 0; i < V; ++i) printf("%s%d", i ? ", " : "", hist[i]);
        printf("]}%s\n", c + 1 < n ? "," : "");
    }
    printf("]}\n");
    return 0;
}
