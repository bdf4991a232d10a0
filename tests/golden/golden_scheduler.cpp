// Drives the reference's DecodeFirstScheduler (src/engine/scheduler.cpp:34-73) and prints every
// step's entries.  The chunk size equals the token budget, so that the reference never cuts one
// request into two entries of the same step (its engine mishandles those).
#include <cstdio>
#include <vector>

#include "lightllm/engine/scheduler.h"

using namespace lightllm::engine;

int main() {
    const int chunk = 24, budget = 24;
    DecodeFirstScheduler s(chunk, budget, 999);
    const int prompts[] = {5, 40, 17, 3, 30};
    const int max_new[] = {4, 3, 6, 2, 3};
    for (int i = 0; i < 5; ++i) {
        Request r;
        r.id = i;
        r.prompt_tokens.assign(prompts[i], 1);
        r.max_new_tokens = max_new[i];
        s.add_request(r);
    }
    // The engine's part, imitated: a request whose prompt completed in a step owns one token after it
    // and one more after each decode entry; it finishes at max_new tokens.
    std::vector<int> generated(5, 0), prefilled(5, 0);
    printf("{\"chunk_size\": %d, \"max_batch_tokens\": %d, \"prompts\": [5, 40, 17, 3, 30], \"max_new\": [4, 3, 6, 2, 3], \"steps\": [\n", chunk, budget);
    bool first = true;
    for (int step = 0; step < 64 && s.num_active() > 0; ++step) {
        ScheduleStep st = s.step();
        if (st.empty()) break;
        printf("%s [", first ? "" : ",\n");
        first = false;
        for (size_t i = 0; i < st.entries.size(); ++i) {
            const auto& e = st.entries[i];
            printf("%s[%d, %d, %d]", i ? ", " : "", e.request_idx, e.num_tokens, e.is_prefill ? 1 : 0);
        }
        printf("]");
        for (const auto& e : st.entries) {
            int id = e.request_idx;
            if (e.is_prefill) {
                prefilled[id] += e.num_tokens;
                if (prefilled[id] == prompts[id]) generated[id] = 1;
            } else {
                generated[id] += 1;
            }
            if (generated[id] >= max_new[id]) s.finish_request(id);
        }
    }
    printf("\n]}\n");
    return 0;
}
