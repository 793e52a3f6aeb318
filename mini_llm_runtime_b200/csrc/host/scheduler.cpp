// Batch planner: which request gets how many tokens in the next step.
//
// The policy is the reference's schedule_batch (src/scheduler.cpp:11-49): under a
// token budget, every decoding request first gets one token (policy "mixed", or
// when no prompt is pending), then each request that still has prompt tokens gets
// min(budget left, prompt left, prefill_chunk) in order, until the budget is spent.
// Policy "prefill_first" leaves decodes out while any prompt is pending.  The
// reference orders requests by priority with aging; here the order is the arrival
// order alone (priorities, deadlines and aging belong to its server, which is not
// part of this engine).
#include <algorithm>
#include <cstdint>
#include <vector>

namespace {
struct Item {
    int64_t key;
    int32_t prefill_remaining;
    int64_t order;
};
}  // namespace

extern "C" {

// policy: 0 = mixed, 1 = prefill_first.  Writes up to n slices; returns their count,
// or -1 on a bad argument.  out_totals[0] = prefill tokens, out_totals[1] = decode tokens.
int mlr_schedule_batch(int n, const int64_t* keys, const int32_t* prefill_remaining,
                       const int64_t* order, int batch_tokens, int prefill_chunk, int policy,
                       int64_t* out_keys, int32_t* out_tokens, int32_t* out_is_prefill,
                       int32_t* out_totals) {
    if (n < 0 || batch_tokens <= 0 || prefill_chunk <= 0 || (policy != 0 && policy != 1)) return -1;
    std::vector<Item> prefill, decode;
    for (int i = 0; i < n; ++i) {
        if (prefill_remaining[i] < 0) return -1;
        (prefill_remaining[i] ? prefill : decode).push_back({keys[i], prefill_remaining[i], order[i]});
    }
    const auto earlier = [](const Item& a, const Item& b) { return a.order < b.order; };
    std::stable_sort(prefill.begin(), prefill.end(), earlier);
    std::stable_sort(decode.begin(), decode.end(), earlier);
    int remaining = batch_tokens;
    int count = 0;
    out_totals[0] = out_totals[1] = 0;
    if (policy == 0 || prefill.empty()) {
        for (const auto& item : decode) {
            if (remaining == 0) break;
            out_keys[count] = item.key;
            out_tokens[count] = 1;
            out_is_prefill[count] = 0;
            ++count;
            ++out_totals[1];
            --remaining;
        }
    }
    for (const auto& item : prefill) {
        const int take = std::min({remaining, item.prefill_remaining, prefill_chunk});
        if (take == 0) break;
        out_keys[count] = item.key;
        out_tokens[count] = take;
        out_is_prefill[count] = 1;
        ++count;
        out_totals[0] += take;
        remaining -= take;
    }
    return count;
}

}  // extern "C"
