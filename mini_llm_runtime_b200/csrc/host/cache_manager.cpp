// Host-side cache manager: pages of keys and values, a block table per request
// and per group, and slots for per-request state of fixed size.  No CUDA here.
//
// The reference keeps the same ledger in src/minillm/cuda/page_table.cpp:32-117
// (free-id stack, prepare -> begin_execution -> commit, clear on finish) and
// src/minillm/cuda/batch_state.cpp:19-64 (per-sequence lengths); both know one
// kind of layer.  Here layers are put into GROUPS by what they need from the cache:
// a group keeps all keys (window 0) or only the last `window` keys.  Each group has
// its own pool of page ids and its own block table; a page id of a group is valid
// for every layer of that group.  Pages go back to the group's free stack when the
// request ends, or, in a window group, as soon as every token of the page lies
// before the window of the next query.  Freed pages are reused last-in first-out.
//
// A step is a transaction: prepare() plans the growth of several requests and
// takes the pages, commit() publishes lengths and releases pages the windows have
// passed, discard() undoes prepare().  prepare() either succeeds for the whole
// batch or changes nothing.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr int kOk = 0;
constexpr int kBadArgument = 1;
constexpr int kNoPages = 2;
constexpr int kNoSlot = 3;
constexpr int kBadPhase = 4;
constexpr int kTooLong = 5;

struct Group {
    int window = 0;                 // 0: every key is kept
    int num_pages = 0;
    std::vector<int32_t> free_ids;  // stack; back() is handed out next
    std::vector<int32_t> table;     // [max_requests][max_blocks], -1 = no page
    std::vector<int32_t> first_block;  // [max_requests]: blocks below were released
};

struct Planned {
    int slot;
    int new_tokens;
};

struct Cache {
    int page_size = 0;
    int max_requests = 0;
    int max_blocks = 0;
    std::vector<Group> groups;
    std::vector<int32_t> length;      // [max_requests] committed tokens
    std::vector<uint8_t> open;        // [max_requests]
    std::vector<int32_t> free_slots;  // stack
    std::vector<Planned> planned;     // requests of the prepared step
    std::vector<int32_t> journal_group, journal_slot, journal_block;  // pages taken by prepare()
    bool prepared = false;
    std::string error;

    int blocks_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
    int fail(int code, std::string message) {
        error = std::move(message);
        return code;
    }
};

// First block that a query at position `next_position` can still read in a group.
int first_needed_block(const Cache& c, const Group& g, int next_position) {
    if (g.window == 0) return 0;
    const int lowest_key = next_position - g.window + 1;
    return lowest_key <= 0 ? 0 : lowest_key / c.page_size;
}

}  // namespace

extern "C" {

void* mlr_cache_create(int n_groups, const int* windows, const int* pages, int page_size,
                       int max_requests, int max_model_len) {
    if (n_groups < 0 || page_size <= 0 || max_requests <= 0 || max_model_len <= 0) return nullptr;
    auto* c = new Cache();
    c->page_size = page_size;
    c->max_requests = max_requests;
    c->max_blocks = (max_model_len + page_size - 1) / page_size;
    c->groups.resize(n_groups);
    for (int g = 0; g < n_groups; ++g) {
        if (windows[g] < 0 || pages[g] <= 0) {
            delete c;
            return nullptr;
        }
        auto& group = c->groups[g];
        group.window = windows[g];
        group.num_pages = pages[g];
        group.free_ids.reserve(pages[g]);
        for (int id = pages[g] - 1; id >= 0; --id) group.free_ids.push_back(id);
        group.table.assign(static_cast<size_t>(max_requests) * c->max_blocks, -1);
        group.first_block.assign(max_requests, 0);
    }
    c->length.assign(max_requests, 0);
    c->open.assign(max_requests, 0);
    for (int s = max_requests - 1; s >= 0; --s) c->free_slots.push_back(s);
    const size_t journal = static_cast<size_t>(max_requests) * c->max_blocks;
    c->journal_group.reserve(journal);
    c->journal_slot.reserve(journal);
    c->journal_block.reserve(journal);
    c->planned.reserve(max_requests);
    return c;
}

void mlr_cache_destroy(void* handle) { delete static_cast<Cache*>(handle); }

const char* mlr_cache_error(void* handle) { return static_cast<Cache*>(handle)->error.c_str(); }

int mlr_cache_max_blocks(void* handle) { return static_cast<Cache*>(handle)->max_blocks; }

// Takes a request slot; its state slot has the same id.  *slot = -1 if none is free.
int mlr_cache_open(void* handle, int* slot) {
    auto* c = static_cast<Cache*>(handle);
    if (c->prepared) return c->fail(kBadPhase, "open() while a step is prepared");
    if (c->free_slots.empty()) {
        *slot = -1;
        return c->fail(kNoSlot, "no request slot is free");
    }
    *slot = c->free_slots.back();
    c->free_slots.pop_back();
    c->open[*slot] = 1;
    c->length[*slot] = 0;
    for (auto& g : c->groups) g.first_block[*slot] = 0;
    return kOk;
}

// Ends a request: every page it holds in every group goes back, then the slot.
int mlr_cache_close(void* handle, int slot) {
    auto* c = static_cast<Cache*>(handle);
    if (c->prepared) return c->fail(kBadPhase, "close() while a step is prepared");
    if (slot < 0 || slot >= c->max_requests || !c->open[slot])
        return c->fail(kBadArgument, "close() of a slot that is not open: " + std::to_string(slot));
    for (auto& g : c->groups) {
        int32_t* row = g.table.data() + static_cast<size_t>(slot) * c->max_blocks;
        for (int b = 0; b < c->max_blocks; ++b) {
            if (row[b] >= 0) {
                g.free_ids.push_back(row[b]);
                row[b] = -1;
            }
        }
        g.first_block[slot] = 0;
    }
    c->length[slot] = 0;
    c->open[slot] = 0;
    c->free_slots.push_back(slot);
    return kOk;
}

int mlr_cache_length(void* handle, int slot) {
    auto* c = static_cast<Cache*>(handle);
    if (slot < 0 || slot >= c->max_requests || !c->open[slot]) return -1;
    return c->length[slot];
}

int mlr_cache_free_pages(void* handle, int group) {
    auto* c = static_cast<Cache*>(handle);
    if (group < 0 || group >= static_cast<int>(c->groups.size())) return -1;
    return static_cast<int>(c->groups[group].free_ids.size());
}

int mlr_cache_free_slots(void* handle) { return static_cast<int>(static_cast<Cache*>(handle)->free_slots.size()); }

// Pages a request of `total_tokens` can hold at most at one time in `group`, when no
// step appends more than `max_step_tokens` tokens to it.  Used for admission credits.
int mlr_cache_peak_pages(void* handle, int group, int total_tokens, int max_step_tokens) {
    auto* c = static_cast<Cache*>(handle);
    if (group < 0 || group >= static_cast<int>(c->groups.size()) || total_tokens < 0) return -1;
    const auto& g = c->groups[group];
    const int all = c->blocks_for(total_tokens);
    if (g.window == 0) return all;
    // Before a step the oldest kept key is at most window-1 behind the next position; the
    // step adds up to max_step_tokens; both ends may straddle a page.
    const int span = g.window - 1 + (max_step_tokens > 0 ? max_step_tokens : 1);
    const int windowed = (span + c->page_size - 1) / c->page_size + 1;
    return windowed < all ? windowed : all;
}

// Plans a step: request slots[i] grows by new_tokens[i].  Takes the pages of every group
// or, if any group lacks pages, takes none and returns kNoPages.
int mlr_cache_prepare(void* handle, int n, const int* slots, const int* new_tokens) {
    auto* c = static_cast<Cache*>(handle);
    if (c->prepared) return c->fail(kBadPhase, "prepare() while a step is already prepared");
    if (n <= 0) return c->fail(kBadArgument, "prepare() of an empty step");
    for (int i = 0; i < n; ++i) {
        const int s = slots[i];
        if (s < 0 || s >= c->max_requests || !c->open[s])
            return c->fail(kBadArgument, "prepare() names a slot that is not open: " + std::to_string(s));
        if (new_tokens[i] <= 0)
            return c->fail(kBadArgument, "prepare() with a non-positive token count for slot " + std::to_string(s));
        for (int j = 0; j < i; ++j)
            if (slots[j] == s) return c->fail(kBadArgument, "prepare() names slot " + std::to_string(s) + " twice");
        if (c->blocks_for(c->length[s] + new_tokens[i]) > c->max_blocks)
            return c->fail(kTooLong, "request in slot " + std::to_string(s) + " would exceed the maximum length");
    }
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        const auto& g = c->groups[gi];
        size_t needed = 0;
        for (int i = 0; i < n; ++i) {
            const int s = slots[i];
            const int32_t* row = g.table.data() + static_cast<size_t>(s) * c->max_blocks;
            const int from = std::max(c->blocks_for(c->length[s]), first_needed_block(*c, g, c->length[s]));
            const int to = c->blocks_for(c->length[s] + new_tokens[i]);
            for (int b = from; b < to; ++b) needed += row[b] < 0 ? 1 : 0;
        }
        if (needed > g.free_ids.size())
            return c->fail(kNoPages, "group " + std::to_string(gi) + " needs " + std::to_string(needed) +
                                         " pages, " + std::to_string(g.free_ids.size()) + " are free");
    }
    c->journal_group.clear();
    c->journal_slot.clear();
    c->journal_block.clear();
    c->planned.clear();
    for (int i = 0; i < n; ++i) c->planned.push_back({slots[i], new_tokens[i]});
    for (size_t gi = 0; gi < c->groups.size(); ++gi) {
        auto& g = c->groups[gi];
        for (int i = 0; i < n; ++i) {
            const int s = slots[i];
            int32_t* row = g.table.data() + static_cast<size_t>(s) * c->max_blocks;
            const int from = std::max(c->blocks_for(c->length[s]), first_needed_block(*c, g, c->length[s]));
            const int to = c->blocks_for(c->length[s] + new_tokens[i]);
            for (int b = from; b < to; ++b) {
                if (row[b] >= 0) continue;
                row[b] = g.free_ids.back();
                g.free_ids.pop_back();
                c->journal_group.push_back(static_cast<int32_t>(gi));
                c->journal_slot.push_back(s);
                c->journal_block.push_back(b);
            }
        }
    }
    c->prepared = true;
    return kOk;
}

// Publishes the prepared step: lengths advance, and window groups give back the pages
// that no later query can read.
int mlr_cache_commit(void* handle) {
    auto* c = static_cast<Cache*>(handle);
    if (!c->prepared) return c->fail(kBadPhase, "commit() without a prepared step");
    for (const auto& p : c->planned) {
        c->length[p.slot] += p.new_tokens;
        for (auto& g : c->groups) {
            if (g.window == 0) continue;
            const int keep_from = first_needed_block(*c, g, c->length[p.slot]);
            int32_t* row = g.table.data() + static_cast<size_t>(p.slot) * c->max_blocks;
            for (int b = g.first_block[p.slot]; b < keep_from; ++b) {
                if (row[b] >= 0) {
                    g.free_ids.push_back(row[b]);
                    row[b] = -1;
                }
            }
            if (keep_from > g.first_block[p.slot]) g.first_block[p.slot] = keep_from;
        }
    }
    c->planned.clear();
    c->prepared = false;
    return kOk;
}

// Undoes prepare(): the pages it took go back in reverse order, lengths stay.
int mlr_cache_discard(void* handle) {
    auto* c = static_cast<Cache*>(handle);
    if (!c->prepared) return c->fail(kBadPhase, "discard() without a prepared step");
    for (size_t i = c->journal_group.size(); i-- > 0;) {
        auto& g = c->groups[c->journal_group[i]];
        int32_t* cell = g.table.data() + static_cast<size_t>(c->journal_slot[i]) * c->max_blocks + c->journal_block[i];
        g.free_ids.push_back(*cell);
        *cell = -1;
    }
    c->planned.clear();
    c->prepared = false;
    return kOk;
}

// Copies the block-table rows of `slots` in `group` into out[n][row_stride] (first
// `columns` entries of each row; row_stride >= columns).
int mlr_cache_fill_table(void* handle, int group, int n, const int* slots, int columns,
                         int32_t* out, int row_stride) {
    auto* c = static_cast<Cache*>(handle);
    if (group < 0 || group >= static_cast<int>(c->groups.size()) || columns < 0 ||
        columns > c->max_blocks || row_stride < columns)
        return c->fail(kBadArgument, "fill_table() with a bad group or width");
    const auto& g = c->groups[group];
    for (int i = 0; i < n; ++i) {
        const int s = slots[i];
        if (s < 0 || s >= c->max_requests || !c->open[s])
            return c->fail(kBadArgument, "fill_table() names a slot that is not open: " + std::to_string(s));
        std::memcpy(out + static_cast<size_t>(i) * row_stride,
                    g.table.data() + static_cast<size_t>(s) * c->max_blocks, sizeof(int32_t) * columns);
    }
    return kOk;
}

}  // extern "C"
