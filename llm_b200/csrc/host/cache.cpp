#include "cache.hpp"

#include <algorithm>

namespace llmh {

Failure& last_failure() {
    static thread_local Failure failure{LLMH_OK, ""};
    return failure;
}

Cache::Cache(long long max_tokens_, int max_seq_len_, int max_slots_, int step_tokens_, const std::vector<int>& windows)
    : max_seq_len(max_seq_len_), max_slots(max_slots_), step_tokens(step_tokens_ > 0 ? step_tokens_ : max_seq_len_),
      max_tokens((std::max<long long>(max_tokens_, PAGE) + PAGE - 1) / PAGE * PAGE), slots(max_slots_, "slot"),
      lengths_(max_slots_, 0) {
    if (max_slots_ < 1 || max_seq_len_ < 1) throw Failure{LLMH_FORMAT, "a cache needs at least one slot and one position"};
    int total_pages = (int)(max_tokens / PAGE);
    int seq_pages = pages_for(max_seq_len);
    groups.reserve(windows.size());
    for (int window : windows) {
        int ring = seq_pages, n_pages = total_pages;
        if (window > 0) {
            // a step writes up to step_tokens new positions before attention runs, and the oldest
            // query of the step still needs the window before it
            ring = std::min(seq_pages, (window + step_tokens - 2) / PAGE + 2);
            n_pages = (int)std::min<long long>(total_pages, (long long)max_slots * ring);
        }
        groups.emplace_back(window, ring, n_pages, max_slots);
    }
}

void Cache::require_held(int slot) const {
    if (!slots.is_held(slot)) throw Failure{LLMH_INVARIANT, "slot " + std::to_string(slot) + " is not held"};
}

int Cache::acquire() {
    int slot = slots.take();
    lengths_[slot] = 0;
    for (Group& group : groups) {
        group.slot_pages[slot].clear();
        std::fill_n(group.table.begin() + (size_t)slot * group.ring_pages, group.ring_pages, 0);
    }
    return slot;
}

void Cache::release(int slot) {
    require_held(slot);
    for (Group& group : groups) {
        for (int page : group.slot_pages[slot]) group.pool.give_back(page);
        group.slot_pages[slot].clear();
    }
    lengths_[slot] = 0;
    slots.give_back(slot);
}

void Cache::reserve(int slot, long long new_length) {
    require_held(slot);
    if (new_length > max_seq_len) throw Failure{LLMH_CONTEXT_FULL, "", new_length, max_seq_len};
    std::vector<int> needs;
    for (Group& group : groups) {
        int want = std::min(pages_for(new_length), group.ring_pages);
        int extra = want - (int)group.slot_pages[slot].size();
        if (extra > group.pool.n_free())
            throw Failure{LLMH_CACHE_FULL, std::string("the ") + group.kind() + " group has " +
                                               std::to_string(group.pool.n_free()) + " free pages, slot " +
                                               std::to_string(slot) + " needs " + std::to_string(extra) +
                                               " more for " + std::to_string(new_length) + " positions"};
        needs.push_back(extra);
    }
    for (size_t g = 0; g < groups.size(); ++g) {
        Group& group = groups[g];
        for (int i = 0; i < needs[g]; ++i) {
            int page = group.pool.take();
            group.table[(size_t)slot * group.ring_pages + group.slot_pages[slot].size()] = page;
            group.slot_pages[slot].push_back(page);
        }
    }
}

void Cache::reserve_many(int n, const int* which, const long long* new_lengths) {
    std::vector<long long> needs(groups.size(), 0);
    for (int i = 0; i < n; ++i) {
        require_held(which[i]);
        if (new_lengths[i] > max_seq_len) throw Failure{LLMH_CONTEXT_FULL, "", new_lengths[i], max_seq_len};
        for (size_t g = 0; g < groups.size(); ++g) {
            int want = std::min(pages_for(new_lengths[i]), groups[g].ring_pages);
            needs[g] += std::max(want - (int)groups[g].slot_pages[which[i]].size(), 0);
        }
    }
    for (size_t g = 0; g < groups.size(); ++g)
        if (needs[g] > groups[g].pool.n_free())
            throw Failure{LLMH_CACHE_FULL, std::string("the ") + groups[g].kind() + " group has " +
                                               std::to_string(groups[g].pool.n_free()) +
                                               " free pages, this step needs " + std::to_string(needs[g])};
    for (int i = 0; i < n; ++i) reserve(which[i], new_lengths[i]);
}

bool Cache::can_hold(int n, const long long* lengths) const {
    if (n > slots.n_free()) return false;
    for (int i = 0; i < n; ++i)
        if (lengths[i] > max_seq_len) return false;
    for (const Group& group : groups) {
        long long pages = 0;
        for (int i = 0; i < n; ++i) pages += std::min(pages_for(lengths[i]), group.ring_pages);
        if (pages > group.pool.n_free()) return false;
    }
    return true;
}

long long Cache::held_tokens() const {
    long long total = 0;
    for (int slot = 0; slot < max_slots; ++slot)
        if (slots.is_held(slot)) total += (long long)pages_for(lengths_[slot]) * PAGE;
    return total;
}

// No slot or page lost, held twice, or shared between two slots; the table mirrors the lists.
void Cache::check() const {
    slots.check();
    for (const Group& group : groups) {
        group.pool.check();
        std::vector<int> owner(group.pool.count(), -1);
        int owned = 0;
        for (int slot = 0; slot < max_slots; ++slot) {
            const std::vector<int>& pages = group.slot_pages[slot];
            if (!pages.empty() && !slots.is_held(slot))
                throw Failure{LLMH_INVARIANT, "freed slot " + std::to_string(slot) + " still lists pages"};
            for (size_t i = 0; i < pages.size(); ++i) {
                int page = pages[i];
                if (page < 0 || page >= group.pool.count() || !group.pool.is_held(page))
                    throw Failure{LLMH_INVARIANT, "slot " + std::to_string(slot) + " lists page " +
                                                      std::to_string(page) + " that is on the free list"};
                if (owner[page] >= 0)
                    throw Failure{LLMH_INVARIANT, "page " + std::to_string(page) + " is held by slots " +
                                                      std::to_string(owner[page]) + " and " + std::to_string(slot)};
                if (group.table[(size_t)slot * group.ring_pages + i] != page)
                    throw Failure{LLMH_INVARIANT, "the page table of slot " + std::to_string(slot) +
                                                      " does not list its page " + std::to_string(i)};
                owner[page] = slot;
                ++owned;
            }
        }
        if (owned != group.pool.n_held())
            throw Failure{LLMH_INVARIANT, std::to_string(group.pool.n_held() - owned) + " pages are held by no slot"};
    }
}

}  // namespace llmh

using namespace llmh;

// ------------------------------------------------------------------------------------ C boundary

// The constants of plan.h for callers that cannot include it: 0 page, 1 gated block, 2 largest head size.
LLMH_EXPORT int llmh_plan_constant(int which) {
    switch (which) {
        case 0: return LLMB_PAGE;
        case 1: return LLMB_GLU_BLOCK;
        case 2: return LLMB_MAX_HEAD_DIM;
        default: return -1;
    }
}

LLMH_EXPORT const char* llmh_last_error() { return last_failure().text.c_str(); }
LLMH_EXPORT void llmh_last_error_numbers(long long* first, long long* second) {
    *first = last_failure().first;
    *second = last_failure().second;
}

// A free list of its own (the cache's lists are reached through llmh_cache_list).
LLMH_EXPORT int llmh_free_list_create(int count, const char* what, void** out) {
    return guarded([&] {
        if (count < 0) throw Failure{LLMH_FORMAT, "a free list cannot hold a negative count"};
        *out = new FreeList(count, what);
    });
}
LLMH_EXPORT void llmh_free_list_destroy(void* list) { delete static_cast<FreeList*>(list); }
LLMH_EXPORT int llmh_free_list_take(void* list, int* item) {
    return guarded([&] { *item = static_cast<FreeList*>(list)->take(); });
}
LLMH_EXPORT int llmh_free_list_give_back(void* list, int item) {
    return guarded([&] { static_cast<FreeList*>(list)->give_back(item); });
}
LLMH_EXPORT int llmh_free_list_is_held(void* list, int item) { return static_cast<FreeList*>(list)->is_held(item) ? 1 : 0; }
LLMH_EXPORT void llmh_free_list_counts(void* list, int* count, int* n_free) {
    *count = static_cast<FreeList*>(list)->count();
    *n_free = static_cast<FreeList*>(list)->n_free();
}
LLMH_EXPORT int llmh_free_list_check(void* list) {
    return guarded([&] { static_cast<FreeList*>(list)->check(); });
}

LLMH_EXPORT int llmh_cache_create(long long max_tokens, int max_seq_len, int max_slots, int step_tokens, int n_groups,
                                  const int* windows, void** out) {
    return guarded([&] { *out = new Cache(max_tokens, max_seq_len, max_slots, step_tokens, std::vector<int>(windows, windows + n_groups)); });
}
LLMH_EXPORT void llmh_cache_destroy(void* cache) { delete static_cast<Cache*>(cache); }
// which = -1: the slots; which = g: the page pool of group g. The list stays the cache's.
LLMH_EXPORT void* llmh_cache_list(void* cache, int which) {
    Cache* c = static_cast<Cache*>(cache);
    if (which < 0) return &c->slots;
    return which < (int)c->groups.size() ? &c->groups[which].pool : nullptr;
}
LLMH_EXPORT void llmh_cache_group_info(void* cache, int group, int* ring_pages, int* n_pages) {
    const Group& g = static_cast<Cache*>(cache)->groups[group];
    *ring_pages = g.ring_pages;
    *n_pages = g.pool.count();
}
LLMH_EXPORT long long llmh_cache_max_tokens(void* cache) { return static_cast<Cache*>(cache)->max_tokens; }
LLMH_EXPORT int llmh_cache_acquire(void* cache, int* slot) {
    return guarded([&] { *slot = static_cast<Cache*>(cache)->acquire(); });
}
LLMH_EXPORT int llmh_cache_release(void* cache, int slot) {
    return guarded([&] { static_cast<Cache*>(cache)->release(slot); });
}
LLMH_EXPORT int llmh_cache_reserve(void* cache, int slot, long long new_length) {
    return guarded([&] { static_cast<Cache*>(cache)->reserve(slot, new_length); });
}
LLMH_EXPORT int llmh_cache_reserve_many(void* cache, int n, const int* slots, const long long* new_lengths) {
    return guarded([&] { static_cast<Cache*>(cache)->reserve_many(n, slots, new_lengths); });
}
LLMH_EXPORT int llmh_cache_can_hold(void* cache, int n, const long long* lengths) {
    return static_cast<Cache*>(cache)->can_hold(n, lengths) ? 1 : 0;
}
LLMH_EXPORT int llmh_cache_length(void* cache, int slot, int* length) {
    return guarded([&] {
        Cache* c = static_cast<Cache*>(cache);
        if (slot < 0 || slot >= c->max_slots) throw Failure{LLMH_INVARIANT, "slot " + std::to_string(slot) + " does not exist"};
        *length = c->length(slot);
    });
}
LLMH_EXPORT int llmh_cache_set_length(void* cache, int slot, int length) {
    return guarded([&] {
        Cache* c = static_cast<Cache*>(cache);
        if (slot < 0 || slot >= c->max_slots) throw Failure{LLMH_INVARIANT, "slot " + std::to_string(slot) + " does not exist"};
        c->set_length(slot, length);
    });
}
LLMH_EXPORT long long llmh_cache_held_tokens(void* cache) { return static_cast<Cache*>(cache)->held_tokens(); }
// The pages of a slot in one group: writes up to `capacity` of them, returns their number in *count.
LLMH_EXPORT int llmh_cache_slot_pages(void* cache, int group, int slot, int* pages, int capacity, int* count) {
    return guarded([&] {
        Cache* c = static_cast<Cache*>(cache);
        if (group < 0 || group >= (int)c->groups.size() || slot < 0 || slot >= c->max_slots)
            throw Failure{LLMH_INVARIANT, "no such group or slot"};
        const std::vector<int>& list = c->groups[group].slot_pages[slot];
        *count = (int)list.size();
        for (int i = 0; i < std::min(capacity, *count); ++i) pages[i] = list[i];
    });
}
// Rows of the page table, one per slot of `slots`: int32 [n, ring_pages], 0 where no page is yet.
LLMH_EXPORT int llmh_cache_table_rows(void* cache, int group, int n, const int* slots, int32_t* out) {
    return guarded([&] {
        Cache* c = static_cast<Cache*>(cache);
        if (group < 0 || group >= (int)c->groups.size()) throw Failure{LLMH_INVARIANT, "no such group"};
        const Group& g = c->groups[group];
        for (int i = 0; i < n; ++i) {
            if (slots[i] < 0 || slots[i] >= c->max_slots) throw Failure{LLMH_INVARIANT, "slot " + std::to_string(slots[i]) + " does not exist"};
            std::copy_n(g.table.begin() + (size_t)slots[i] * g.ring_pages, g.ring_pages, out + (size_t)i * g.ring_pages);
        }
    });
}
LLMH_EXPORT int llmh_cache_check(void* cache) {
    return guarded([&] { static_cast<Cache*>(cache)->check(); });
}
