// Bookkeeping of the paged cache: slots (one per live sequence, each with its own length),
// and per group of layers a pool of pages of 64 positions with, per slot, the list of its
// pages. Logical page i of a sequence is pages[i % ring]: a `full` group's ring covers the
// longest sequence, a `window` group's ring only the window plus one step. The device memory
// itself belongs to the caller; this class decides which page holds what.
//
// MythEclipse/llm keeps one cache per session with one length (apps/engine/src/model.rs:351-436);
// here one cache serves a batch.
#pragma once

#include <cstdint>
#include <vector>

#include "../plan.h"
#include "free_list.hpp"

namespace llmh {

constexpr int PAGE = LLMB_PAGE;

inline int pages_for(long long positions) { return (int)((positions + PAGE - 1) / PAGE); }

struct Group {
    int window;                                   // 0: keeps every position
    int ring_pages;                               // logical pages per sequence
    FreeList pool;
    std::vector<std::vector<int>> slot_pages;     // per slot: its physical pages, in logical order
    std::vector<int32_t> table;                   // [slots, ring_pages], mirrors slot_pages, 0 elsewhere
    Group(int window_, int ring, int n_pages, int max_slots)
        : window(window_), ring_pages(ring),
          pool(n_pages, std::string("page of the ") + (window_ ? "window" : "full") + " group"),
          slot_pages(max_slots), table((size_t)max_slots * ring, 0) {}
    const char* kind() const { return window ? "window" : "full"; }
};

class Cache {
public:
    Cache(long long max_tokens, int max_seq_len, int max_slots, int step_tokens, const std::vector<int>& windows);

    int acquire();
    void release(int slot);
    void reserve(int slot, long long new_length);
    void reserve_many(int n, const int* slots, const long long* new_lengths);
    bool can_hold(int n, const long long* lengths) const;
    long long held_tokens() const;
    void check() const;

    void require_held(int slot) const;
    int length(int slot) const { return lengths_[slot]; }
    void set_length(int slot, int length) { lengths_[slot] = length; }

    int max_seq_len, max_slots, step_tokens;
    long long max_tokens;
    FreeList slots;
    std::vector<Group> groups;

private:
    std::vector<int> lengths_;
};

}  // namespace llmh
