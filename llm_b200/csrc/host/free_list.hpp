// Integers 0 .. count-1, handed out lowest first and taken back. Taking from an empty list,
// returning an item that is free or does not exist are errors, never silent.
#pragma once

#include <algorithm>
#include <functional>
#include <string>
#include <vector>

#include "host.hpp"

namespace llmh {

class FreeList {
public:
    FreeList(int count, std::string what) : count_(count), what_(std::move(what)), held_(count, 0) {
        free_.reserve(count);
        for (int i = 0; i < count; ++i) free_.push_back(i);          // ascending = a valid min-heap
    }
    int count() const { return count_; }
    int n_free() const { return (int)free_.size(); }
    int n_held() const { return count_ - (int)free_.size(); }
    bool is_held(int item) const { return item >= 0 && item < count_ && held_[item]; }
    const std::string& what() const { return what_; }

    int take() {
        if (free_.empty())
            throw Failure{LLMH_CACHE_FULL, "no free " + what_ + " left (all " + std::to_string(count_) + " are held)"};
        std::pop_heap(free_.begin(), free_.end(), std::greater<int>());
        int item = free_.back();
        free_.pop_back();
        if (held_[item])
            throw Failure{LLMH_INVARIANT, what_ + " " + std::to_string(item) + " was on the free list while held"};
        held_[item] = 1;
        return item;
    }
    void give_back(int item) {
        if (item < 0 || item >= count_)
            throw Failure{LLMH_INVARIANT, what_ + " " + std::to_string(item) + " does not exist"};
        if (!held_[item])
            throw Failure{LLMH_INVARIANT, what_ + " " + std::to_string(item) + " is freed twice"};
        held_[item] = 0;
        free_.push_back(item);
        std::push_heap(free_.begin(), free_.end(), std::greater<int>());
    }
    // Every item is either free once or held, never both or neither.
    void check() const {
        std::vector<int> seen(count_, 0);
        for (int item : free_) {
            if (item < 0 || item >= count_)
                throw Failure{LLMH_INVARIANT, "the free list of " + what_ + "s holds " + std::to_string(item)};
            ++seen[item];
        }
        for (int item = 0; item < count_; ++item)
            if (seen[item] + (held_[item] ? 1 : 0) != 1)
                throw Failure{LLMH_INVARIANT, what_ + " " + std::to_string(item) + ": on the free list " +
                                                  std::to_string(seen[item]) + " times, held=" +
                                                  (held_[item] ? "true" : "false")};
    }

private:
    int count_;
    std::string what_;
    std::vector<int> free_;          // min-heap
    std::vector<char> held_;
};

}  // namespace llmh
