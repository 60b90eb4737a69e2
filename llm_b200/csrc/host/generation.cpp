// The decisions of the generation loop for one batch of sequences that started together.
// Per sequence the order is that of MythEclipse/llm's loop (apps/engine/src/generate.rs:78-127):
// sample from the current logits; a stop token ends the sequence without being emitted or fed;
// else emit, stop if the context is full or the limit of new tokens is reached, and feed the token
// for the next logits. Here every live sequence advances by one token per step, and the next step
// is planned before the sampled ids are known (everyone whose limits allow one more token goes
// on; a sequence that turns out to have drawn a stop token drops that step's result).
//
// The caller owns slots, kernels, timing and callbacks; this class only says who is live, who
// leaves and why. Reasons: 0 stop token ("eos"), 1 max_tokens, 2 cancelled, 3 context_full.
#include <algorithm>
#include <vector>

#include "host.hpp"

using namespace llmh;

namespace {

enum Reason { STOP_TOKEN = 0, MAX_TOKENS = 1, CANCELLED = 2, CONTEXT_FULL = 3 };

struct Sequence {
    int max_tokens = 0;
    int emitted = 0;
    std::vector<int> stop_tokens;
    bool finished = false;
};

class Generation {
public:
    Generation(int n, const int* max_tokens, const int* stop_counts, const int* stops, int max_seq_len)
        : max_seq_len_(max_seq_len), sequences_(n) {
        int at = 0;
        for (int i = 0; i < n; ++i) {
            sequences_[i].max_tokens = std::max(max_tokens[i], 0);
            sequences_[i].stop_tokens.assign(stops + at, stops + at + stop_counts[i]);
            at += stop_counts[i];
            live_.push_back(i);
        }
    }

    const std::vector<int>& live() const { return live_; }

    // Sequences that may not emit anything more leave before sampling. kept_rows: the rows of the
    // live list (as it was) that stay, in order.
    void drop_exhausted(std::vector<int>* kept_rows, std::vector<int>* finished) {
        std::vector<int> kept;
        for (size_t row = 0; row < live_.size(); ++row) {
            Sequence& s = sequences_[live_[row]];
            if (s.emitted < s.max_tokens) {
                kept_rows->push_back((int)row);
                kept.push_back(live_[row]);
            } else {
                s.finished = true;
                finished->push_back(live_[row]);
            }
        }
        live_ = kept;
    }

    // Who goes on after the token being sampled now, whatever it is (unless it is a stop token):
    // lengths[row] is the sequence's length in the cache before that token is fed.
    void plan_onward(const int* lengths, std::vector<int>* onward_rows) {
        room_.assign(live_.size(), 0);
        onward_.clear();
        for (size_t row = 0; row < live_.size(); ++row) {
            const Sequence& s = sequences_[live_[row]];
            room_[row] = lengths[row] < max_seq_len_;
            if (s.emitted + 1 < s.max_tokens && room_[row]) onward_.push_back((int)row);
        }
        *onward_rows = onward_;
    }

    // The sampled ids of the live rows. emitted[row] = 1 if the token counts as output; finished
    // sequences with their reasons; going_rows: for every sequence that stays live, its index in
    // the list that plan_onward returned.
    void take_tokens(const int* tokens, int* emitted, std::vector<std::pair<int, int>>* finished,
                     std::vector<int>* going_rows) {
        if (room_.size() != live_.size()) throw Failure{LLMH_INVARIANT, "take_tokens without plan_onward"};
        std::vector<int> going;
        for (size_t row = 0; row < live_.size(); ++row) {
            int index = live_[row];
            Sequence& s = sequences_[index];
            emitted[row] = 0;
            if (std::find(s.stop_tokens.begin(), s.stop_tokens.end(), tokens[row]) != s.stop_tokens.end()) {
                s.finished = true;
                finished->emplace_back(index, STOP_TOKEN);
                continue;
            }
            emitted[row] = 1;
            ++s.emitted;
            if (!room_[row]) {
                s.finished = true;
                finished->emplace_back(index, CONTEXT_FULL);
            } else if (s.emitted >= s.max_tokens) {
                s.finished = true;
                finished->emplace_back(index, MAX_TOKENS);
            } else {
                auto where = std::find(onward_.begin(), onward_.end(), (int)row);
                if (where == onward_.end()) throw Failure{LLMH_INVARIANT, "a sequence goes on that was not planned to"};
                going_rows->push_back((int)(where - onward_.begin()));
                going.push_back(index);
            }
        }
        live_ = going;
        room_.clear();
    }

    void cancel(std::vector<int>* finished) {
        for (int index : live_) {
            sequences_[index].finished = true;
            finished->push_back(index);
        }
        live_.clear();
    }

private:
    int max_seq_len_;
    std::vector<Sequence> sequences_;
    std::vector<int> live_, onward_;
    std::vector<char> room_;
};

int copy(const std::vector<int>& from, int* to) {
    std::copy(from.begin(), from.end(), to);
    return (int)from.size();
}

}  // namespace

// Arrays that receive lists must have room for one int per sequence of the batch.
LLMH_EXPORT int llmh_generation_create(int n, const int* max_tokens, const int* stop_counts, const int* stops,
                                       int max_seq_len, void** out) {
    return guarded([&] {
        if (n < 0) throw Failure{LLMH_FORMAT, "a batch cannot have a negative size"};
        *out = new Generation(n, max_tokens, stop_counts, stops, max_seq_len);
    });
}
LLMH_EXPORT void llmh_generation_destroy(void* g) { delete static_cast<Generation*>(g); }
LLMH_EXPORT int llmh_generation_live(void* g, int* live) { return copy(static_cast<Generation*>(g)->live(), live); }
LLMH_EXPORT int llmh_generation_drop_exhausted(void* g, int* kept_rows, int* n_kept, int* finished, int* n_finished) {
    return guarded([&] {
        std::vector<int> kept, done;
        static_cast<Generation*>(g)->drop_exhausted(&kept, &done);
        *n_kept = copy(kept, kept_rows);
        *n_finished = copy(done, finished);
    });
}
LLMH_EXPORT int llmh_generation_plan_onward(void* g, const int* lengths, int* onward_rows, int* n_onward) {
    return guarded([&] {
        std::vector<int> rows;
        static_cast<Generation*>(g)->plan_onward(lengths, &rows);
        *n_onward = copy(rows, onward_rows);
    });
}
LLMH_EXPORT int llmh_generation_take_tokens(void* g, const int* tokens, int* emitted, int* finished, int* reasons,
                                            int* n_finished, int* going_rows, int* n_going) {
    return guarded([&] {
        std::vector<std::pair<int, int>> done;
        std::vector<int> going;
        static_cast<Generation*>(g)->take_tokens(tokens, emitted, &done, &going);
        for (size_t i = 0; i < done.size(); ++i) {
            finished[i] = done[i].first;
            reasons[i] = done[i].second;
        }
        *n_finished = (int)done.size();
        *n_going = copy(going, going_rows);
    });
}
LLMH_EXPORT int llmh_generation_cancel(void* g, int* finished, int* n_finished) {
    return guarded([&] {
        std::vector<int> done;
        static_cast<Generation*>(g)->cancel(&done);
        *n_finished = copy(done, finished);
    });
}
