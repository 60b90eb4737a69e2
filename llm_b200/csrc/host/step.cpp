// What a step does on the host before anything is launched: check the batch, and pack the
// integers that the kernels read into one buffer that goes to the device in one copy.
//
// A batch is n entries; entry i is the sequence in slots[i] bringing counts[i] new tokens
// (tokens flat, in entry order) and asking for the logits at want_counts[i] places among them
// (wants flat, each an index into the entry's own tokens). Positions come from each slot's
// length, as `start = kv.len()` does for one sequence in MythEclipse/llm
// (apps/engine/src/model.rs:764-784 for the checks, :775 for the positions).
//
// Sections of the buffer (int32, each starting on a 16-byte boundary), T tokens, B entries,
// R wanted rows, G cache groups:
//   0 tokens[T]   1 positions[T]   2 entry of each token[T]   3 first token of each entry[B+1]
//   4 length of each sequence after the step[B]   5 slots[B]   6 wanted rows[R] (indices into T)
//   7 entries in order of falling length[B] (attention takes the longest sequences first)
//   8+g page-table rows of group g [B, ring_g]
#include <algorithm>
#include <vector>

#include "cache.hpp"

using namespace llmh;

namespace {

constexpr int FIXED_SECTIONS = 8;

long long padded(long long n) { return (n + 3) / 4 * 4; }

void layout(const Cache& cache, int n, const int* counts, const int* want_counts, long long* offsets, long long* sizes,
            long long* total) {
    long long tokens = 0, rows = 0;
    for (int i = 0; i < n; ++i) {
        tokens += counts[i];
        rows += want_counts[i];
    }
    long long fixed[FIXED_SECTIONS] = {tokens, tokens, tokens, n + 1, n, n, rows, n};
    long long at = 0;
    int section = 0;
    for (; section < FIXED_SECTIONS; ++section) {
        offsets[section] = at;
        sizes[section] = fixed[section];
        at += padded(fixed[section]);
    }
    for (const Group& group : cache.groups) {
        offsets[section] = at;
        sizes[section] = (long long)n * group.ring_pages;
        at += padded(sizes[section]);
        ++section;
    }
    *total = std::max<long long>(at, 4);
}

}  // namespace

// Everything that can be wrong with a batch, found before anything is launched or changed.
LLMH_EXPORT int llmh_step_check(void* cache_, int n, const int* slots, const int* counts, const int* tokens,
                                const int* want_counts, const int* wants, int vocab, int max_seq_len) {
    return guarded([&] {
        const Cache& cache = *static_cast<Cache*>(cache_);
        std::vector<char> seen(cache.max_slots, 0);
        long long token_at = 0, want_at = 0;
        for (int i = 0; i < n; ++i) {
            int slot = slots[i];
            cache.require_held(slot);
            if (seen[slot]) throw Failure{LLMH_FORMAT, "slot " + std::to_string(slot) + " appears twice in one step"};
            seen[slot] = 1;
            if (counts[i] <= 0) throw Failure{LLMH_FORMAT, "slot " + std::to_string(slot) + " brings no token"};
            for (int t = 0; t < counts[i]; ++t) {
                int id = tokens[token_at + t];
                if (id < 0 || id >= vocab)
                    throw Failure{LLMH_FORMAT, "token id " + std::to_string(id) + " is outside the vocabulary of " + std::to_string(vocab)};
            }
            for (int w = 0; w < want_counts[i]; ++w) {
                int place = wants[want_at + w];
                if (place < 0 || place >= counts[i])
                    throw Failure{LLMH_FORMAT, "wanted place " + std::to_string(place) + " is outside the " +
                                                   std::to_string(counts[i]) + " tokens of slot " + std::to_string(slot)};
            }
            long long new_length = (long long)cache.length(slot) + counts[i];
            if (new_length > max_seq_len) throw Failure{LLMH_CONTEXT_FULL, "", new_length, max_seq_len};
            token_at += counts[i];
            want_at += want_counts[i];
        }
    });
}

// Pages for every entry's new length, all or nothing.
LLMH_EXPORT int llmh_step_reserve(void* cache_, int n, const int* slots, const int* counts) {
    return guarded([&] {
        Cache& cache = *static_cast<Cache*>(cache_);
        std::vector<long long> lengths(n);
        for (int i = 0; i < n; ++i) {
            cache.require_held(slots[i]);
            lengths[i] = (long long)cache.length(slots[i]) + counts[i];
        }
        cache.reserve_many(n, slots, lengths.data());
    });
}

LLMH_EXPORT int llmh_step_sections(void* cache_) { return FIXED_SECTIONS + (int)static_cast<Cache*>(cache_)->groups.size(); }

LLMH_EXPORT int llmh_step_layout(void* cache_, int n, const int* counts, const int* want_counts, long long* offsets,
                                 long long* sizes, long long* total) {
    return guarded([&] { layout(*static_cast<Cache*>(cache_), n, counts, want_counts, offsets, sizes, total); });
}

// Fills `out` (capacity in int32). summary: [tokens, wanted rows, 1 if every entry brings one token,
// longest sequence after the step, int32 used].
LLMH_EXPORT int llmh_step_pack(void* cache_, int n, const int* slots, const int* counts, const int* tokens,
                               const int* want_counts, const int* wants, int32_t* out, long long capacity,
                               long long* offsets, long long* sizes, long long* summary) {
    return guarded([&] {
        const Cache& cache = *static_cast<Cache*>(cache_);
        long long total = 0;
        layout(cache, n, counts, want_counts, offsets, sizes, &total);
        if (total > capacity) throw Failure{LLMH_INVARIANT, "the step buffer holds " + std::to_string(capacity) + " integers, the step needs " + std::to_string(total)};
        int32_t* tok = out + offsets[0];
        int32_t* pos = out + offsets[1];
        int32_t* seq = out + offsets[2];
        int32_t* cu = out + offsets[3];
        int32_t* lens = out + offsets[4];
        int32_t* slot_ids = out + offsets[5];
        int32_t* rows = out + offsets[6];
        int32_t* order = out + offsets[7];
        long long at = 0, row_at = 0, want_at = 0;
        int decode = 1, max_len = 0;
        cu[0] = 0;
        for (int i = 0; i < n; ++i) {
            cache.require_held(slots[i]);
            int start = cache.length(slots[i]), count = counts[i];
            for (int t = 0; t < count; ++t) {
                tok[at + t] = tokens[at + t];
                pos[at + t] = start + t;
                seq[at + t] = i;
            }
            for (int w = 0; w < want_counts[i]; ++w) rows[row_at++] = (int32_t)(at + wants[want_at + w]);
            want_at += want_counts[i];
            at += count;
            cu[i + 1] = (int32_t)at;
            lens[i] = start + count;
            slot_ids[i] = slots[i];
            if (count != 1) decode = 0;
            max_len = std::max(max_len, start + count);
        }
        for (int i = 0; i < n; ++i) order[i] = i;
        std::stable_sort(order, order + n, [&](int32_t a, int32_t b) { return lens[a] > lens[b]; });
        for (size_t g = 0; g < cache.groups.size(); ++g) {
            const Group& group = cache.groups[g];
            int32_t* table = out + offsets[FIXED_SECTIONS + g];
            for (int i = 0; i < n; ++i)
                std::copy_n(group.table.begin() + (size_t)slots[i] * group.ring_pages, group.ring_pages,
                            table + (size_t)i * group.ring_pages);
        }
        summary[0] = at;
        summary[1] = row_at;
        summary[2] = decode;
        summary[3] = max_len;
        summary[4] = total;
    });
}

// After the step's kernels are queued: every sequence is as long as the step made it.
LLMH_EXPORT int llmh_step_commit(void* cache_, int n, const int* slots, const int* counts) {
    return guarded([&] {
        Cache& cache = *static_cast<Cache*>(cache_);
        for (int i = 0; i < n; ++i) {
            cache.require_held(slots[i]);
            cache.set_length(slots[i], cache.length(slots[i]) + counts[i]);
        }
    });
}
