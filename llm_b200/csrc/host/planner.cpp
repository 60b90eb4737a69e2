// Placing the scratch buffers of a step into one arena. As in MythEclipse/llm's workspace
// (apps/engine/src/workspace.rs:63-106): requests {name, bytes, first_use, last_use} over numbered
// phases are placed in order of (first use, name), each at the lowest aligned offset that overlaps
// no buffer live at the same time; a buffer written in the phase in which another is last read
// counts as live with it.
#include <algorithm>
#include <set>
#include <string>
#include <vector>

#include "host.hpp"

using namespace llmh;

LLMH_EXPORT int llmh_plan_place(int n, const char* const* names, const long long* nbytes, const int* first_use,
                                const int* last_use, long long alignment, long long* offsets, long long* total) {
    return guarded([&] {
        if (alignment < 1) throw Failure{LLMH_FORMAT, "the alignment must be positive"};
        std::set<std::string> seen;
        std::vector<int> order(n);
        for (int i = 0; i < n; ++i) {
            order[i] = i;
            if (!seen.insert(names[i]).second) throw Failure{LLMH_FORMAT, "two scratch buffers share the name " + std::string(names[i])};
            if (last_use[i] < first_use[i]) throw Failure{LLMH_FORMAT, std::string(names[i]) + " is read before it is written"};
            if (nbytes[i] < 0) throw Failure{LLMH_FORMAT, std::string(names[i]) + " has a negative size"};
        }
        std::sort(order.begin(), order.end(), [&](int a, int b) {
            if (first_use[a] != first_use[b]) return first_use[a] < first_use[b];
            return std::string(names[a]) < std::string(names[b]);
        });
        auto align = [&](long long v) { return (v + alignment - 1) / alignment * alignment; };
        long long high = 0;
        std::vector<int> placed;
        for (int i : order) {
            std::vector<std::pair<long long, long long>> busy;
            for (int p : placed)
                if (first_use[p] <= last_use[i] && first_use[i] <= last_use[p]) busy.emplace_back(offsets[p], offsets[p] + nbytes[p]);
            std::sort(busy.begin(), busy.end());
            long long offset = 0;
            for (const auto& range : busy) {
                if (offset + nbytes[i] <= range.first) break;
                offset = std::max(offset, align(range.second));
            }
            offsets[i] = offset;
            placed.push_back(i);
            high = std::max(high, offset + nbytes[i]);
        }
        *total = align(high);
    });
}
