// A recorded pass over the layers, walked from native code.
//
// Every launching entry point of the kernel libraries has a packed door, name_packed(const llmb_slot*),
// that takes its arguments as 8-byte slots (csrc/common.cuh). A plan is the list of (door, argument
// block) pairs that one pass of a model made, recorded once by the Python layer while that pass ran;
// llmh_plan_run calls them in order, so a later pass of the same shape costs the host one call
// instead of one marshalled call per kernel. This is the native layer loop of MythEclipse/llm
// (apps/engine/src/model.rs:755-825: body() walks the layers and calls the kernels' C entry points)
// for a model whose layers are put together at run time: the composition stays open, the walk is
// native. The stream is not part of the record: every launch's stream slot is set at run time.
#include <cstring>
#include <vector>

#include "host.hpp"

namespace {

union Slot {
    void* p;
    long long i;
    double f;
};
typedef int (*Door)(const Slot*);

struct Op {
    Door door;
    int first, count, stream_slot;       // slots[first, first + count); stream_slot < 0: none
};

struct Plan {
    std::vector<Op> ops;
    std::vector<Slot> slots;
};

}  // namespace

// doors[i] takes counts[i] slots, the next counts[i] entries of `slots`; stream_slots[i] is the index
// (within the op) of its stream argument, or -1.
LLMH_EXPORT int llmh_plan_create(int n_ops, void* const* doors, const int* counts, const int* stream_slots,
                                 const void* slots, void** out) {
    return llmh::guarded([&] {
        if (n_ops < 0 || !out) throw llmh::Failure{LLMH_FORMAT, "plan: bad arguments"};
        auto* plan = new Plan();
        long long total = 0;
        for (int i = 0; i < n_ops; ++i) {
            if (!doors[i] || counts[i] < 0 || stream_slots[i] >= counts[i]) {
                delete plan;
                throw llmh::Failure{LLMH_FORMAT, "plan: an operation without a door or with a bad slot count"};
            }
            plan->ops.push_back(Op{reinterpret_cast<Door>(doors[i]), (int)total, counts[i], stream_slots[i]});
            total += counts[i];
        }
        plan->slots.resize((size_t)total);
        if (total) std::memcpy(plan->slots.data(), slots, (size_t)total * sizeof(Slot));
        *out = plan;
    });
}

LLMH_EXPORT void llmh_plan_destroy(void* handle) { delete static_cast<Plan*>(handle); }

LLMH_EXPORT int llmh_plan_size(void* handle) { return (int)static_cast<Plan*>(handle)->ops.size(); }

// Calls every recorded launch in order on `stream`. Returns 0, or the first non-zero code a door
// returned with *failed = the index of that launch (its library holds the error text).
LLMH_EXPORT int llmh_plan_run(void* handle, void* stream, int* failed) {
    Plan* plan = static_cast<Plan*>(handle);
    if (failed) *failed = -1;
    for (size_t i = 0; i < plan->ops.size(); ++i) {
        const Op& op = plan->ops[i];
        Slot* args = plan->slots.data() + op.first;
        if (op.stream_slot >= 0) args[op.stream_slot].p = stream;
        int code = op.door(args);
        if (code != 0) {
            if (failed) *failed = (int)i;
            return code;
        }
    }
    return 0;
}
