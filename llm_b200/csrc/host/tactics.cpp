// Which kernel variant serves which shape. One table per kernel family; a row names a variant, a
// rank, a guard that states every assumption the kernel makes, and the evidence for its rank. The
// highest-ranked row that is not switched off and whose guard holds is chosen, and every refusal
// keeps its reason. The scheme is the tactics table of MythEclipse/llm
// (apps/engine/src/tactics.rs:99-109 rows, :353-396 selection with recorded fallback reasons); the
// rows are this library's own kernels.
#include <algorithm>
#include <cstring>
#include <functional>
#include <set>
#include <string>
#include <vector>

#include "../plan.h"
#include "host.hpp"

using namespace llmh;

namespace {

struct Shape {
    // linear: out[m, n] = x[m, k] . w[n, k]^T, rows of x `lda` elements apart
    int m = 0, n = 0, k = 0, lda = 0;
    // attention
    int decode = 0, n_heads = 1, n_kv_heads = 1, head_dim = 0, window = 0, packed = 0;
    // both
    int bf16 = 0;          // operands (and caches) are bfloat16
    int aligned = 1;       // operands start on 16-byte boundaries
};

struct Row {
    const char* name;
    int rank;
    std::function<std::string(const Shape&)> guard;      // empty: the kernel can run
    const char* evidence;
};

std::string always(const Shape&) { return ""; }

std::string skinny_guard(const Shape& s) {
    if (!s.bf16) return "bfloat16 operands only";
    if (s.m > 64) return std::to_string(s.m) + " rows exceed 64";
    if (s.k % 8 || s.lda % 8)
        return "K " + std::to_string(s.k) + " or the row stride " + std::to_string(s.lda) +
               " is no multiple of 8 elements (16-byte loads)";
    if (!s.aligned) return "an operand does not start on a 16-byte boundary";
    return "";
}

std::string tc_guard(const Shape& s) {
    if (!s.bf16) return "bfloat16 operands only";
    if (s.k % 8 || s.lda % 8)
        return "K " + std::to_string(s.k) + " or the row stride " + std::to_string(s.lda) +
               " is no multiple of 8 elements: a TMA row stride must be a multiple of 16 bytes";
    if (!s.aligned) return "an operand does not start on a 16-byte boundary (TMA base address)";
    return "";
}

std::string generic_guard(const Shape& s) {
    if (s.head_dim > LLMB_MAX_HEAD_DIM)
        return "head_dim " + std::to_string(s.head_dim) + " exceeds " + std::to_string(LLMB_MAX_HEAD_DIM);
    return "";
}

bool mma_head_dim(int d) { return d == 32 || d == 64 || d == 96 || d == 128; }

std::string decode_guard(const Shape& s) {
    if (!s.decode) return "serves steps in which every sequence brings one token";
    if (!s.bf16) return "bfloat16 caches only";
    if (s.window) return "no window";
    if (s.n_heads / s.n_kv_heads > 8) return "group of " + std::to_string(s.n_heads / s.n_kv_heads) + " query heads exceeds 8";
    if (!mma_head_dim(s.head_dim)) return "head_dim " + std::to_string(s.head_dim) + " (served: 32, 64, 96, 128)";
    return "";
}

std::string prefill_guard(const Shape& s) {
    if (!s.packed) return "needs the packed batch description (cu_seqlens and seq_lens)";
    if (!s.bf16) return "bfloat16 caches only";
    if (s.window) return "no window";
    if (!mma_head_dim(s.head_dim)) return "head_dim " + std::to_string(s.head_dim) + " (served: 32, 64, 96, 128)";
    return "";
}

std::string prefill_tc_guard(const Shape& s) {
    std::string reason = prefill_guard(s);
    if (!reason.empty()) return reason;
    if (s.head_dim != 64 && s.head_dim != 128) return "head_dim " + std::to_string(s.head_dim) + " (served: 64, 128)";
    if (!s.aligned) return "the projection's rows are not 16-byte aligned (TMA)";
    return "";
}

const std::vector<Row>& table(int family) {
    static const std::vector<Row> linear = {
        {"gemm_tc", 30, tc_guard,
         "tcgen05.mma with the accumulator in tensor memory, operands by TMA; weights on the 128-row side and "
         "split K while the output has few tiles (always up to 128 tokens), pairs of SMs on 256 x 256 tiles "
         "above; a folded norm's scale, the next norm's input and the rotation with the cache write ride in its "
         "epilogues. Measured on a B200 at Llama-3.1-8B layer sizes: 1,400 TFLOP/s at 2,048 tokens (73.6 us for "
         "2048 x 6144 x 4096), 2.9 to 5.9 TB/s of weights at 8 tokens"},
        {"gemm_skinny", 20, skinny_guard,
         "decode product for up to 64 rows: W streamed once with 128-bit loads into mma.sync fragments, K split "
         "over warps with an ordered last-arriver sum; within a few percent of gemm_tc at 8 rows, behind it from 16"},
        {"gemm_simt", 0, always,
         "CUDA-core product with a fixed summation order; any shape and stride; the only variant of the 32-bit path"},
    };
    static const std::vector<Row> attention = {
        {"attention_decode", 20, decode_guard,
         "split-KV decode attention: pages through shared memory with cp.async (a ring sized by the head size), "
         "the query heads of a group as rows of mma.sync tiles, partials merged by a second kernel. Measured: "
         "45.2 us for 8 sequences of 8,192 keys with 8 kv heads of 128 (5.94 TB/s)"},
        {"attention_prefill_tc", 15, prefill_tc_guard,
         "flash attention with both products on tcgen05 (accumulators in tensor memory, K and V pages by TMA), "
         "two score buffers of 64 keys so that Q K^T runs under the softmax, one thread per query row, two "
         "blocks an SM; head sizes 64 and 128. Measured with 32/8 heads of 128: 46.3 us at 2,048 tokens, 497.7 us "
         "at 8,192 (742 and 1,105 TFLOP/s of causal work); with heads of 64: 40.5 us at 2,048 tokens"},
        {"attention_prefill", 10, prefill_guard,
         "flash attention over the paged cache for steps with several new tokens a sequence: 64-query tiles, "
         "mma.sync, online softmax, heaviest tile first; head sizes 32, 64, 96, 128. Measured: 170 us at 2,048 "
         "tokens with 32/8 heads of 128, 90 us with heads of 64"},
        {"attention_generic", 0, generic_guard,
         "one block per (token, head), 32-bit arithmetic, any head size up to 256, any group, window and ring; "
         "the only variant of the 32-bit path"},
    };
    return family == 0 ? linear : attention;
}

std::set<std::string>& switched_off() {
    static std::set<std::string> names;
    return names;
}

// The chosen row's name; `reasons` gets one line per higher-ranked row that was passed over.
const char* choose(int family, const Shape& shape, std::string* reasons) {
    std::vector<const Row*> rows;
    for (const Row& row : table(family)) rows.push_back(&row);
    std::stable_sort(rows.begin(), rows.end(), [](const Row* a, const Row* b) { return a->rank > b->rank; });
    for (const Row* row : rows) {
        std::string reason = switched_off().count(row->name) ? "disabled" : row->guard(shape);
        if (reason.empty()) return row->name;
        if (reasons) *reasons += std::string("  not ") + row->name + ": " + reason + "\n";
    }
    throw Failure{LLMH_INVARIANT, "no kernel accepts the shape:\n" + (reasons ? *reasons : std::string())};
}

void copy_out(const std::string& text, char* out, int capacity) {
    if (!out || capacity <= 0) return;
    size_t n = std::min<size_t>(text.size(), (size_t)capacity - 1);
    std::memcpy(out, text.data(), n);
    out[n] = 0;
}

}  // namespace

// family: 0 products, 1 attention. shape: 12 ints {m, n, k, lda, decode, n_heads, n_kv_heads, head_dim,
// window, packed, bf16, aligned}. name and reasons are filled up to their capacities.
LLMH_EXPORT int llmh_tactics_choose(int family, const int* shape, char* name, int name_capacity, char* reasons,
                                    int reasons_capacity) {
    return guarded([&] {
        if (family != 0 && family != 1) throw Failure{LLMH_FORMAT, "unknown kernel family"};
        Shape s;
        s.m = shape[0]; s.n = shape[1]; s.k = shape[2]; s.lda = shape[3];
        s.decode = shape[4]; s.n_heads = std::max(shape[5], 1); s.n_kv_heads = std::max(shape[6], 1);
        s.head_dim = shape[7]; s.window = shape[8]; s.packed = shape[9]; s.bf16 = shape[10]; s.aligned = shape[11];
        std::string why;
        copy_out(choose(family, s, &why), name, name_capacity);
        copy_out(why, reasons, reasons_capacity);
    });
}

// Take a variant out of the choice, or put it back. Names that are no row's (switches that a
// kernel reads for itself, such as "gemm_tc_pair") are kept as well.
LLMH_EXPORT void llmh_tactics_set_disabled(const char* name, int disabled) {
    if (disabled) switched_off().insert(name);
    else switched_off().erase(name);
}
LLMH_EXPORT int llmh_tactics_is_disabled(const char* name) { return switched_off().count(name) ? 1 : 0; }

LLMH_EXPORT int llmh_tactics_rows(int family) { return (family == 0 || family == 1) ? (int)table(family).size() : 0; }
LLMH_EXPORT int llmh_tactics_row(int family, int index, const char** name, int* rank, const char** evidence) {
    return guarded([&] {
        if ((family != 0 && family != 1) || index < 0 || index >= (int)table(family).size())
            throw Failure{LLMH_INVARIANT, "no such row"};
        const Row& row = table(family)[index];
        *name = row.name;
        *rank = row.rank;
        *evidence = row.evidence;
    });
}
