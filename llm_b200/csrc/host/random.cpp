// Random weights on the host: the same values, bit for bit, as the device kernel
// llmb_random_normal (csrc/elementwise.cu) and the plain statement of the tests give; the
// formulas are in csrc/random_normal.h. Work is cut over the machine's threads, which
// changes nothing: every element depends on (key, index) alone.
#include <algorithm>
#include <thread>
#include <vector>

#include "../random_normal.h"
#include "host.hpp"

namespace {

template <typename Store>
void fill(long long n, unsigned long long key, float mean, float deviation, Store store) {
    unsigned threads = std::max(1u, std::min(std::thread::hardware_concurrency(), 64u));
    if (n < (1 << 16)) threads = 1;
    std::vector<std::thread> pool;
    long long per = (n + threads - 1) / threads;
    for (unsigned t = 0; t < threads; ++t) {
        long long begin = t * per, end = std::min(n, begin + per);
        if (begin >= end) break;
        auto work = [=]() {
            for (long long i = begin; i < end; ++i) store(i, llmb_random::value(key, (uint64_t)i, mean, deviation));
        };
        if (threads == 1) work();
        else pool.emplace_back(work);
    }
    for (auto& th : pool) th.join();
}

}  // namespace

// out: n values of float (dtype 0) or bfloat16 (dtype 1): mean + deviation * N(0, 1) keyed by (key, index).
LLMH_EXPORT int llmh_random_normal(void* out, int dtype, long long n, unsigned long long key, float mean,
                                   float deviation) {
    return llmh::guarded([&] {
        if (n < 0 || (n > 0 && !out)) throw llmh::Failure{LLMH_FORMAT, "random_normal: bad arguments"};
        if (dtype == 0) {
            float* o = static_cast<float*>(out);
            fill(n, key, mean, deviation, [o](long long i, float v) { o[i] = v; });
        } else if (dtype == 1) {
            uint16_t* o = static_cast<uint16_t*>(out);
            fill(n, key, mean, deviation, [o](long long i, float v) { o[i] = llmb_random::to_bfloat16_bits(v); });
        } else {
            throw llmh::Failure{LLMH_FORMAT, "random_normal: unknown dtype"};
        }
    });
}
