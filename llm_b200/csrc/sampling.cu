// Token sampling on the device, one block per row of logits.
//
// The chain and its order are those of MythEclipse/llm's sampler
// (apps/engine/src/sampler.rs:54-96): repeat penalty over the recent window
// (sampler.rs:110-128, once per occurrence), greedy when temperature <= 0 with
// the first maximum winning (sampler.rs:167-175), else logits / temperature,
// top-k, softmax over the survivors in descending order, top-p, min-p, and an
// inverse-CDF walk in that order with a uniform number from xorshift64*
// (sampler.rs:98-107: state seed | 1, top 24 bits). Each row has its own
// parameters and its own generator state, so a row's draw does not depend on
// the batch it is in.
//
// top_k must lie in [1, MAX_TOP_K] for the ranked chain. top_k == 0 (no top-k)
// is served only with top_p >= 1: softmax over the whole row, min-p, and an
// inverse-CDF walk in index order (the same distribution; which token a given
// uniform number picks differs from a walk in descending order).
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_sampling)

constexpr int THREADS = 512;
constexpr int MAX_TOP_K = 1024;
constexpr int CANDIDATES = 2048;   // room for ties at the top-k threshold
constexpr int RADIX_BINS = 2048;   // bins of the widest digit of the radix select
constexpr int WINDOW = 1024;       // recent tokens the penalty handles in parallel (longer windows: one thread)

__device__ __forceinline__ unsigned ordered_key(float v) {
    unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // larger float -> larger key
}

struct ArgMax {
    float value;
    int index;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

// Calls visit(value, index) for every element of row[0..n) that falls to this thread, in rising
// index order. Rows that start on a 16-byte boundary are read four values a load and eight loads
// ahead: a thread's share of a 128,256-entry row is 8 rounds of loads instead of 250 dependent ones
// (one block has to keep enough bytes in flight to fetch half a megabyte quickly).
template <typename Visit>
__device__ __forceinline__ void for_each_of_row(const float* row, int n, Visit visit) {
    int quads = (reinterpret_cast<uintptr_t>(row) & 15) == 0 ? n >> 2 : 0;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    auto visit4 = [&](const float4& v, int q) {
        visit(v.x, 4 * q);
        visit(v.y, 4 * q + 1);
        visit(v.z, 4 * q + 2);
        visit(v.w, 4 * q + 3);
    };
    int q = threadIdx.x;
    for (; q + 7 * THREADS < quads; q += 8 * THREADS) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = row4[q + u * THREADS];          // eight loads in flight
#pragma unroll
        for (int u = 0; u < 8; ++u) visit4(v[u], q + u * THREADS);
    }
    for (; q < quads; q += THREADS) visit4(row4[q], q);
    for (int i = 4 * quads + threadIdx.x; i < n; i += THREADS) visit(row[i], i);
}

// First maximum of scale * row[0..n). NaN never wins (comparisons with NaN are false).
__device__ ArgMax block_argmax(const float* row, int n, ArgMax* scratch, float scale = 1.0f) {
    ArgMax best{-INFINITY, 0x7fffffff};
    for_each_of_row(row, n, [&](float v, int i) {
        v *= scale;
        if (v > best.value) best = ArgMax{v, i};
    });
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, best.value, offset),
                     __shfl_xor_sync(0xffffffffu, best.index, offset)};
        best = better(best, other);
    }
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    if (warp == 0) {
        int n_warps = blockDim.x >> 5;
        ArgMax v = lane < n_warps ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            ArgMax other{__shfl_xor_sync(0xffffffffu, v.value, offset),
                         __shfl_xor_sync(0xffffffffu, v.index, offset)};
            v = better(v, other);
        }
        if (lane == 0) scratch[0] = v;
    }
    __syncthreads();
    ArgMax result = scratch[0];
    if (result.index == 0x7fffffff) result.index = 0;
    __syncthreads();
    return result;
}

__global__ void __launch_bounds__(THREADS)
argmax_rows_kernel(const float* __restrict__ logits, int stride, int vocab, int* __restrict__ out) {
    __shared__ ArgMax scratch[32];
    ArgMax best = block_argmax(logits + (size_t)blockIdx.x * stride, vocab, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = best.index;
}

LLMB_EXPORT int llmb_argmax_rows(const float* logits, int stride, int n_rows, int vocab, int* out,
                                 cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(n_rows > 0 && vocab > 0 && stride >= vocab, "argmax: bad sizes");
    argmax_rows_kernel<<<n_rows, THREADS, 0, stream>>>(logits, stride, vocab, out);
    return check_launch("argmax_rows");
}

__device__ __forceinline__ float next_uniform(unsigned long long* state) {
    unsigned long long x = *state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    *state = x;
    unsigned long long value = x * 0x2545F4914F6CDD1DULL;
    return (float)(value >> 40) / 16777216.0f;
}

// Sum of `value` over the threads before this one (thread 0 first), for every thread of the block.
__device__ unsigned block_exclusive_sum(unsigned value, unsigned* warp_totals) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned inclusive = value;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        unsigned below = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= offset) inclusive += below;
    }
    if (lane == 31) warp_totals[warp] = inclusive;
    __syncthreads();
    unsigned before = 0u;
    for (int w = 0; w < warp; ++w) before += warp_totals[w];
    __syncthreads();
    return before + inclusive - value;
}

// params[row] = {temperature, top_p, min_p, repeat_penalty}; iparams[row] =
// {top_k, repeat_last_n}. recent[row, 0..recent_cap) holds the row's generated
// tokens as a ring: token number i (counted from 0) is at recent[row, i % cap],
// recent_len[row] counts all of them. `logits` is modified in place (the penalty
// on the recent tokens' entries). status[row] is set to 1 when the row was refused (its parameters, or
// more equal logits at the top-k cut than the kernel ranks) and token 0 stands in its place; the kernel
// never clears it, so a refusal in any step stays visible until the host has read and cleared it.
__global__ void __launch_bounds__(THREADS)
sample_rows_kernel(float* __restrict__ logits, int stride, int vocab,
                   const float4* __restrict__ params, const int2* __restrict__ iparams,
                   int* __restrict__ recent, int* __restrict__ recent_len,
                   int recent_cap, unsigned long long* __restrict__ rng, int* __restrict__ out,
                   int* __restrict__ status, int record, const int* __restrict__ state_rows) {
    __shared__ ArgMax scratch[32];
    __shared__ unsigned histogram[RADIX_BINS];
    __shared__ unsigned block_sums_u[32];
    __shared__ float cand_value[CANDIDATES];
    __shared__ int cand_index[CANDIDATES];
    __shared__ unsigned shared_prefix, shared_need, shared_count;
    __shared__ float block_sums[THREADS];
    __shared__ int window[WINDOW];

    // row of logits and of `out`; the sequence's parameters, window, generator and status are in
    // row state_rows[row] of their arrays (the same row if state_rows is null)
    int logits_row = blockIdx.x;
    int row_id = state_rows ? state_rows[logits_row] : logits_row;
    LLMB_STAMP(0, 0);
    float* row = logits + (size_t)logits_row * stride;
    float temperature = params[row_id].x, top_p = params[row_id].y, min_p = params[row_id].z;
    float penalty = params[row_id].w;
    int top_k = iparams[row_id].x, last_n = iparams[row_id].y;
    int tid = threadIdx.x;
    // thread 0 calls this once: the token is the row's result and, with `record`, the newest entry
    // of the row's window (a ring over its generated tokens)
    auto finish = [&](int token) {
        out[logits_row] = token;
        if (record && recent != nullptr) {
            int total = recent_len[row_id];
            recent[(size_t)row_id * recent_cap + (total % recent_cap)] = token;
            recent_len[row_id] = total + 1;
        }
    };

    if (penalty != 1.0f && last_n > 0 && recent != nullptr) {
        // A token that occurs c times in the window is penalised c times, one after the other
        // (apps/engine/src/sampler.rs:115-127). One thread per window place; the first place of a
        // token applies all of its c steps, so the arithmetic is that of the serial loop.
        int total = recent_len[row_id];
        int span = min(min(total, last_n), recent_cap);
        if (span <= WINDOW) {
            for (int t = tid; t < span; t += THREADS)
                window[t] = recent[(size_t)row_id * recent_cap + ((total - span + t) % recent_cap)];
            __syncthreads();
            for (int t = tid; t < span; t += THREADS) {
                int id = window[t];
                if (id < 0 || id >= vocab) continue;
                int count = 0;
                bool first = true;
                for (int u = 0; u < span; ++u) {
                    if (window[u] != id) continue;
                    if (u < t) { first = false; break; }
                    ++count;
                }
                if (!first) continue;
                float v = row[id];
                for (int c = 0; c < count; ++c) v = v > 0.f ? v / penalty : v * penalty;
                row[id] = v;
            }
        } else if (tid == 0) {
            for (int i = total - span; i < total; ++i) {
                int id = recent[(size_t)row_id * recent_cap + (i % recent_cap)];
                if (id < 0 || id >= vocab) continue;
                float v = row[id];
                row[id] = v > 0.f ? v / penalty : v * penalty;
            }
        }
    }
    __syncthreads();

    if (!(temperature > 0.f)) {
        ArgMax best = block_argmax(row, vocab, scratch);
        if (tid == 0) finish(best.index);
        return;
    }
    // every later reading of the row takes its values times 1 / temperature (the same rounding each
    // time) instead of a pass that writes the scaled row back
    float inverse = 1.0f / temperature;
    LLMB_STAMP(1, 0);                                 // the penalty is applied

    if (top_k <= 0 || top_k >= vocab) {
        if (vocab <= MAX_TOP_K) {
            top_k = vocab;                      // a small row: rank all of it
        } else if (top_k > 0 || (top_p >= 0.f && top_p < 1.f)) {
            // the ranked chain is limited to MAX_TOP_K candidates
            if (tid == 0) { status[row_id] = 1; finish(0); }
            return;
        }
    } else if (top_k > MAX_TOP_K) {
        if (tid == 0) { status[row_id] = 1; finish(0); }
        return;
    }

    if (top_k <= 0) {
        // ---- whole row, index order: softmax, min-p, inverse CDF
        ArgMax best = block_argmax(row, vocab, scratch, inverse);
        float cut = min_p > 0.f ? min_p : 0.f;
        int per_thread = (vocab + THREADS - 1) / THREADS;
        int begin = min(tid * per_thread, vocab), end = min(begin + per_thread, vocab);
        float local = 0.f;
        for (int i = begin; i < end; ++i) {
            float p = expf(row[i] * inverse - best.value);
            if (p >= cut) local += p;
        }
        block_sums[tid] = local;
        __syncthreads();
        if (tid == 0) {
            float total = 0.f;
            for (int i = 0; i < THREADS; ++i) total += block_sums[i];
            unsigned long long state = rng[row_id];
            float target = next_uniform(&state) * total;
            rng[row_id] = state;
            int owner = -1;
            float before = 0.f;
            for (int i = 0; i < THREADS; ++i) {
                if (block_sums[i] > 0.f && target - (before + block_sums[i]) <= 0.f) { owner = i; break; }
                before += block_sums[i];
            }
            int pick = best.index;
            if (owner >= 0) {
                float remaining = target - before;
                int b = min(owner * per_thread, vocab), e = min(b + per_thread, vocab);
                for (int i = b; i < e; ++i) {
                    float p = expf(row[i] * inverse - best.value);
                    if (p < cut) continue;
                    pick = i;
                    remaining -= p;
                    if (remaining <= 0.f) break;
                }
            }
            finish(pick);
        }
        return;
    }

    // ---- ranked chain: radix select of the top_k-th largest key, three digits of 11, 11 and 10 bits.
    // The first digit is the sign, the exponent and two bits of the mantissa: wide enough to spread
    // a row of logits over some hundred bins, so that the threads' additions seldom meet.
    if (tid == 0) { shared_prefix = 0u; shared_need = (unsigned)top_k; }
    __syncthreads();
    for (int digit = 0; digit < 3; ++digit) {
        const int shift = digit == 0 ? 21 : digit == 1 ? 10 : 0;
        const int n_bins = digit == 2 ? 1024 : 2048;
        for (int i = tid; i < RADIX_BINS; i += THREADS) histogram[i] = 0u;
        __syncthreads();
        unsigned prefix = shared_prefix;
        unsigned mask = digit == 0 ? 0u : (0xffffffffu << (digit == 1 ? 21 : 10));
        for_each_of_row(row, vocab, [&](float v, int) {
            unsigned key = ordered_key(v * inverse);
            if ((key & mask) == prefix) atomicAdd(&histogram[(key >> shift) & (unsigned)(n_bins - 1)], 1u);
        });
        __syncthreads();
        // the bin, counted from the top, in which the running count reaches what is still needed:
        // every thread sums four neighbouring bins, the block scans the threads from the top down
        unsigned need = shared_need;
        int top_bin = n_bins - 1 - 4 * tid;                       // this thread's highest bin
        unsigned mine = 0u;
        if (top_bin >= 3)
            mine = histogram[top_bin] + histogram[top_bin - 1] + histogram[top_bin - 2] + histogram[top_bin - 3];
        unsigned before = block_exclusive_sum(mine, block_sums_u);  // of the threads with higher bins
        if (top_bin >= 3 && before < need && before + mine >= need) {
            unsigned left = need - before;
            int bin = top_bin;
            for (; bin > top_bin - 3; --bin) {
                if (histogram[bin] >= left) break;
                left -= histogram[bin];
            }
            shared_need = left;
            shared_prefix = prefix | ((unsigned)bin << shift);
        }
        __syncthreads();
    }
    LLMB_STAMP(2, 0);                                 // the radix select has its threshold
    unsigned threshold = shared_prefix;        // key of the top_k-th largest value
    if (tid == 0) shared_count = 0u;
    __syncthreads();
    for_each_of_row(row, vocab, [&](float v, int i) {
        v *= inverse;
        if (ordered_key(v) >= threshold) {
            unsigned at = atomicAdd(&shared_count, 1u);
            if (at < CANDIDATES) { cand_value[at] = v; cand_index[at] = i; }
        }
    });
    __syncthreads();
    LLMB_STAMP(3, 0);                                 // the candidates are gathered
    int count = (int)min(shared_count, (unsigned)CANDIDATES);
    if (shared_count > (unsigned)CANDIDATES) {
        // more ties at the threshold than the buffer holds
        if (tid == 0) { status[row_id] = 1; finish(0); }
        return;
    }
    // bitonic sort, descending by value, ascending by index among equals
    int padded = 1;
    while (padded < count) padded <<= 1;
    for (int i = count + tid; i < padded; i += THREADS) { cand_value[i] = -INFINITY; cand_index[i] = 0x7fffffff; }
    __syncthreads();
    for (int size = 2; size <= padded; size <<= 1) {
        for (int step = size >> 1; step > 0; step >>= 1) {
            for (int i = tid; i < padded; i += THREADS) {
                int partner = i ^ step;
                if (partner > i) {
                    bool descending = (i & size) == 0;
                    float va = cand_value[i], vb = cand_value[partner];
                    int ia = cand_index[i], ib = cand_index[partner];
                    bool a_first = va > vb || (va == vb && ia < ib);
                    if (a_first != descending) {
                        cand_value[i] = vb; cand_value[partner] = va;
                        cand_index[i] = ib; cand_index[partner] = ia;
                    }
                }
            }
            __syncthreads();
        }
    }
    LLMB_STAMP(4, 0);                                 // the candidates are sorted
    int kept = min(count, top_k);
    float top_value = cand_value[0];
    for (int i = tid; i < kept; i += THREADS) cand_value[i] = expf(cand_value[i] - top_value);
    __syncthreads();
    if (tid == 0) {
        float sum = 0.f;
        for (int i = 0; i < kept; ++i) sum += cand_value[i];
        if (sum > 0.f)
            for (int i = 0; i < kept; ++i) cand_value[i] /= sum;
        if (top_p >= 0.f && top_p < 1.f) {
            float cumulative = 0.f;
            for (int i = 0; i < kept; ++i) {
                cumulative += cand_value[i];
                if (cumulative > top_p) { kept = i + 1; break; }
            }
        }
        if (min_p > 0.f) {
            float cut = cand_value[0] * min_p;
            int keep = 0;
            while (keep < kept && cand_value[keep] >= cut) ++keep;
            kept = keep;
        }
        float total = 0.f;
        for (int i = 0; i < kept; ++i) total += cand_value[i];
        int pick = cand_index[0];
        if (total > 0.f) {
            unsigned long long state = rng[row_id];
            float target = next_uniform(&state) * total;
            rng[row_id] = state;
            for (int i = 0; i < kept; ++i) {
                target -= cand_value[i];
                if (target <= 0.f) { pick = cand_index[i]; break; }
            }
        }
        finish(pick);
        LLMB_STAMP(5, 0);                             // the token is drawn
    }
}

// The stamps of the last sampling launch in a build with -DLLMB_TRACE (see common.cuh); 1 otherwise.
LLMB_EXPORT int llmb_sampling_trace(unsigned long long* out, int clear) { return llmb_read_trace(out, clear); }

LLMB_EXPORT int llmb_sample_rows(float* logits, int stride, int n_rows, int vocab,
                                 const float* params, const int* iparams, int* recent,
                                 int* recent_len, int recent_cap,
                                 unsigned long long* rng, int* out, int* status, int record,
                                 const int* state_rows, cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(n_rows > 0 && vocab > 0 && stride >= vocab, "sample: bad sizes");
    LLMB_REQUIRE(recent == nullptr || recent_cap > 0, "sample: recent window without capacity");
    sample_rows_kernel<<<n_rows, THREADS, 0, stream>>>(
        logits, stride, vocab, (const float4*)params, (const int2*)iparams, recent, recent_len,
        recent_cap, rng, out, status, record, state_rows);
    return check_launch("sample_rows");
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_argmax_rows)
LLMB_PACKED(llmb_sample_rows)
