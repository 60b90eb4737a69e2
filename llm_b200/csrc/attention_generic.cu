// Causal grouped-query attention of new tokens over the paged cache, for any
// head size, head count, group size and window: the kernel of the true 32-bit
// path and the fallback of the bfloat16 path.
//
// One block per (token, query head), four warps; warp w takes the visible keys
// first + w, first + w + 4, ... key after key (four of them fetched at a time) with the lanes spread over
// the head dimension (the shape of attention_split in MythEclipse/llm,
// apps/engine/kernels/gpu.cu:649-733), keeps a running (max, sum, weighted
// values) and the four partial results are merged in a fixed order with
// out = sum_i acc_i e^(m_i - m) / sum_i l_i e^(m_i - m) (gpu.cu:745-760).
// Scores, softmax statistics and the weighted sum are 32-bit.
//
// Which keys a query sees depends only on its own position and the window:
// key j is visible to a query at position p iff j <= p and (window == 0 or
// j > p - window) (causal rule: apps/engine/src/compute.rs:1088). The order in
// which they are reduced depends only on p and the window too, so the result
// for a token does not depend on the batch or on how the tokens were cut into
// steps. The new tokens' keys must already be in the cache.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_attention_generic)

constexpr int MAX_PER_LANE = LLMB_MAX_HEAD_DIM / 32;   // elements of a head per lane
constexpr int WARPS = 4;

// AHEAD: keys a warp fetches together. Four hide the loads' latency where a step has few blocks
// (decoding); with thousands of blocks the SMs are full of other blocks' work and the registers
// of one key at a time keep more of them resident.
template <typename T, int AHEAD>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                         const T* __restrict__ v_cache, const int* __restrict__ block_table,
                         int table_stride, int ring_pages, const int* __restrict__ tok_pos,
                         const int* __restrict__ tok_seq, T* __restrict__ out, int out_stride,
                         int n_heads, int n_kv_heads, int head_dim, float scale, int window) {
    int t = blockIdx.x, head = blockIdx.y;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int kv_head = head / (n_heads / n_kv_heads);
    int pos = tok_pos[t];
    int b = tok_seq[t];
    int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* pages = block_table + (size_t)b * table_stride;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* q_row = q + (size_t)t * q_stride + (size_t)head * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        int d = lane + 32 * i;
        qv[i] = d < head_dim ? to_float(q_row[d]) : 0.f;
        acc[i] = 0.f;
    }
    float running_max = -INFINITY, running_sum = 0.f;

    // AHEAD keys of this warp are read together (their loads overlap), then folded into the running
    // state one after the other: the arithmetic and its order are those of one key per iteration.
    for (int j0 = first + warp; j0 <= pos; j0 += WARPS * AHEAD) {
        float kv[AHEAD][MAX_PER_LANE], vv[AHEAD][MAX_PER_LANE];
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            int j = j0 + u * WARPS;
            bool visible = j <= pos;
            int page = visible ? pages[(j / LLMB_PAGE) % ring_pages] : 0;
            size_t offset = (((size_t)page * n_kv_heads + kv_head) * LLMB_PAGE + (j % LLMB_PAGE)) * head_dim;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                int d = lane + 32 * i;
                bool live = visible && d < head_dim;
                kv[u][i] = live ? to_float(k_cache[offset + d]) : 0.f;
                vv[u][i] = live ? to_float(v_cache[offset + d]) : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < AHEAD; ++u) {
            if (j0 + u * WARPS > pos) break;
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                int d = lane + 32 * i;
                if (d < head_dim) dot = fmaf(qv[i], kv[u][i], dot);
            }
            float score = warp_sum(dot) * scale;
            float new_max = fmaxf(running_max, score);
            float rescale = expf(running_max - new_max);    // exp(-inf) = 0 on the first key
            float p = expf(score - new_max);
            running_sum = running_sum * rescale + p;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; ++i) {
                int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(p, vv[u][i], acc[i] * rescale);
            }
            running_max = new_max;
        }
    }

    __shared__ float part_acc[WARPS][MAX_PER_LANE * 32];
    __shared__ float part_max[WARPS], part_sum[WARPS];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) part_acc[warp][lane + 32 * i] = acc[i];
    if (lane == 0) { part_max[warp] = running_max; part_sum[warp] = running_sum; }
    __syncthreads();
    if (warp == 0) {
        float m = part_max[0];
#pragma unroll
        for (int w = 1; w < WARPS; ++w) m = fmaxf(m, part_max[w]);
        float weight[WARPS], denom = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            weight[w] = part_max[w] == -INFINITY ? 0.f : expf(part_max[w] - m);
            denom += part_sum[w] * weight[w];
        }
        T* o = out + (size_t)t * out_stride + (size_t)head * head_dim;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            int d = lane + 32 * i;
            if (d < head_dim) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) v += part_acc[w][d] * weight[w];
                o[d] = from_float<T>(v / denom);
            }
        }
    }
}

LLMB_EXPORT int llmb_attention_generic(const void* q, int q_stride, const void* k_cache,
                                       const void* v_cache, const int* block_table,
                                       int table_stride, int ring_pages, const int* tok_pos,
                                       const int* tok_seq, void* out, int out_stride, int dtype,
                                       int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                       float scale, int window, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(head_dim > 0 && head_dim <= 32 * MAX_PER_LANE,
                 "attention_generic: head_dim %d exceeds %d", head_dim, 32 * MAX_PER_LANE);
    LLMB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
                 "attention_generic: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    LLMB_REQUIRE(n_heads <= 65535 && ring_pages > 0 && window >= 0, "attention_generic: bad sizes");
    dim3 grid(n_tokens, n_heads);
    bool few = (long long)n_tokens * n_heads < 4096;       // the result is the same either way
#define LLMB_GENERIC(T, AHEAD)                                                                          \
    attention_generic_kernel<T, AHEAD><<<grid, WARPS * 32, 0, stream>>>(                                 \
        (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, block_table, table_stride,         \
        ring_pages, tok_pos, tok_seq, (T*)out, out_stride, n_heads, n_kv_heads, head_dim, scale, window)
    if (dtype == LLMB_DTYPE_F32) {
        if (few) LLMB_GENERIC(float, 4); else LLMB_GENERIC(float, 1);
    } else if (dtype == LLMB_DTYPE_BF16) {
        if (few) LLMB_GENERIC(__nv_bfloat16, 4); else LLMB_GENERIC(__nv_bfloat16, 1);
    } else {
        return fail(LLMB_ERR_ARGUMENT, "attention_generic: unknown dtype %d", dtype);
    }
#undef LLMB_GENERIC
    return check_launch("attention_generic");
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_attention_generic)
