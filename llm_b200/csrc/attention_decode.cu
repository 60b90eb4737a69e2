// Decode attention: one new query per sequence over that sequence's pages of
// the cache, bfloat16, split over the keys.
//
// The structure is attention_split + attention_combine of MythEclipse/llm
// (apps/engine/kernels/gpu.cu:649-762): blocks take slices of the positions,
// each writes (weighted values, max, sum) partials, and a second kernel merges
// them with out = sum_i acc_i e^(m_i - m) / sum_i l_i e^(m_i - m). What differs
// is the inside of a block. The step is bound by reading keys and values once,
// so a block serves one (sequence, kv head): the Hq/Hkv query heads that share
// those keys ride along as rows of one tensor-core tile, and the keys and
// values of a page (64 positions, contiguous per kv head) stream through shared
// memory with cp.async three pages deep.
//
// * grid (splits, kv heads, sequences); a block's pages are an even share of
//   the sequence's pages, computed from the device-side length, so a captured
//   launch stays right as sequences grow;
// * four warps; each takes 16 of a page's 64 keys: S = Q K^T as
//   mma.sync.m16n8k16 with K fragments from ldmatrix, softmax statistics in
//   32-bit registers (base-2 exponentials, scale folded in), P V with V
//   fragments from ldmatrix.trans; each warp keeps its own running (max, sum,
//   acc) and the four are merged once at the end in a fixed order;
// * rows of the tile are the query heads of the group: up to 8.
//
// Refused (the generic kernel serves them): a window, groups above 8, head
// sizes that are no multiple of 16 or exceed 128, 32-bit caches.
#include "common.cuh"
#include "mma.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_attention_decode)

constexpr int WARPS = 4;
constexpr int PAD = 8;                       // bf16 elements of row padding (bank spread)
// Pages in the ring of a block: as many as fit in about 110 KB (two blocks an SM), between 3 and 8.
// A small head size has small pages; it needs more of them in flight to keep HBM busy.
// Pages per stage of the ring: two where a page is small (head sizes up to 64), so that the fixed
// cost of a stage (the barrier, the wait for its copies) is paid once per 128 keys.
template <int D>
__host__ __device__ constexpr int pages_per_stage() { return D <= 64 ? 2 : 1; }

template <int D>
__host__ __device__ constexpr int stages_for() {
    constexpr int bytes = pages_per_stage<D>() * 2 * LLMB_PAGE * (D + PAD) * 2;
    constexpr int fit = (110 * 1024) / bytes;
    return fit < 3 ? 3 : fit > 8 ? 8 : fit;
}

// partial layout: acc [seq, head, split, D] floats; stats [seq, head, split, 2] = (max, sum),
// max in base-2 units (score * scale * log2 e).
template <int D>
__global__ void __launch_bounds__(WARPS * 32)
attention_decode_split_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                              const __nv_bfloat16* __restrict__ k_cache,
                              const __nv_bfloat16* __restrict__ v_cache,
                              const int* __restrict__ block_table, int table_stride, int ring_pages,
                              const int* __restrict__ seq_lens, const int* __restrict__ seq_order,
                              float* __restrict__ part_acc, float* __restrict__ part_stats,
                              __nv_bfloat16* __restrict__ out, int out_stride,
                              int n_heads, int n_kv_heads, float scale_log2) {
    constexpr int LDS = D + PAD;
    constexpr int PAGE_ELEMS = LLMB_PAGE * LDS;
    constexpr int STAGES = stages_for<D>();
    constexpr int UNIT = pages_per_stage<D>();
    constexpr int STAGE_ELEMS = UNIT * 2 * PAGE_ELEMS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [STAGES][UNIT][k, v][64][LDS]

    // The kernel before this one in a step writes the queries and the newest position of the
    // cache; lengths, page tables and every older page are already final. So the first pages of
    // this block's slice are fetched before griddep_wait(), except the page that holds the
    // newest position.
    griddep_launch();
    LLMB_STAMP(0, 0);                               // the block has started
    // blocks start in the order of blockIdx; seq_order (optional) lists the sequences by falling
    // length, so that the longest ones start first and the short ones fill the end of the step
    int split = blockIdx.x, n_splits = gridDim.x, kv_head = blockIdx.y;
    int seq = seq_order ? seq_order[blockIdx.z] : (int)blockIdx.z;
    int group = n_heads / n_kv_heads;
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    int len = seq_lens[seq];
    int n_pages = (len + LLMB_PAGE - 1) / LLMB_PAGE;
    int per_split = (n_pages + n_splits - 1) / n_splits;
    int page_begin = min(split * per_split, n_pages);
    int page_end = min(page_begin + per_split, n_pages);
    const int* pages = block_table + (size_t)seq * table_stride;

    auto load_page = [&](int logical_page, int stage, int place) {
        int page = pages[logical_page % ring_pages];
        size_t base = ((size_t)page * n_kv_heads + kv_head) * LLMB_PAGE * D;
        __nv_bfloat16* ks = smem + (size_t)stage * STAGE_ELEMS + (size_t)place * 2 * PAGE_ELEMS;
        __nv_bfloat16* vs = ks + PAGE_ELEMS;
        constexpr int CHUNKS_PER_ROW = D / 8;
        for (int c = tid; c < LLMB_PAGE * CHUNKS_PER_ROW; c += WARPS * 32) {
            int row = c / CHUNKS_PER_ROW, col = (c % CHUNKS_PER_ROW) * 8;
            cp_async16(ks + row * LDS + col, k_cache + base + (size_t)row * D + col);
            cp_async16(vs + row * LDS + col, v_cache + base + (size_t)row * D + col);
        }
    };
    int n_my = page_end - page_begin;
    int n_units = (n_my + UNIT - 1) / UNIT;         // stages' worth of pages in this slice
    // unit u = pages page_begin + u * UNIT ... ; `hold_back`: leave out the page of the newest position
    int late_unit = -1, late_place = 0;
    auto load_unit = [&](int u, int stage, bool hold_back) {
#pragma unroll
        for (int place = 0; place < UNIT; ++place) {
            int logical = page_begin + u * UNIT + place;
            if (logical >= page_end) break;
            if (hold_back && logical == n_pages - 1) {
                late_unit = u;
                late_place = place;
            } else {
                load_page(logical, stage, place);
            }
        }
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < n_units) load_unit(s, s, true);
        cp_async_commit();
    }
    griddep_wait();
    LLMB_STAMP(1, 0);                               // the kernel before this one has completed
    if (late_unit >= 0) {
        load_page(page_begin + late_unit * UNIT + late_place, late_unit, late_place);
        cp_async_commit();
    }

    // Q fragments of this warp's lane: row g = head kv_head * group + g (zero beyond the group)
    uint32_t qa0[D / 16], qa2[D / 16];
    {
        const __nv_bfloat16* q_row = q + (size_t)seq * q_stride + (size_t)(kv_head * group + g) * D;
        bool valid = g < group;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qa0[ks] = valid ? *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + 2 * t) : 0u;
            qa2[ks] = valid ? *reinterpret_cast<const uint32_t*>(q_row + ks * 16 + 8 + 2 * t) : 0u;
        }
    }

    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    float run_max = -INFINITY, run_sum = 0.f;      // for head row g (this lane's keys only for the sum)

    for (int i = 0; i < n_units; ++i) {
        // the newest page, fetched late, is in the last unit of its slice and the youngest group
        if (late_unit >= 0 && i == n_units - 1) cp_async_wait<0>();
        else cp_async_wait<STAGES - 2>();
        __syncthreads();                            // unit i landed; everyone is done with unit i - 1
        if (i == 0) LLMB_STAMP(2, 0);               // the first pages have landed
        if (i + STAGES - 1 < n_units) load_unit(i + STAGES - 1, (i + STAGES - 1) % STAGES, false);
        cp_async_commit();

#pragma unroll
      for (int place = 0; place < UNIT; ++place) {
        int logical = page_begin + i * UNIT + place;
        if (logical >= page_end) break;
        const __nv_bfloat16* ks = smem + (size_t)(i % STAGES) * STAGE_ELEMS + (size_t)place * 2 * PAGE_ELEMS;
        const __nv_bfloat16* vs = ks + PAGE_ELEMS;
        int key_base = warp * 16;
        int first_key = logical * LLMB_PAGE + key_base;
        if (first_key >= len) continue;             // this warp's 16 keys are all beyond the sequence

        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kstep = 0; kstep < D / 16; ++kstep) {
            uint32_t b[4];
            int row = key_base + (lane >> 4) * 8 + (lane & 7);
            int col = kstep * 16 + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(b, ks + row * LDS + col);
            mma_bf16(s0, qa0[kstep], 0u, qa2[kstep], 0u, b[0], b[1]);
            mma_bf16(s1, qa0[kstep], 0u, qa2[kstep], 0u, b[2], b[3]);
        }
        // lane holds head g, keys first_key + 2t, +1 (s0) and first_key + 8 + 2t, +1 (s1)
        float v[4] = {s0[0], s0[1], s1[0], s1[1]};
        int key[4] = {first_key + 2 * t, first_key + 2 * t + 1, first_key + 8 + 2 * t, first_key + 9 + 2 * t};
        float local_max = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[j] = key[j] < len ? v[j] * scale_log2 : -INFINITY;
            local_max = fmaxf(local_max, v[j]);
        }
        local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 1));
        local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, 2));
        float new_max = fmaxf(run_max, local_max);      // finite: key first_key < len
        float rescale = exp2f(run_max - new_max);       // 0 on the first block (run_max = -inf)
        float p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) p[j] = exp2f(v[j] - new_max);
        run_sum = run_sum * rescale + (p[0] + p[1] + p[2] + p[3]);
        run_max = new_max;
        uint32_t pa0 = pack_bf16(p[0], p[1]), pa2 = pack_bf16(p[2], p[3]);
#pragma unroll
        for (int n = 0; n < D / 8; ++n) { acc[n][0] *= rescale; acc[n][1] *= rescale; }
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            uint32_t b[4];
            int row = key_base + ((lane >> 3) & 1) * 8 + (lane & 7);
            int col = (n + (lane >> 4)) * 8;
            ldmatrix_x4_trans(b, vs + row * LDS + col);
            mma_bf16(acc[n], pa0, 0u, pa2, 0u, b[0], b[1]);
            mma_bf16(acc[n + 1], pa0, 0u, pa2, 0u, b[2], b[3]);
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();                                 // the stage buffers are free: reuse them
    LLMB_STAMP(3, 0);                                // the slice's keys are done

    // merge the four warps: [WARPS][8 heads][D] weighted values, [WARPS][8] max and sum
    run_sum += __shfl_xor_sync(0xffffffffu, run_sum, 1);
    run_sum += __shfl_xor_sync(0xffffffffu, run_sum, 2);
    float* merge_acc = reinterpret_cast<float*>(smem_raw);
    float* merge_max = merge_acc + WARPS * 8 * D;
    float* merge_sum = merge_max + WARPS * 8;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        merge_acc[(warp * 8 + g) * D + n * 8 + 2 * t] = acc[n][0];
        merge_acc[(warp * 8 + g) * D + n * 8 + 2 * t + 1] = acc[n][1];
    }
    if (t == 0) { merge_max[warp * 8 + g] = run_max; merge_sum[warp * 8 + g] = run_sum; }
    __syncthreads();
    for (int idx = tid; idx < group * D; idx += WARPS * 32) {
        int head = idx / D, d = idx - head * D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, merge_max[w * 8 + head]);
        float value = 0.f, sum = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            float mw = merge_max[w * 8 + head];
            float weight = mw == -INFINITY ? 0.f : exp2f(mw - m);
            value += merge_acc[(w * 8 + head) * D + d] * weight;
            sum += merge_sum[w * 8 + head] * weight;
        }
        if (n_splits == 1) {                          // nothing to combine: this is the result
            out[(size_t)seq * out_stride + (size_t)(kv_head * group + head) * D + d] = __float2bfloat16_rn(value / sum);
            continue;
        }
        size_t slot = ((size_t)seq * n_heads + kv_head * group + head) * n_splits + split;
        part_acc[slot * D + d] = value;
        if (d == 0) { part_stats[slot * 2] = m; part_stats[slot * 2 + 1] = sum; }
    }
    LLMB_STAMP(4, 0);                                // the partial result is written
}

template <int D>
__global__ void attention_decode_combine_kernel(const float* __restrict__ part_acc,
                                                const float* __restrict__ part_stats,
                                                __nv_bfloat16* __restrict__ out, int out_stride,
                                                int n_heads, int n_splits) {
    griddep_launch();
    griddep_wait();
    int seq = blockIdx.y, head = blockIdx.x;
    size_t base = ((size_t)seq * n_heads + head) * n_splits;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, part_stats[(base + s) * 2]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float value = 0.f, sum = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            float ms = part_stats[(base + s) * 2];
            float weight = ms == -INFINITY ? 0.f : exp2f(ms - m);
            value += part_acc[(base + s) * D + d] * weight;
            sum += part_stats[(base + s) * 2 + 1] * weight;
        }
        out[(size_t)seq * out_stride + (size_t)head * D + d] = __float2bfloat16_rn(value / sum);
    }
}

template <int D>
static int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                  const int* block_table, int table_stride, int ring_pages, const int* seq_lens,
                  const int* seq_order, void* out, int out_stride, float* scratch, int n_seqs, int n_heads,
                  int n_kv_heads, float scale, int n_splits, cudaStream_t stream) {
    constexpr int LDS = D + PAD;
    constexpr int STAGES = stages_for<D>();
    size_t stage_bytes = (size_t)STAGES * pages_per_stage<D>() * 2 * LLMB_PAGE * LDS * sizeof(__nv_bfloat16);
    size_t merge_bytes = (size_t)(WARPS * 8 * D + 2 * WARPS * 8) * sizeof(float);
    size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
    static bool configured = false;
    if (!configured) {
        LLMB_CUDA(cudaFuncSetAttribute(attention_decode_split_kernel<D>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    float* part_acc = scratch;
    float* part_stats = scratch + (size_t)n_seqs * n_heads * n_splits * D;
    dim3 grid(n_splits, n_kv_heads, n_seqs);
    llmb::launch(attention_decode_split_kernel<D>, grid, WARPS * 32, smem, stream, true,
                 (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache,
                 (const __nv_bfloat16*)v_cache, block_table, table_stride, ring_pages, seq_lens, seq_order,
                 part_acc, part_stats, (__nv_bfloat16*)out, out_stride, n_heads, n_kv_heads, scale * 1.4426950408889634f);
    int code = check_launch("attention_decode_split");
    if (code || n_splits == 1) return code;
    llmb::launch(attention_decode_combine_kernel<D>, dim3(n_heads, n_seqs), D >= 128 ? 128 : 64, 0, stream, true,
                 (const float*)part_acc, (const float*)part_stats, (__nv_bfloat16*)out, out_stride, n_heads, n_splits);
    return check_launch("attention_decode_combine");
}

// The stamps of the last launches in a build with -DLLMB_TRACE (see common.cuh): rows are linear block
// ids (x fastest), only the first LLMB_TRACE_BLOCKS of them; 1 in a build without.
LLMB_EXPORT int llmb_attention_decode_trace(unsigned long long* out, int clear) { return llmb_read_trace(out, clear); }

// Floats of scratch for a call: partial values and (max, sum) per (sequence, head, split).
LLMB_EXPORT long long llmb_attention_decode_scratch_floats(int n_seqs, int n_heads, int head_dim,
                                                           int n_splits) {
    return (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
}

// Whether the kernel serves this shape; the text of the refusal is in last_error.
LLMB_EXPORT int llmb_attention_decode_supports(int n_heads, int n_kv_heads, int head_dim, int window) {
    LLMB_REQUIRE(window == 0, "attention_decode: a window of %d is not served", window);
    LLMB_REQUIRE(n_kv_heads > 0 && n_heads % n_kv_heads == 0 && n_heads / n_kv_heads <= 8,
                 "attention_decode: %d heads over %d kv heads (groups up to 8)", n_heads, n_kv_heads);
    LLMB_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128,
                 "attention_decode: head_dim %d (served: 32, 64, 96, 128)", head_dim);
    return LLMB_OK;
}

LLMB_EXPORT int llmb_attention_decode(const void* q, int q_stride, const void* k_cache,
                                      const void* v_cache, const int* block_table, int table_stride,
                                      int ring_pages, const int* seq_lens, const int* seq_order, void* out,
                                      int out_stride, float* scratch, long long scratch_floats, int n_seqs,
                                      int n_heads, int n_kv_heads, int head_dim, float scale,
                                      int window, int n_splits, cudaStream_t stream) {
    if (n_seqs == 0) return LLMB_OK;
    int code = llmb_attention_decode_supports(n_heads, n_kv_heads, head_dim, window);
    if (code) return code;
    LLMB_REQUIRE(n_splits >= 1 && n_splits <= 65535 && n_seqs <= 65535 && ring_pages > 0,
                 "attention_decode: bad sizes");
    LLMB_REQUIRE(q_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0,
                 "attention_decode: q must be 4-byte aligned with an even row stride");
    LLMB_REQUIRE(scratch != nullptr && scratch_floats >= llmb_attention_decode_scratch_floats(
                                                             n_seqs, n_heads, head_dim, n_splits),
                 "attention_decode: scratch too small");
#define ARGS q, q_stride, k_cache, v_cache, block_table, table_stride, ring_pages, seq_lens, seq_order, out, \
             out_stride, scratch, n_seqs, n_heads, n_kv_heads, scale, n_splits, stream
    switch (head_dim) {
        case 32: return launch<32>(ARGS);
        case 64: return launch<64>(ARGS);
        case 96: return launch<96>(ARGS);
        default: return launch<128>(ARGS);
    }
#undef ARGS
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_attention_decode)
