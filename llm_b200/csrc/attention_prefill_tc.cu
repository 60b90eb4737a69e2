// Prefill attention on the fifth-generation tensor cores: S = Q K^T and O = P V as
// tcgen05.mma with accumulators in tensor memory, keys and values brought page by page from
// the cache by TMA, the softmax in between on the CUDA cores with one thread per query row.
//
// What it computes is what attention_prefill.cu computes (the flash prefill of
// MythEclipse/llm, apps/engine/kernels/gpu.cu:1444-1655: online softmax with a running
// (max, sum) per row and the accumulator rescaled by exp(m_old - m_new), probabilities as the
// left operand of the second product, heaviest query tile first), for head size 128.
//
// One block serves 128 queries of one head of one sequence and walks the visible keys in
// blocks of 128 (two cache pages):
//
// * warp 0, one lane: TMA. Q once (two 64-column boxes of 128 rows); per key block the two
//   pages of K and of V for the block's kv head, four 64 x 64 boxes each, into a two-stage ring.
// * warp 1, one lane: issues the products. S[128 q, 128 keys] = Q K^T (8 instructions of K=16
//   over the head dimension, both operands K-major in shared memory) into tensor-memory
//   columns 0-127; later PV[128 q, 128 d] = P V with P read from tensor memory (columns
//   256-319, bfloat16 pairs) and V from shared memory as an MN-major operand (its rows are
//   keys, the contiguous direction is d), into columns 128-255.
// * warps 2-5: thread r owns query row r. It reads its row of S twice from tensor memory
//   (first the maximum, then the exponentials: nothing of the row is kept in registers),
//   writes P back to tensor memory, and after the second product adds PV into its 128
//   accumulator registers, rescaled. Rows need no exchange between threads.
//
// The key block's keys beyond a query's own position are masked by value (-inf), so the
// diagonal needs no special path; blocks wholly above the tile's diagonal are never loaded.
// All waits are bounded by a clock limit and report through the status word of this library.
#include "tc.cuh"

using namespace llmb;
using namespace llmb::tc;

LLMB_DEFINE_LAST_ERROR(llmb_attention_prefill_tc)

namespace {

constexpr int HD = 128;                 // head dimension served
constexpr int BQ = 128;                 // queries per block = lanes of tensor memory
constexpr int BKV = 128;                // keys per step = two pages
constexpr int STAGES = 2;
constexpr int THREADS = 192;
constexpr int HALF_BYTES = 128 * 64 * 2;          // a [128 rows, 64 columns] piece: 16 KB
constexpr int TILE_BYTES = 2 * HALF_BYTES;        // Q, or the K or V of one key block: 32 KB
constexpr int BOX_BYTES = 64 * 64 * 2;            // one page, one 64-column half: 8 KB
constexpr uint32_t S_COL = 0, PV_COL = 128, P_COL = 256, TMEM_COLS = 512;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int table_stride, int ring_pages, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out, int out_stride,
                            int n_heads, int n_kv_heads, float scale_log2, int* status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = base;
    unsigned char* k_tiles = base + TILE_BYTES;
    unsigned char* v_tiles = k_tiles + STAGES * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_tiles + STAGES * TILE_BYTES);
    uint64_t* q_full = bars;
    uint64_t* kv_full = bars + 1;             // [STAGES]
    uint64_t* kv_empty = kv_full + STAGES;    // [STAGES]
    uint64_t* s_full = kv_empty + STAGES;     // S is complete
    uint64_t* p_full = s_full + 1;            // P is written (and S has been read)
    uint64_t* o_full = p_full + 1;            // PV is complete
    uint64_t* o_free = o_full + 1;            // PV has been read
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    int seq = blockIdx.z, head = blockIdx.y;
    int first_token = cu_seqlens[seq];
    int n_new = cu_seqlens[seq + 1] - first_token;
    int n_tiles = (n_new + BQ - 1) / BQ;
    if ((int)blockIdx.x >= n_tiles) return;                  // uniform for the block: nothing is allocated yet
    int tile = n_tiles - 1 - blockIdx.x;                     // the heaviest tile first
    int start = seq_lens[seq] - n_new;
    int kv_head = head / (n_heads / n_kv_heads);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int tile_last_pos = start + min(tile * BQ + BQ - 1, n_new - 1);
    int n_blocks = tile_last_pos / BKV + 1;
    const int* pages = block_table + (size_t)seq * table_stride;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(q_full), 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&kv_full[s]), 1);
            mbar_init(smem_u32(&kv_empty[s]), 1);
        }
        mbar_init(smem_u32(s_full), 1);
        mbar_init(smem_u32(p_full), 128);
        mbar_init(smem_u32(o_full), 1);
        mbar_init(smem_u32(o_free), 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t bar = smem_u32(q_full);
            mbar_expect_tx(bar, TILE_BYTES);
            for (int h = 0; h < 2; ++h)
                tma_load_2d(smem_u32(q_tile + h * HALF_BYTES), &map_q, bar, head * HD + h * 64,
                            first_token + tile * BQ);
            for (int kb = 0; kb < n_blocks; ++kb) {
                int s = kb % STAGES;
                uint32_t round = (uint32_t)(kb / STAGES);
                if (!mbar_wait(smem_u32(&kv_empty[s]), (round & 1) ^ 1, abort_flag, status, 11)) break;
                bar = smem_u32(&kv_full[s]);
                mbar_expect_tx(bar, 2 * TILE_BYTES);
                for (int p = 0; p < 2; ++p) {
                    int page = pages[(kb * 2 + p) % ring_pages];
                    int row = (page * n_kv_heads + kv_head) * LLMB_PAGE;
                    for (int h = 0; h < 2; ++h) {
                        // piece h of the tile holds 128 key rows: page 0 then page 1
                        uint32_t offset = (uint32_t)(s * TILE_BYTES + h * HALF_BYTES + p * BOX_BYTES);
                        tma_load_2d(smem_u32(k_tiles + offset), &map_k, bar, h * 64, row);
                        tma_load_2d(smem_u32(v_tiles + offset), &map_v, bar, h * 64, row);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // D 32-bit, A and B bfloat16, M = 128, N = 128; the second product takes B MN-major
            constexpr uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) |
                                          ((uint32_t)(BQ >> 4) << 24);
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                          ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            auto issue_qk = [&](int s) {
                uint32_t q0 = smem_u32(q_tile), k0 = smem_u32(k_tiles + s * TILE_BYTES);
#pragma unroll
                for (int j = 0; j < HD / 16; ++j) {
                    uint32_t off = (uint32_t)((j >> 2) * HALF_BYTES + (j & 3) * 32);
                    tcgen05_mma(tmem_base + S_COL, smem_desc(q0 + off), smem_desc(k0 + off), idesc_qk, j > 0 ? 1u : 0u);
                }
                tcgen05_commit(smem_u32(s_full));
            };
            bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, status, 12) &&
                      mbar_wait(smem_u32(&kv_full[0]), 0, abort_flag, status, 13);
            if (ok) {
                tcgen05_fence_after();
                issue_qk(0);
            }
            for (int kb = 0; kb < n_blocks && ok; ++kb) {
                int s = kb % STAGES;
                ok = mbar_wait(smem_u32(p_full), kb & 1, abort_flag, status, 14);
                if (ok && kb > 0) ok = mbar_wait(smem_u32(o_free), (kb - 1) & 1, abort_flag, status, 15);
                if (!ok) break;
                tcgen05_fence_after();
                uint32_t v0 = smem_u32(v_tiles + s * TILE_BYTES);
#pragma unroll
                for (int j = 0; j < BKV / 16; ++j)        // 16 keys a step: 8 columns of P, 2048 bytes of V rows
                    tcgen05_mma_ts(tmem_base + PV_COL, tmem_base + P_COL + j * 8,
                                   smem_desc_mn(v0 + j * 2048, HALF_BYTES), idesc_pv, j > 0 ? 1u : 0u);
                tcgen05_commit(smem_u32(o_full));
                tcgen05_commit(smem_u32(&kv_empty[s]));
                if (kb + 1 < n_blocks) {
                    int s1 = (kb + 1) % STAGES;
                    ok = mbar_wait(smem_u32(&kv_full[s1]), ((kb + 1) / STAGES) & 1, abort_flag, status, 13);
                    if (!ok) break;
                    tcgen05_fence_after();
                    issue_qk(s1);
                }
            }
        }
    } else {
        int quarter = warp & 3;
        int row = quarter * 32 + lane;                       // query row of the tile = lane of tensor memory
        int q_index = tile * BQ + row;                       // among the sequence's new tokens
        int pos = start + q_index;
        uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float acc[HD];
#pragma unroll
        for (int d = 0; d < HD; ++d) acc[d] = 0.f;
        float run_max = -INFINITY, run_sum = 0.f;
        bool ok = true;
        for (int kb = 0; kb < n_blocks && ok; ++kb) {
            ok = mbar_wait(smem_u32(s_full), kb & 1, abort_flag, status, 16);
            if (!ok) break;
            tcgen05_fence_after();
            int key0 = kb * BKV;
            // first reading of the row: its maximum over the visible keys
            float block_max = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < BKV; c += 32) {
                uint32_t r[32];
                tmem_ld32(lane_addr + S_COL + c, r);
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (key0 + c + j <= pos) block_max = fmaxf(block_max, __uint_as_float(r[j]));
            }
            float new_max = fmaxf(run_max, block_max);       // finite for a real row: key 0 is visible
            float alpha = fast_exp2((run_max - new_max) * scale_log2);
            float shift = new_max * scale_log2;
            run_max = new_max;
            // second reading: probabilities, written back as bfloat16 pairs
            float add = 0.f;
#pragma unroll 1
            for (int c = 0; c < BKV; c += 32) {
                uint32_t r[32], packed[16];
                tmem_ld32(lane_addr + S_COL + c, r);
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float p0 = key0 + c + j <= pos ? fast_exp2(fmaf(__uint_as_float(r[j]), scale_log2, -shift)) : 0.f;
                    float p1 = key0 + c + j + 1 <= pos ? fast_exp2(fmaf(__uint_as_float(r[j + 1]), scale_log2, -shift)) : 0.f;
                    add += p0 + p1;
                    packed[j >> 1] = pack2(p0, p1);
                }
                tmem_st16(lane_addr + P_COL + (c >> 1), packed);
            }
            run_sum = run_sum * alpha + add;
            tmem_st_wait();
            tcgen05_fence_before();
            mbar_arrive(smem_u32(p_full));
            // the second product, then this block's share of the output
            ok = mbar_wait(smem_u32(o_full), kb & 1, abort_flag, status, 17);
            if (!ok) break;
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                uint32_t r[32];
                tmem_ld32(lane_addr + PV_COL + c, r);
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(acc[c + j], alpha, __uint_as_float(r[j]));
            }
            tcgen05_fence_before();
            mbar_arrive(smem_u32(o_free));
        }
        if (ok && q_index < n_new) {
            float inv = 1.0f / run_sum;
            __nv_bfloat16* o = out + (size_t)(first_token + q_index) * out_stride + (size_t)head * HD;
#pragma unroll
            for (int d = 0; d < HD; d += 8) {
                uint4 packed;
                packed.x = pack2(acc[d] * inv, acc[d + 1] * inv);
                packed.y = pack2(acc[d + 2] * inv, acc[d + 3] * inv);
                packed.z = pack2(acc[d + 4] * inv, acc[d + 5] * inv);
                packed.w = pack2(acc[d + 6] * inv, acc[d + 7] * inv);
                *reinterpret_cast<uint4*>(o + d) = packed;
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 100; ++i) __nanosleep(10000);
        __syncthreads();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

LLMB_EXPORT int llmb_attention_prefill_tc_status() {
    int* s = status_word();
    if (!s) return -1;
    int v = *s;
    *s = 0;
    return v;
}

LLMB_EXPORT int llmb_attention_prefill_tc_supports(int n_heads, int n_kv_heads, int head_dim, int window) {
    LLMB_REQUIRE(window == 0, "attention_prefill_tc: a window of %d is not served", window);
    LLMB_REQUIRE(n_kv_heads > 0 && n_heads % n_kv_heads == 0,
                 "attention_prefill_tc: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    LLMB_REQUIRE(head_dim == HD, "attention_prefill_tc: head_dim %d (served: %d)", head_dim, HD);
    return LLMB_OK;
}

// q: the fused projection of the new tokens [n_tokens, q_stride] (queries in its first columns);
// k_cache, v_cache: one layer of the paged cache [n_pages, n_kv_heads, 64, 128]; the rest as in
// llmb_attention_prefill. out must be 16-byte aligned with a row stride that is a multiple of 8.
LLMB_EXPORT int llmb_attention_prefill_tc(const void* q, int q_stride, int n_tokens, const void* k_cache,
                                          const void* v_cache, int n_pages, const int* block_table,
                                          int table_stride, int ring_pages, const int* cu_seqlens,
                                          const int* seq_lens, void* out, int out_stride, int n_seqs,
                                          int max_new, int n_heads, int n_kv_heads, int head_dim,
                                          float scale, int window, cudaStream_t stream) {
    if (n_seqs == 0 || max_new == 0) return LLMB_OK;
    int code = llmb_attention_prefill_tc_supports(n_heads, n_kv_heads, head_dim, window);
    if (code) return code;
    LLMB_REQUIRE(n_seqs <= 65535 && n_heads <= 65535 && ring_pages > 0 && n_pages > 0, "attention_prefill_tc: bad sizes");
    LLMB_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0,
                 "attention_prefill_tc: operands must be 16-byte aligned with row strides that are multiples of 8");
    CUtensorMap map_q, map_k, map_v;
    if ((code = make_map_2d(&map_q, q, n_tokens, (long long)n_heads * HD, q_stride, 64, BQ))) return code;
    long long cache_rows = (long long)n_pages * n_kv_heads * LLMB_PAGE;
    if ((code = make_map_2d(&map_k, k_cache, cache_rows, HD, HD, 64, LLMB_PAGE))) return code;
    if ((code = make_map_2d(&map_v, v_cache, cache_rows, HD, HD, 64, LLMB_PAGE))) return code;
    size_t smem = 1024 + (size_t)(1 + 2 * STAGES) * TILE_BYTES + 16 * 8 + 16;
    static bool configured = false;
    if (!configured) {
        LLMB_CUDA(cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    int* status = status_word();
    int* status_dev = nullptr;
    if (status) cudaHostGetDevicePointer((void**)&status_dev, status, 0);
    dim3 grid((max_new + BQ - 1) / BQ, n_heads, n_seqs);
    attention_prefill_tc_kernel<<<grid, THREADS, smem, stream>>>(
        map_q, map_k, map_v, block_table, table_stride, ring_pages, cu_seqlens, seq_lens,
        (__nv_bfloat16*)out, out_stride, n_heads, n_kv_heads, scale * 1.4426950408889634f, status_dev);
    return check_launch("attention_prefill_tc");
}
