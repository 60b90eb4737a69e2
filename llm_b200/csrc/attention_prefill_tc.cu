// Prefill attention on the fifth-generation tensor cores: S = Q K^T and O = P V as
// tcgen05.mma with accumulators in tensor memory, keys and values brought page by page from
// the cache by TMA, the softmax in between on the CUDA cores with one thread per query row.
//
// What it computes is what attention_prefill.cu computes (the flash prefill of
// MythEclipse/llm, apps/engine/kernels/gpu.cu:1444-1655: online softmax with a running
// (max, sum) per row and the accumulator rescaled by exp(m_old - m_new), probabilities as the
// left operand of the second product, heaviest query tile first), for head sizes 64 and 128.
//
// One block serves 128 queries of one head of one sequence and walks the visible keys in
// blocks of 64 (one cache page):
//
// * warp 0, one lane: TMA for Q (once) and for the keys; warp 6, one lane: TMA for the values. 64 x 64
//   boxes, two buffers each for K and V with barriers of their own, so that a buffer is requested
//   again as soon as the product that read it is complete.
// * warp 1, one lane: issues the products. S[128 q, 64 keys] = Q K^T (K=16 steps over the head
//   dimension, both operands K-major in shared memory) into one of TWO score buffers in tensor memory
//   (columns 0-63 and 64-127); then O[128 q, d] += P V with P read from tensor memory and V from shared
//   memory as an MN-major operand (its rows are keys, the contiguous direction is d), accumulating in
//   columns 128... The scores of key block kb + 2 are issued right behind P V of key block kb, into the
//   buffer whose probabilities that product has just consumed: while the softmax works on one buffer,
//   the products fill the other, so neither side waits for the other's whole turn.
// * warps 2-5: thread r owns query row r. It reads its 64 scores from tensor memory once (both loads in
//   flight), keeps them in registers for the maximum and the exponentials, and writes P over the
//   buffer's first 32 columns. O stays in tensor memory over all key blocks; when a row's maximum
//   outgrows the exponent's reference by 2^8, its warp rescales O in place, behind the exponentials
//   and before P is released (rare after the first blocks). Rows need no exchange between threads.
// * 96 KB of shared memory, 256 columns of tensor memory and 120 registers a thread let two
//   blocks share an SM.
//
// How it got here, on a B200 at 2,048 / 8,192 tokens, 32 heads over 8 kv heads of 128: one score buffer
// of 128 keys read twice by the softmax threads, 53.0 / 573 us; a build with phase counters
// (-DLLMB_TRACE, microbench.py attention_prefill --timeline) showed each side idle for the other's
// whole turn (softmax threads 2,000 of 4,500 cycles a key block waiting for S, the product thread
// 3,000 waiting for P), and two blocks an SM did not fill the gaps. Two threads a row (8 softmax
// warps), one read of all 128 scores into registers, and half of the exponentials as a polynomial on
// the multiply-add units each measured slower (56.7, 60.2 and 55.9 us): the softmax is not short of
// threads or of special-function throughput, every added instruction costs issue slots that the
// product and TMA threads share. Two score buffers of 64 keys: 50.6 / 510 us; the values' TMA in a
// warp of its own (one lane waiting for two kinds of buffers delayed the keys): 46.2 / 498 us.
// One block an SM with two score buffers of 128 keys (all 512 columns of tensor memory) and two threads a
// row: 57.7 / 582 us. The two warps of a row sit on the same SM partition and reach their exponentials
// together (1,276 cycles for 64 of them a thread, the special-function unit's rate), and nothing runs
// under the reading of S and the meeting of the halves; two blocks an SM drift apart and fill each
// other's gaps. The same block with the two warps of a quarter taking the key blocks in turns (128
// scores a thread, the reference told through shared memory): 62.5 / 604 us, since each warp then has
// one of the two score buffers and waits through both products of its key block again. Two threads a
// row on the present layout (32 scores each): 48.9 / 513 us.
//
// The key block's keys beyond a query's own position are masked by value (-inf), so the
// diagonal needs no special path; blocks wholly above the tile's diagonal are never loaded.
// All waits are bounded by a clock limit and report through the status word of this library.
#include "tc.cuh"

using namespace llmb;
using namespace llmb::tc;

LLMB_DEFINE_LAST_ERROR(llmb_attention_prefill_tc)

namespace {

constexpr int BQ = 128;                 // queries per block = lanes of tensor memory
constexpr int BKV = 64;                 // keys per step = one cache page
constexpr int THREADS = 224;             // keys by TMA, products, four softmax warps, values by TMA
constexpr int Q_PIECE = 128 * 64 * 2;             // 128 query rows, 64 columns of the head: 16 KB
constexpr int KV_PIECE = 64 * 64 * 2;             // one page, 64 columns of the head: 8 KB
// tensor memory: two buffers of scores (64 columns of 32-bit values each), each overwritten in place
// by its probabilities (32 columns of bfloat16 pairs); O (head_dim columns) accumulates beside them
constexpr uint32_t S_COL = 0, O_COL = 128, TMEM_COLS = 256;

// A build with -DLLMB_TRACE adds up, per block, the SM clock cycles that one softmax thread and the
// product thread spend in each phase of the loop over key blocks (llmb_attention_prefill_tc_trace).
#ifdef LLMB_TRACE
#define LAPS_BEGIN long long lap_t = clock64(); long long laps[6] = {0, 0, 0, 0, 0, 0};
#define LAP(i) do { long long now_ = clock64(); laps[i] += now_ - lap_t; lap_t = now_; } while (0)
#define LAPS_END(first_slot, count, n_blocks)                                                       \
    do {                                                                                            \
        unsigned block_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;            \
        if (block_ < LLMB_TRACE_BLOCKS) {                                                           \
            for (int i_ = 0; i_ < (count); ++i_)                                                    \
                llmb_trace_buffer[block_ * LLMB_TRACE_SLOTS + (first_slot) + i_] = laps[i_];         \
            llmb_trace_buffer[block_ * LLMB_TRACE_SLOTS + LLMB_TRACE_SLOTS - 1] = (n_blocks);       \
        }                                                                                           \
    } while (0)
#else
#define LAPS_BEGIN
#define LAP(i) do { } while (0)
#define LAPS_END(first_slot, count, n_blocks) do { } while (0)
#endif

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
// HD: head dimension, 64 or 128 (one or two 64-column pieces per tile). Two blocks fit on an SM
// (96 KB of shared memory, 256 columns of tensor memory, at most 168 registers).
template <int HD>
__global__ void __launch_bounds__(THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int table_stride, int ring_pages, const int* __restrict__ cu_seqlens,
                            const int* __restrict__ seq_lens, const int* __restrict__ seq_order,
                            __nv_bfloat16* __restrict__ out, int out_stride,
                            int n_heads, int n_kv_heads, float scale_log2, int* status) {
    constexpr int PIECES = HD / 64;
    constexpr int Q_BYTES = PIECES * Q_PIECE;         // the block's queries
    constexpr int KV_BYTES = PIECES * KV_PIECE;       // the K or the V of one key block
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = base;
    unsigned char* k_tile = base + Q_BYTES;           // two buffers each: the next key block's K arrives
    unsigned char* v_tile = k_tile + 2 * KV_BYTES;    // under this block's products, its V under the softmax
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_tile + 2 * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;              // [2]
    uint64_t* k_empty = bars + 3;             // [2]
    uint64_t* v_full = bars + 5;              // [2]
    uint64_t* v_empty = bars + 7;             // [2]
    uint64_t* s_full = bars + 9;              // [2] a buffer's scores are complete
    uint64_t* p_full = bars + 11;             // [2] its probabilities are written and O has been rescaled
    uint64_t* o_full = bars + 13;             // a key block's P V has been added to O
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    griddep_launch();            // the next kernel may set itself up; this one needs the one before it whole
    griddep_wait();
    // seq_order (optional): sequences by falling length, so that the longest start first
    int seq = seq_order ? seq_order[blockIdx.z] : (int)blockIdx.z, head = blockIdx.x;
    int first_token = cu_seqlens[seq];
    int n_new = cu_seqlens[seq + 1] - first_token;
    int n_tiles = (n_new + BQ - 1) / BQ;
    if ((int)blockIdx.y >= n_tiles) return;                  // uniform for the block: nothing is allocated yet
    // blocks start in the order x, y, z: the heaviest tile of every head first, then the next
    // lighter one of every head, so that the light tiles fill the end of the triangle's work
    int tile = n_tiles - 1 - blockIdx.y;
    int start = seq_lens[seq] - n_new;
    int kv_head = head / (n_heads / n_kv_heads);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int tile_last_pos = start + min(tile * BQ + BQ - 1, n_new - 1);
    int n_blocks = tile_last_pos / BKV + 1;
    const int* pages = block_table + (size_t)seq * table_stride;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 14; ++i) mbar_init(smem_u32(&bars[i]), (i == 11 || i == 12) ? 128 : 1);
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

    if (warp == 0 || warp == 6) {
        // warp 0 brings Q and the keys, warp 6 the values: each waits only for its own buffers
        if (lane == 0) {
            bool keys = warp == 0;
            if (keys) {
                uint32_t bar = smem_u32(q_full);
                mbar_expect_tx(bar, Q_BYTES);
                for (int h = 0; h < PIECES; ++h)
                    tma_load_2d(smem_u32(q_tile + h * Q_PIECE), &map_q, bar, head * HD + h * 64,
                                first_token + tile * BQ);
            }
            const CUtensorMap* map = keys ? &map_k : &map_v;
            unsigned char* tiles = keys ? k_tile : v_tile;
            uint64_t* full = keys ? k_full : v_full;
            uint64_t* empty = keys ? k_empty : v_empty;
            for (int kb = 0; kb < n_blocks; ++kb) {
                int b = kb & 1;
                if (kb >= 2 && !mbar_wait(smem_u32(&empty[b]), ((kb >> 1) - 1) & 1, abort_flag, status, keys ? 11 : 12))
                    break;
                uint32_t bar = smem_u32(&full[b]);
                mbar_expect_tx(bar, KV_BYTES);
                int page = pages[kb % ring_pages];
                int row = (page * n_kv_heads + kv_head) * LLMB_PAGE;
                for (int h = 0; h < PIECES; ++h)
                    tma_load_2d(smem_u32(tiles + b * KV_BYTES + h * KV_PIECE), map, bar, h * 64, row);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // D 32-bit, A and B bfloat16, M = 128; S has N = 64 keys, O has N = HD with B MN-major
            constexpr uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BKV >> 3) << 17) |
                                          ((uint32_t)(BQ >> 4) << 24);
            constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                          ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
            // the descriptors of the tiles' first bytes are made once; a step inside a tile adds a constant
            // to the address field (this thread's instructions set the pace of the products)
            const uint64_t q_desc = smem_desc(smem_u32(q_tile));
            const uint64_t k_desc0 = smem_desc(smem_u32(k_tile)), v_desc0 = smem_desc_mn(smem_u32(v_tile), KV_PIECE);
            constexpr uint64_t BUFFER = (uint64_t)(KV_BYTES >> 4);       // the second buffer, in the address field
            // S[buffer kb & 1] = Q K(kb)^T; the buffer's last probabilities have been consumed by a
            // product that this thread issued earlier (products run in the order of their issue)
            auto issue_qk = [&](int kb) -> bool {
                int b = kb & 1;
                if (!mbar_wait(smem_u32(&k_full[b]), (kb >> 1) & 1, abort_flag, status, 14)) return false;
                tcgen05_fence_after();
#pragma unroll
                for (int j = 0; j < HD / 16; ++j) {
                    uint64_t q_off = (uint64_t)(((j >> 2) * Q_PIECE + (j & 3) * 32) >> 4);
                    uint64_t k_off = (uint64_t)(((j >> 2) * KV_PIECE + (j & 3) * 32) >> 4);
                    tcgen05_mma(tmem_base + S_COL + b * BKV, q_desc + q_off, k_desc0 + b * BUFFER + k_off, idesc_qk,
                                j > 0 ? 1u : 0u);
                }
                tcgen05_commit(smem_u32(&s_full[b]));
                tcgen05_commit(smem_u32(&k_empty[b]));
                return true;
            };
            LAPS_BEGIN
            bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, status, 13) && issue_qk(0);
            if (ok && n_blocks > 1) ok = issue_qk(1);
            LAP(4);
            for (int kb = 0; kb < n_blocks && ok; ++kb) {
                int b = kb & 1, phase = (kb >> 1) & 1;
                ok = mbar_wait(smem_u32(&p_full[b]), phase, abort_flag, status, 15);
                LAP(0);
                ok = ok && mbar_wait(smem_u32(&v_full[b]), phase, abort_flag, status, 16);
                LAP(1);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int j = 0; j < BKV / 16; ++j)        // 16 keys a step: 8 columns of P, 2048 bytes of V rows
                    tcgen05_mma_ts(tmem_base + O_COL, tmem_base + S_COL + b * BKV + j * 8,
                                   v_desc0 + b * BUFFER + (uint64_t)((j * 2048) >> 4), idesc_pv,
                                   (kb > 0 || j > 0) ? 1u : 0u);
                tcgen05_commit(smem_u32(o_full));
                tcgen05_commit(smem_u32(&v_empty[b]));
                LAP(2);
                // the scores of the key block after the next go where these probabilities were: the
                // softmax of the next key block runs meanwhile on the other buffer
                if (kb + 2 < n_blocks) ok = issue_qk(kb + 2);
                LAP(3);
            }
            LAPS_END(6, 5, n_blocks);
        }
    } else {
        int quarter = warp & 3;
        int row = quarter * 32 + lane;                       // query row of the tile = lane of tensor memory
        int q_index = tile * BQ + row;                       // among the sequence's new tokens
        int pos = start + q_index;
        uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float run_max = -INFINITY, run_sum = 0.f;
        bool ok = true;
        LAPS_BEGIN
        for (int kb = 0; kb < n_blocks && ok; ++kb) {
            int b = kb & 1;
            ok = mbar_wait(smem_u32(&s_full[b]), (kb >> 1) & 1, abort_flag, status, 17);
            LAP(0);
            if (!ok) break;
            __syncwarp();
            tcgen05_fence_after();
            int key0 = kb * BKV;
            bool whole = key0 + BKV - 1 <= pos;              // no key of the block is hidden from this row
            // The row's 64 scores are read from tensor memory once, both loads in flight, and stay in
            // registers for the maximum and for the exponentials.
            uint32_t s_addr = lane_addr + S_COL + b * BKV;
            uint32_t ra[32], rb[32];
            tmem_ld32_start(s_addr, ra);
            tmem_ld32_start(s_addr + 32, rb);
            float block_max = -INFINITY;
            auto row_max = [&](const uint32_t (&r)[32], int c) {
                if (whole) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2)
                        block_max = max3(block_max, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (key0 + c + j <= pos) block_max = fmaxf(block_max, __uint_as_float(r[j]));
                }
            };
            tmem_ld32_wait(ra);
            tmem_ld32_wait(rb);
            row_max(ra, 0);
            row_max(rb, 32);
            LAP(1);
            // The exponent's reference moves only when the block's maximum exceeds it by more than
            // 2^8 (softmax does not depend on the reference; probabilities up to 256 are as exact in
            // bfloat16 as those up to 1). O, which holds the sum in units of 2^-reference, is then
            // rescaled in place. The tensor-memory accesses are warp-wide, so the warp rescales when
            // any of its rows moves; the others multiply by one. A row that sees no key of this block
            // (the upper rows of a tile in its last key block) has the maximum -inf and never moves.
            bool move = kb == 0 || (block_max - run_max) * scale_log2 > 8.f;
            float new_max = move ? block_max : run_max;      // finite for a real row: key 0 is visible
            float alpha = (move && kb > 0) ? fast_exp2((run_max - new_max) * scale_log2) : 1.f;
            float shift = new_max * scale_log2;
            run_max = new_max;
            // probabilities, written over the scores' first columns as bfloat16 pairs (every score of
            // the buffer is in a register by now)
            float add = 0.f;
            auto to_probabilities = [&](const uint32_t (&r)[32], int c) {
                uint32_t packed[16];
                if (whole) {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float p0 = fast_exp2(fmaf(__uint_as_float(r[j]), scale_log2, -shift));
                        float p1 = fast_exp2(fmaf(__uint_as_float(r[j + 1]), scale_log2, -shift));
                        add += p0 + p1;
                        packed[j >> 1] = pack2(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float p0 = key0 + c + j <= pos ? fast_exp2(fmaf(__uint_as_float(r[j]), scale_log2, -shift)) : 0.f;
                        float p1 = key0 + c + j + 1 <= pos ? fast_exp2(fmaf(__uint_as_float(r[j + 1]), scale_log2, -shift)) : 0.f;
                        add += p0 + p1;
                        packed[j >> 1] = pack2(p0, p1);
                    }
                }
                tmem_st16(s_addr + (c >> 1), packed);
            };
            to_probabilities(ra, 0);
            to_probabilities(rb, 32);
            run_sum = run_sum * alpha + add;
            LAP(4);
            // O is rescaled behind the exponentials: the product before this one, which has to be
            // complete first, has had their time to finish, and the next one waits for the release below
            if (kb > 0) {
                ok = mbar_wait(smem_u32(o_full), (kb - 1) & 1, abort_flag, status, 18);
                if (!ok) break;
                __syncwarp();
                tcgen05_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(lane_addr + O_COL + c, r);
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                        tmem_st32(lane_addr + O_COL + c, r);
                    }
                }
            }
            LAP(3);
            tmem_st_wait();
            tcgen05_fence_before();
            mbar_arrive(smem_u32(&p_full[b]));
            LAP(5);
        }
#ifdef LLMB_TRACE
        if (threadIdx.x == 64) LAPS_END(0, 6, n_blocks);
#endif
        if (ok) ok = mbar_wait(smem_u32(o_full), (n_blocks - 1) & 1, abort_flag, status, 19);
        if (ok) {
            __syncwarp();
            tcgen05_fence_after();
            float inv = 1.0f / run_sum;
            __nv_bfloat16* o = out + (size_t)(first_token + q_index) * out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t r[32];
                tmem_ld32(lane_addr + O_COL + c, r);
                if (q_index < n_new) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 packed;
                        packed.x = pack2(__uint_as_float(r[d]) * inv, __uint_as_float(r[d + 1]) * inv);
                        packed.y = pack2(__uint_as_float(r[d + 2]) * inv, __uint_as_float(r[d + 3]) * inv);
                        packed.z = pack2(__uint_as_float(r[d + 4]) * inv, __uint_as_float(r[d + 5]) * inv);
                        packed.w = pack2(__uint_as_float(r[d + 6]) * inv, __uint_as_float(r[d + 7]) * inv);
                        *reinterpret_cast<uint4*>(o + c + d) = packed;
                    }
                }
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

// The phase sums of the last launch's first blocks (a build with -DLLMB_TRACE): LLMB_TRACE_BLOCKS rows of
// LLMB_TRACE_SLOTS values: SM clock cycles of a softmax thread in slots 0-5 (waiting for S, reading it
// and its maximum, unused, waiting for O and rescaling, exponentials and P, releasing P), of the product
// thread in slots 6-10 (waiting for P, for V, issuing P V, waiting for K and issuing Q K^T, the first two
// Q K^T), and the block's number of key blocks in the last slot. Returns 1 in a build without.
LLMB_EXPORT int llmb_attention_prefill_tc_trace(unsigned long long* out, int clear) { return llmb_read_trace(out, clear); }

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
    LLMB_REQUIRE(head_dim == 64 || head_dim == 128, "attention_prefill_tc: head_dim %d (served: 64, 128)", head_dim);
    return LLMB_OK;
}

namespace {
template <int HD>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
           const int* block_table, int table_stride, int ring_pages, const int* cu_seqlens,
           const int* seq_lens, const int* seq_order, void* out, int out_stride, int n_seqs, int max_new, int n_heads,
           int n_kv_heads, float scale, cudaStream_t stream) {
    constexpr int Q_BYTES = (HD / 64) * Q_PIECE, KV_BYTES = (HD / 64) * KV_PIECE;
    // never less than 80 KB, so that no third block lands on an SM and waits for tensor memory
    size_t smem = 1024 + (size_t)Q_BYTES + 4 * KV_BYTES + 16 * 8 + 16;
    if (smem < 80 * 1024) smem = 80 * 1024;
    static bool configured = false;
    if (!configured) {
        LLMB_CUDA(cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    int* status = status_word();
    int* status_dev = nullptr;
    if (status) cudaHostGetDevicePointer((void**)&status_dev, status, 0);
    dim3 grid(n_heads, (max_new + BQ - 1) / BQ, n_seqs);
    llmb::launch(attention_prefill_tc_kernel<HD>, grid, THREADS, smem, stream, true,
                 map_q, map_k, map_v, block_table, table_stride, ring_pages, cu_seqlens, seq_lens, seq_order,
                 (__nv_bfloat16*)out, out_stride, n_heads, n_kv_heads, scale * 1.4426950408889634f, status_dev);
    return check_launch("attention_prefill_tc");
}
}  // namespace

// q: the fused projection of the new tokens [n_tokens, q_stride] (queries in its first columns);
// k_cache, v_cache: one layer of the paged cache [n_pages, n_kv_heads, 64, head_dim]; the rest as in
// llmb_attention_prefill. out must be 16-byte aligned with a row stride that is a multiple of 8.
LLMB_EXPORT int llmb_attention_prefill_tc(const void* q, int q_stride, int n_tokens, const void* k_cache,
                                          const void* v_cache, int n_pages, const int* block_table,
                                          int table_stride, int ring_pages, const int* cu_seqlens,
                                          const int* seq_lens, const int* seq_order, void* out, int out_stride, int n_seqs,
                                          int max_new, int n_heads, int n_kv_heads, int head_dim,
                                          float scale, int window, cudaStream_t stream) {
    if (n_seqs == 0 || max_new == 0) return LLMB_OK;
    int code = llmb_attention_prefill_tc_supports(n_heads, n_kv_heads, head_dim, window);
    if (code) return code;
    LLMB_REQUIRE(n_seqs <= 65535 && max_new / BQ < 65535 && ring_pages > 0 && n_pages > 0, "attention_prefill_tc: bad sizes");
    LLMB_REQUIRE(q_stride % 8 == 0 && out_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0,
                 "attention_prefill_tc: operands must be 16-byte aligned with row strides that are multiples of 8");
    CUtensorMap map_q, map_k, map_v;
    if ((code = make_map_2d(&map_q, q, n_tokens, (long long)n_heads * head_dim, q_stride, 64, BQ))) return code;
    long long cache_rows = (long long)n_pages * n_kv_heads * LLMB_PAGE;
    if ((code = make_map_2d(&map_k, k_cache, cache_rows, head_dim, head_dim, 64, LLMB_PAGE))) return code;
    if ((code = make_map_2d(&map_v, v_cache, cache_rows, head_dim, head_dim, 64, LLMB_PAGE))) return code;
    if (head_dim == 64)
        return launch<64>(map_q, map_k, map_v, block_table, table_stride, ring_pages, cu_seqlens, seq_lens, seq_order, out,
                          out_stride, n_seqs, max_new, n_heads, n_kv_heads, scale, stream);
    return launch<128>(map_q, map_k, map_v, block_table, table_stride, ring_pages, cu_seqlens, seq_lens, seq_order, out,
                       out_stride, n_seqs, max_new, n_heads, n_kv_heads, scale, stream);
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_attention_prefill_tc)
