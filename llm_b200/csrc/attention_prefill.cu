// Prefill attention: the new tokens of every sequence of a step attend, causally,
// to everything their sequence has in the paged cache (their own keys included),
// bfloat16, tiled so that nothing of the size of the context is ever stored.
//
// The scheme is the flash prefill of MythEclipse/llm (attention_prefill_mma,
// apps/engine/kernels/gpu.cu:1444-1655): query tiles against key tiles with
// mma.sync, a running (max, sum) per query row and the accumulator rescaled by
// exp(m_old - m_new) (gpu.cu:1560-1613), probabilities reused as the A operand of
// the second product (gpu.cu:1615-1631), and the heaviest query tile of a
// sequence launched first (gpu.cu:1457-1461). What is different: sequences of
// unequal length in one launch, keys and values read page by page from the slot
// cache through a block table, any group size (one head per block; the heads
// of a group find their shared pages in L2), head sizes 32 to 128.
//
// * grid (query tiles, heads, sequences); tile 0 of the grid is a sequence's last
//   64 queries. A block has four warps of 16 query rows each.
// * K and V of a page (64 keys) come through shared memory with cp.async, two
//   pages in flight; S = Q K^T and O += P V are mma.sync.m16n8k16 with fragments
//   from ldmatrix / ldmatrix.trans; softmax statistics are 32-bit, exponentials
//   base 2 with the scale folded in.
// * a key at position j is visible to the query at position p iff j <= p; only
//   the pages that cross a warp's diagonal are masked element by element, and
//   pages wholly above it are skipped by that warp.
//
// Refused (the generic kernel serves them): windows, 32-bit caches, head sizes
// other than 32, 64, 96, 128.
#include "common.cuh"
#include "mma.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_attention_prefill)

constexpr int WARPS = 4;
constexpr int BQ = WARPS * 16;               // queries per block
constexpr int STAGES = 2;
constexpr int PAD = 8;

// 2^x by the hardware approximation (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D>
__global__ void __launch_bounds__(WARPS * 32, 3)          // three blocks per SM: at most 170 registers
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride,
                         const __nv_bfloat16* __restrict__ k_cache,
                         const __nv_bfloat16* __restrict__ v_cache,
                         const int* __restrict__ block_table, int table_stride, int ring_pages,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_lens,
                         __nv_bfloat16* __restrict__ out, int out_stride, int n_heads,
                         int n_kv_heads, float scale_log2) {
    constexpr int LDS = D + PAD;
    constexpr int PAGE_ELEMS = LLMB_PAGE * LDS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [STAGES][2][64][LDS]

    int seq = blockIdx.z, head = blockIdx.x;
    int first_token = cu_seqlens[seq];
    int n_new = cu_seqlens[seq + 1] - first_token;
    int n_tiles = (n_new + BQ - 1) / BQ;
    if ((int)blockIdx.y >= n_tiles) return;
    int tile = n_tiles - 1 - blockIdx.y;                 // the heaviest tile of every head first (x runs fastest)
    int start = seq_lens[seq] - n_new;                   // position of the sequence's first new token
    int kv_head = head / (n_heads / n_kv_heads);
    int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int* pages = block_table + (size_t)seq * table_stride;

    int row0 = tile * BQ + warp * 16 + g, row1 = row0 + 8;      // index among the new tokens
    int pos0 = start + row0, pos1 = start + row1;               // positions (also of rows beyond n_new)
    int warp_last_pos = start + min(tile * BQ + warp * 16 + 15, n_new - 1);
    if (tile * BQ + warp * 16 >= n_new) warp_last_pos = -1;    // no query in this warp: skip every page
    int tile_last_pos = start + min(tile * BQ + BQ - 1, n_new - 1);
    int n_pages = tile_last_pos / LLMB_PAGE + 1;

    uint32_t qa[D / 16][4];
    {
        const __nv_bfloat16* q0 = q + (size_t)(first_token + row0) * q_stride + (size_t)head * D;
        const __nv_bfloat16* q1 = q + (size_t)(first_token + row1) * q_stride + (size_t)head * D;
        bool ok0 = row0 < n_new, ok1 = row1 < n_new;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qa[ks][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t) : 0u;
            qa[ks][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * t) : 0u;
            qa[ks][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * t) : 0u;
        }
    }

    auto load_page = [&](int logical_page, int stage) {
        int page = pages[logical_page % ring_pages];
        size_t base = ((size_t)page * n_kv_heads + kv_head) * LLMB_PAGE * D;
        __nv_bfloat16* ks = smem + (size_t)stage * 2 * PAGE_ELEMS;
        __nv_bfloat16* vs = ks + PAGE_ELEMS;
        constexpr int CHUNKS_PER_ROW = D / 8;
        for (int c = tid; c < LLMB_PAGE * CHUNKS_PER_ROW; c += WARPS * 32) {
            int row = c / CHUNKS_PER_ROW, col = (c % CHUNKS_PER_ROW) * 8;
            cp_async16(ks + row * LDS + col, k_cache + base + (size_t)row * D + col);
            cp_async16(vs + row * LDS + col, v_cache + base + (size_t)row * D + col);
        }
    };

    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
    float max0 = -INFINITY, max1 = -INFINITY, sum0 = 0.f, sum1 = 0.f;

    load_page(0, 0);
    cp_async_commit();
    for (int p = 0; p < n_pages; ++p) {
        cp_async_wait<0>();
        __syncthreads();                                // page p landed; everyone is done with page p - 1
        if (p + 1 < n_pages) load_page(p + 1, (p + 1) % STAGES);
        cp_async_commit();
        int key0 = p * LLMB_PAGE;
        if (key0 > warp_last_pos) continue;             // wholly above this warp's diagonal

        const __nv_bfloat16* ks = smem + (size_t)(p % STAGES) * 2 * PAGE_ELEMS;
        const __nv_bfloat16* vs = ks + PAGE_ELEMS;
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
#pragma unroll
        for (int kstep = 0; kstep < D / 16; ++kstep) {
#pragma unroll
            for (int nb = 0; nb < 8; nb += 2) {
                uint32_t b[4];
                int row = nb * 8 + (lane >> 4) * 8 + (lane & 7);
                int col = kstep * 16 + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(b, ks + row * LDS + col);
                mma_bf16(s[nb], qa[kstep][0], qa[kstep][1], qa[kstep][2], qa[kstep][3], b[0], b[1]);
                mma_bf16(s[nb + 1], qa[kstep][0], qa[kstep][1], qa[kstep][2], qa[kstep][3], b[2], b[3]);
            }
        }
        // s[nb][0..1]: row0, keys key0 + nb * 8 + 2t, +1; s[nb][2..3]: row1, the same keys.
        // Maxima are kept on the raw scores (the scale is positive); the scale and log2(e) are
        // applied inside the exponent with one fused multiply-add per score.
        bool diagonal = key0 + LLMB_PAGE - 1 > start + tile * BQ + warp * 16;   // some key may be hidden
        float local0 = -INFINITY, local1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (diagonal) {
                    int key = key0 + nb * 8 + 2 * t + i;
                    if (key > pos0) s[nb][i] = -INFINITY;
                    if (key > pos1) s[nb][2 + i] = -INFINITY;
                }
                local0 = fmaxf(local0, s[nb][i]);
                local1 = fmaxf(local1, s[nb][2 + i]);
            }
        }
        local0 = fmaxf(local0, __shfl_xor_sync(0xffffffffu, local0, 1));
        local0 = fmaxf(local0, __shfl_xor_sync(0xffffffffu, local0, 2));
        local1 = fmaxf(local1, __shfl_xor_sync(0xffffffffu, local1, 1));
        local1 = fmaxf(local1, __shfl_xor_sync(0xffffffffu, local1, 2));
        // key 0 is visible to every row, so after page 0 both maxima are finite
        float new0 = fmaxf(max0, local0), new1 = fmaxf(max1, local1);
        float rescale0 = fast_exp2((max0 - new0) * scale_log2), rescale1 = fast_exp2((max1 - new1) * scale_log2);
        max0 = new0;
        max1 = new1;
        float shift0 = new0 * scale_log2, shift1 = new1 * scale_log2;
        float add0 = 0.f, add1 = 0.f;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                s[nb][i] = fast_exp2(fmaf(s[nb][i], scale_log2, -shift0));
                s[nb][2 + i] = fast_exp2(fmaf(s[nb][2 + i], scale_log2, -shift1));
                add0 += s[nb][i];
                add1 += s[nb][2 + i];
            }
        }
        sum0 = sum0 * rescale0 + add0;
        sum1 = sum1 * rescale1 + add1;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            acc[n][0] *= rescale0; acc[n][1] *= rescale0;
            acc[n][2] *= rescale1; acc[n][3] *= rescale1;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            uint32_t pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            uint32_t pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            uint32_t pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int n = 0; n < D / 8; n += 2) {
                uint32_t b[4];
                int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                int col = (n + (lane >> 4)) * 8;
                ldmatrix_x4_trans(b, vs + row * LDS + col);
                mma_bf16(acc[n], pa0, pa1, pa2, pa3, b[0], b[1]);
                mma_bf16(acc[n + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();

    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    float inv0 = 1.0f / sum0, inv1 = 1.0f / sum1;
    __nv_bfloat16* o0 = out + (size_t)(first_token + row0) * out_stride + (size_t)head * D;
    __nv_bfloat16* o1 = out + (size_t)(first_token + row1) * out_stride + (size_t)head * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        if (row0 < n_new)
            *reinterpret_cast<__nv_bfloat162*>(o0 + n * 8 + 2 * t) = __floats2bfloat162_rn(acc[n][0] * inv0, acc[n][1] * inv0);
        if (row1 < n_new)
            *reinterpret_cast<__nv_bfloat162*>(o1 + n * 8 + 2 * t) = __floats2bfloat162_rn(acc[n][2] * inv1, acc[n][3] * inv1);
    }
}

template <int D>
static int launch(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                  const int* block_table, int table_stride, int ring_pages, const int* cu_seqlens,
                  const int* seq_lens, void* out, int out_stride, int n_seqs, int max_new, int n_heads,
                  int n_kv_heads, float scale, cudaStream_t stream) {
    constexpr int LDS = D + PAD;
    size_t smem = (size_t)STAGES * 2 * LLMB_PAGE * LDS * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        LLMB_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<D>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    dim3 grid(n_heads, (max_new + BQ - 1) / BQ, n_seqs);
    attention_prefill_kernel<D><<<grid, WARPS * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        block_table, table_stride, ring_pages, cu_seqlens, seq_lens, (__nv_bfloat16*)out, out_stride,
        n_heads, n_kv_heads, scale * 1.4426950408889634f);
    return check_launch("attention_prefill");
}

LLMB_EXPORT int llmb_attention_prefill_supports(int n_heads, int n_kv_heads, int head_dim, int window) {
    LLMB_REQUIRE(window == 0, "attention_prefill: a window of %d is not served", window);
    LLMB_REQUIRE(n_kv_heads > 0 && n_heads % n_kv_heads == 0,
                 "attention_prefill: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    LLMB_REQUIRE(head_dim == 32 || head_dim == 64 || head_dim == 96 || head_dim == 128,
                 "attention_prefill: head_dim %d (served: 32, 64, 96, 128)", head_dim);
    return LLMB_OK;
}

// q: the new tokens' queries, packed sequence after sequence [T, q_stride]; token i of sequence b
// is row cu_seqlens[b] + i and stands at position seq_lens[b] - n_new(b) + i, where seq_lens are
// the lengths after this step. max_new: the most new tokens any sequence brings.
LLMB_EXPORT int llmb_attention_prefill(const void* q, int q_stride, const void* k_cache,
                                       const void* v_cache, const int* block_table, int table_stride,
                                       int ring_pages, const int* cu_seqlens, const int* seq_lens,
                                       void* out, int out_stride, int n_seqs, int max_new,
                                       int n_heads, int n_kv_heads, int head_dim, float scale,
                                       int window, cudaStream_t stream) {
    if (n_seqs == 0 || max_new == 0) return LLMB_OK;
    int code = llmb_attention_prefill_supports(n_heads, n_kv_heads, head_dim, window);
    if (code) return code;
    LLMB_REQUIRE(n_seqs <= 65535 && max_new / BQ < 65535 && ring_pages > 0, "attention_prefill: bad sizes");
    LLMB_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 3) == 0,
                 "attention_prefill: q and out must be 4-byte aligned with even row strides");
#define ARGS q, q_stride, k_cache, v_cache, block_table, table_stride, ring_pages, cu_seqlens, seq_lens, \
             out, out_stride, n_seqs, max_new, n_heads, n_kv_heads, scale, stream
    switch (head_dim) {
        case 32: return launch<32>(ARGS);
        case 64: return launch<64>(ARGS);
        case 96: return launch<96>(ARGS);
        default: return launch<128>(ARGS);
    }
#undef ARGS
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_attention_prefill)
