// C = A . B^T on the fifth-generation tensor cores: tcgen05.mma with the
// accumulator in tensor memory, operands staged in shared memory by TMA.
//
// A is [rows_a, K] and B is [rows_b, K], both bfloat16 with K contiguous (the
// row-major [out, in] weights of MythEclipse/llm, apps/engine/src/tensor.rs:14,91,
// and activations [tokens, K]). One block computes a 128 x BN tile of
// D[a_row, b_row] = sum_k A[a_row, k] B[b_row, k]. It replaces the mma.sync prompt
// kernel q8_matmul_mma (apps/engine/kernels/gpu.cu:907-1212): the tile loop,
// the token tile running fastest over the grid so that a weight tile is reused
// from L2 (gpu.cu:942-966) and the bias/residual epilogue (gpu.cu:1194-1209)
// are kept, the machinery is Blackwell's:
//
// * warp 0, one lane: TMA producer. Per k-block of 64 it waits for a free
//   stage, arms the stage's mbarrier with the byte count and issues two
//   cp.async.bulk.tensor.2d loads (128-byte swizzle), A rows and B rows.
// * warp 1: allocates BN columns of tensor memory; one lane issues four
//   tcgen05.mma (M 128, N BN, K 16) per k-block from shared-memory descriptors,
//   then tcgen05.commit frees the stage; a last commit signals the epilogue.
// * warps 2-5: epilogue. Each reads its 32 lanes of the accumulator with
//   tcgen05.ld, adds the bias, and stores bfloat16 or 32-bit, or adds into the
//   32-bit residual stream.
//
// Two orientations share the kernel. `swap == 0` (prefill): A = activations,
// B = weights, D[token, out] is stored row by row. `swap == 1` (decode, few
// tokens): A = weights, B = activations, so that the 128-row side of the
// instruction is filled by weight rows and the tokens are the narrow N side
// (16 to 64); D[out, token] is stored transposed. For decode the k-blocks are
// split over `splits` blocks per tile so that a product with few output tiles
// still fills 148 SMs: each block writes its partial tile to scratch, and the
// block that arrives last at the tile's counter adds the partials in split
// order and runs the epilogue (the counter returns to zero).
//
// The kernel is persistent: at most as many blocks as the GPU holds at once, each taking
// work units (an output tile and one slice of its k-blocks) round robin. The operand ring
// and two accumulator buffers in tensor memory carry on from unit to unit, so the loads and
// products of the next unit run under the epilogue of the last.
//
// Every wait on an mbarrier is bounded by a clock limit. A wait that runs out
// sets a status word that the host can read, raises the block's abort flag so
// that every role leaves its loop, and the block still frees its tensor memory.
#include <cuda.h>

#include "common.cuh"
#include "fusion.h"
#include "tc.cuh"

using namespace llmb;
using namespace llmb::tc;      // mbarrier, TMA and tcgen05 wrappers, descriptors, the tensor-map encoder

LLMB_DEFINE_LAST_ERROR(llmb_gemm_tc)

namespace {

constexpr int BM = 128;             // rows of A per tile = lanes of tensor memory
constexpr int BK = 64;              // k-values per stage: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;        // producer warp, mma warp, four epilogue warps

struct Epilogue {
    const float* bias;       // indexed by the output column n
    void* out;               // [tokens, ldo]
    float* residual;         // [tokens, ldo] 32-bit, added into
    int out_is_bf16;
    int ldo;
    int tokens, outs;        // valid tokens and output columns (rows of the weight matrix)
    int glu;                 // gated activation: the weight rows alternate 16 gate rows, 16 up rows;
                             // out is bfloat16 [tokens, ldo] with outs / 2 columns silu(gate) * up
    llmb_gemm_fusion f;      // what else the epilogue does (fusion.h); all zero: nothing
};

// 1 / sqrt(mean of squares + eps) of an input row from the partial sums its producer left. A whole warp
// computes it: lane i adds parts i and i + 32, then the lanes are summed as a butterfly, so every
// consumer of a row gets the same bits, and the loads of a row are in flight together.
__device__ __forceinline__ float warp_row_rstd(const llmb_gemm_fusion& f, int token) {
    int lane = threadIdx.x & 31;
    const float* p = f.norm_sumsq + (size_t)token * LLMB_SUMSQ_LD;
    float v = (lane < f.norm_parts ? __ldcg(p + lane) : 0.f) + (lane + 32 < f.norm_parts ? __ldcg(p + lane + 32) : 0.f);
    v = warp_sum(v);
    return 1.0f / sqrtf(v / f.norm_width + f.norm_eps);
}

// The same value, bit for bit, computed by ONE thread: v[i] = part i + part i + 32 as lane i has it, then
// the butterfly's levels as a tree (lane i's sum after the level of offset w is v[i] + v[i + w] for
// i < w; additions commute). A thread has all of its row's loads in flight at once, so the rows of a
// wide tile take one trip to L2 together instead of one trip each.
__device__ __forceinline__ float thread_row_rstd(const llmb_gemm_fusion& f, int token) {
    const float4* p = reinterpret_cast<const float4*>(f.norm_sumsq + (size_t)token * LLMB_SUMSQ_LD);
    int parts = f.norm_parts;
    float v[32];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        float4 lo = 4 * g < parts ? __ldcg(p + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 hi = 32 + 4 * g < parts ? __ldcg(p + 8 + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float l[4] = {lo.x, lo.y, lo.z, lo.w}, h[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int i = 4 * g + j;
            v[i] = (i < parts ? l[j] : 0.f) + (i + 32 < parts ? h[j] : 0.f);
        }
    }
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) {
#pragma unroll
        for (int i = 0; i < w; ++i) v[i] += v[i + w];
    }
    return 1.0f / sqrtf(v[0] / f.norm_width + f.norm_eps);
}
static_assert(LLMB_SUMSQ_LD == 64, "thread_row_rstd and warp_row_rstd read a row of 64 partial sums");

// The scales of a tile's token rows into shared memory, by the four epilogue warps, before the tile's
// accumulator is awaited: up to 16 rows a warp a row (quarter = 0..3 takes every fourth), more rows a
// thread a row. The caller synchronises the epilogue warps afterwards.
__device__ __forceinline__ void tile_rstd(const Epilogue& ep, float* rstd, int quarter, int first_token, int n_tile_tokens) {
    int lane = threadIdx.x & 31;
    if (n_tile_tokens > 16) {
        for (int i = quarter * 32 + lane; i < n_tile_tokens; i += 128) {
            int token = first_token + i;
            rstd[i] = token < ep.tokens ? thread_row_rstd(ep.f, token) : 1.f;
        }
        return;
    }
#pragma unroll 4
    for (int i = quarter; i < n_tile_tokens; i += 4) {
        int token = first_token + i;
        float r = token < ep.tokens ? warp_row_rstd(ep.f, token) : 1.f;
        if (lane == 0) rstd[i] = r;
    }
}

static_assert(LLMB_GLU_BLOCK == 16, "the gated epilogue reads 16 gate and 16 up columns of tensor memory per pair");

__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + expf(-gate)) * up; }

// One work unit: output tile (tile_a, tile_b) and one slice of its k-blocks.
struct Unit {
    int tile_a, tile_b, split;
};
__device__ __forceinline__ Unit unit_of(int u, int tiles_a, int splits) {
    Unit w;
    w.split = u % splits;
    int t = u / splits;
    w.tile_a = t % tiles_a;            // the A tile runs fastest: neighbours share a B tile in L2
    w.tile_b = t / tiles_a;
    return w;
}

// Stores 16 consecutive accumulator columns (c .. c+15) of this thread's row.
// `preloaded` (swapped products with a residual only): the residual's values at these 16 places,
// read by the caller earlier so that their latency ran under other loads.
// `rstd` (shared memory, or nullptr): the scales of the tile's token rows (a folded norm).
template <int BN>
__device__ __forceinline__ void store_columns(const Epilogue& ep, int swap, int a_row, int tile_b,
                                              int c, float (&v)[16], const float* preloaded = nullptr,
                                              const float* rstd = nullptr, int tile_row = 0) {
    if (rstd) {
        if (swap) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] *= rstd[c + j];
        } else {
            float r = rstd[tile_row];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] *= r;
        }
    }
    if (swap && ep.glu) {
        // lanes 0-15 of a warp hold 16 gate rows, lanes 16-31 the up rows of the same features
        int lane = threadIdx.x & 31;
        int feature = (a_row >> 5) * 16 + (a_row & 15);
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(ep.out);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float up = __shfl_xor_sync(0xffffffffu, v[j], 16);
            int token = tile_b * BN + c + j;
            if (lane < 16 && a_row < ep.outs && token < ep.tokens)
                o[(size_t)token * ep.ldo + feature] = __float2bfloat16_rn(silu_mul(v[j], up));
        }
        return;
    }
    if (swap) {
        // D[out column a_row, token]: one token at a time, lanes along the output row
        if (a_row >= ep.outs) return;
        float b = ep.bias ? ep.bias[a_row] : 0.f;
        int first_token = tile_b * BN + c;
        if (ep.residual) {
            // all loads first, then all stores: a load placed after a store would have to
            // wait for it (the compiler cannot know that the addresses differ)
            float old[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                if (preloaded) old[j] = preloaded[j];
                else old[j] = first_token + j < ep.tokens ? ep.residual[(size_t)(first_token + j) * ep.ldo + a_row] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (first_token + j < ep.tokens)
                    ep.residual[(size_t)(first_token + j) * ep.ldo + a_row] = old[j] + (v[j] + b);
            return;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            int token = first_token + j;
            if (token >= ep.tokens) break;
            size_t at = (size_t)token * ep.ldo + a_row;
            float value = v[j] + b;
            if (ep.out_is_bf16) reinterpret_cast<__nv_bfloat16*>(ep.out)[at] = __float2bfloat16_rn(value);
            else reinterpret_cast<float*>(ep.out)[at] = value;
        }
        return;
    }
    if (a_row >= ep.tokens) return;
    // D[token a_row, out column]: 16 consecutive columns of this thread's row
    int n0 = tile_b * BN + c;
    if (n0 >= ep.outs) return;
    size_t at = (size_t)a_row * ep.ldo + n0;
    bool whole = n0 + 16 <= ep.outs;
    if (ep.bias) {
#pragma unroll
        for (int j = 0; j < 16; ++j) if (n0 + j < ep.outs) v[j] += ep.bias[n0 + j];
    }
    if (ep.residual) {
        if (whole && (ep.ldo & 3) == 0) {
            float4* p = reinterpret_cast<float4*>(ep.residual + at);
            float4 old[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) old[j] = p[j];              // loads first, then stores
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                old[j].x += v[4 * j]; old[j].y += v[4 * j + 1]; old[j].z += v[4 * j + 2]; old[j].w += v[4 * j + 3];
                p[j] = old[j];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) if (n0 + j < ep.outs) ep.residual[at + j] += v[j];
        }
    } else if (ep.out_is_bf16) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(ep.out) + at;
        if (whole && (ep.ldo & 7) == 0) {
            uint4 packed[2];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            reinterpret_cast<uint4*>(o)[0] = packed[0];
            reinterpret_cast<uint4*>(o)[1] = packed[1];
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) if (n0 + j < ep.outs) o[j] = __float2bfloat16_rn(v[j]);
        }
    } else {
        float* o = reinterpret_cast<float*>(ep.out) + at;
        if (whole && (ep.ldo & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                reinterpret_cast<float4*>(o)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) if (n0 + j < ep.outs) o[j] = v[j];
        }
    }
}

// ---- the fused epilogues of a decode tile (weights on the 128-row side, tiles of 16 tokens), run by the
// four epilogue warps of the block that arrived last at the tile; v[j] is the summed (and scaled) product
// for output column a_row and token first_token + j, j < valid.

// Adds into the residual and also leaves what the next norm needs: the updated rows as bfloat16 and,
// per token, the sum of their squares over this tile's 128 columns as partial `tile_a` of the row.
// The sum runs over lanes, then over the four warps in a fixed order. exch: 64 floats.
__device__ __forceinline__ void finish_emit(const Epilogue& ep, int a_row, int tile_a, int first_token, int valid,
                                            float (&v)[16], const float (&old)[16], float* exch) {
    int lane = threadIdx.x & 31, quarter = (threadIdx.x >> 5) & 3;
    bool live = a_row < ep.outs;
    float b = (ep.bias && live) ? ep.bias[a_row] : 0.f;
    __nv_bfloat16* rows = reinterpret_cast<__nv_bfloat16*>(ep.f.emit_rows);
    float sq[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float updated = old[j] + (v[j] + b);
        bool here = live && j < valid;
        if (here) {
            size_t at = (size_t)(first_token + j) * ep.ldo + a_row;
            ep.residual[at] = updated;
            rows[at] = __float2bfloat16_rn(updated);
        }
        sq[j] = here ? updated * updated : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j)
        if (j < valid) sq[j] = warp_sum(sq[j]);          // (valid is the same for the whole block)
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) exch[quarter * 16 + j] = sq[j];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    int local = (int)threadIdx.x - 64;
    if (local < valid)
        ep.f.emit_sumsq[(size_t)(first_token + local) * LLMB_SUMSQ_LD + tile_a] =
            ((exch[local] + exch[16 + local]) + exch[32 + local]) + exch[48 + local];
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

// The q/k/v product's epilogue: bias, rotation of the query and key heads, queries to `out`, keys and
// values into the paged cache (what llmb_rope_cache_write does in a kernel of its own). A head's values
// lie in one tile (128 % head_dim == 0); pairs (p, p + head_dim/2) are exchanged through shared memory
// (exch: 16 x 128 floats), interleaved pairs (2p, 2p+1) between neighbouring lanes.
//
// What the epilogue needs from global memory besides the products is fetched before the products are
// awaited (stage_rope, by every block of the tile, since any may be the last): each token's position, the
// page of its position and its row of angles wait in shared memory. Read in the epilogue itself, these
// small loads miss the L2 (a layer's weights have passed through it since their last use) and two of
// them in a chain cost the last block of a tile three microseconds.
struct RopeStage {
    float angles[16][BM];          // [token of the tile][head_dim values: cosines, then sines]
    int pos[16];
    int page[16];
};

__device__ __forceinline__ void stage_rope(const Epilogue& ep, RopeStage* stage, int first_token) {
    const llmb_gemm_fusion& f = ep.f;
    int local = (int)threadIdx.x - 64;
    int valid = min(16, ep.tokens - first_token);
    if (local < 16) {
        int pos = 0, page = 0;
        if (local < valid) {
            pos = f.tok_pos[first_token + local];
            page = f.block_table[(size_t)f.tok_seq[first_token + local] * f.table_stride + ((pos / LLMB_PAGE) % f.ring_pages)];
        }
        stage->pos[local] = pos;
        stage->page[local] = page;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (f.rope_table) {
        int dim = f.head_dim;
        for (int i = local; i < valid * dim; i += 128) {
            int j = i / dim, e = i - j * dim;
            stage->angles[j][e] = f.rope_table[(size_t)stage->pos[j] * dim + e];
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

__device__ __forceinline__ void finish_rope(const Epilogue& ep, int a_row, int tile_row, int first_token, int valid,
                                            float (&v)[16], float* exch, const RopeStage* stage) {
    const llmb_gemm_fusion& f = ep.f;
    int dim = f.head_dim, half = dim >> 1;
    int head = a_row / dim, r = a_row - head * dim;
    bool live = a_row < ep.outs;
    float b = (ep.bias && live) ? ep.bias[a_row] : 0.f;
    float partner[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] += b;
    if (f.interleaved) {
#pragma unroll
        for (int j = 0; j < 16; ++j) partner[j] = __shfl_xor_sync(0xffffffffu, v[j], 1);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) exch[j * BM + tile_row] = v[j];
        asm volatile("bar.sync 1, 128;" ::: "memory");
        int other = r < half ? tile_row + half : tile_row - half;
#pragma unroll
        for (int j = 0; j < 16; ++j) partner[j] = exch[j * BM + other];
        asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    bool is_q = head < f.n_heads, is_k = !is_q && head < f.n_heads + f.n_kv_heads;
    bool rotates = f.rope_table != nullptr && (is_q || is_k);
    bool low = f.interleaved ? (r & 1) == 0 : r < half;
    int pair = f.interleaved ? r >> 1 : (r < half ? r : r - half);
    __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(ep.out);
    __nv_bfloat16* cache = reinterpret_cast<__nv_bfloat16*>(is_k ? f.k_cache : f.v_cache);
    int kv_head = is_k ? head - f.n_heads : head - f.n_heads - f.n_kv_heads;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        if (j >= valid || !live) break;
        float value = v[j];
        if (rotates) {
            float c = stage->angles[j][pair], s = stage->angles[j][half + pair];
            value = low ? v[j] * c - partner[j] * s : partner[j] * s + v[j] * c;
        }
        if (is_q) {
            q_out[(size_t)(first_token + j) * ep.ldo + a_row] = __float2bfloat16_rn(value);
        } else if (f.write_cache) {
            int pos = stage->pos[j];
            cache[(((size_t)stage->page[j] * f.n_kv_heads + kv_head) * LLMB_PAGE + (pos % LLMB_PAGE)) * dim + r] =
                __float2bfloat16_rn(value);
        }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");      // the staged values are free for the block's next unit
}

// Persistent: the grid has at most as many blocks as fit on the GPU at once, and block b
// takes the units b, b + gridDim.x, ... . The shared-memory ring and the two accumulator
// buffers in tensor memory run on across units, so the loads and products of the next unit
// overlap the epilogue of this one.
//
// Split K: every block leaves its partial tile in global memory. Either the block that arrives
// last at the tile's counter sums them in split order (one round of loads for up to 8 tokens), or,
// with sum_later (more than 16 tokens: the tile is wide and one block would sum for a long time),
// the blocks only write and splitk_sum_kernel, launched behind this kernel, sums with the whole
// GPU. The order of the sum is the same on both ways.
template <int BN>
__global__ void __launch_bounds__(THREADS, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               Epilogue ep, int swap, int n_kblocks, int kblocks_per_split, int splits, int tiles_a,
               int n_units, float* __restrict__ partials, unsigned* __restrict__ counters,
               int* status, int stages, int sum_later) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;       // two accumulator buffers
    // 1024-byte alignment of every tile is required by the 128-byte swizzle
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = base;
    unsigned char* b_tiles = base + (size_t)stages * A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_tiles + (size_t)stages * B_BYTES);
    uint64_t* full_bar = bars;                         // [stages] operands landed
    uint64_t* empty_bar = bars + stages;               // [stages] operands consumed
    uint64_t* acc_full_bar = bars + 2 * stages;        // [2] accumulator complete
    uint64_t* acc_empty_bar = bars + 2 * stages + 2;   // [2] accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * stages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
    float* exch = reinterpret_cast<float*>(tmem_slot + 4);      // the fused epilogues' exchange (sized by the host)
    RopeStage* rope_stage = reinterpret_cast<RopeStage*>(exch + 16 * BM);   // only with a fused rotation
    __shared__ float rstd_s[2][BM];                             // scales of a tile's token rows (a folded norm)

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    LLMB_STAMP(0, 0);                                           // the block has started
    griddep_launch();                                           // the next kernel of the stream may set itself up
    uint32_t early = 0;                                         // k-blocks whose weight tile is on its way

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full_bar[b]), 1);
            mbar_init(smem_u32(&acc_empty_bar[b]), 4);          // one arrival per epilogue warp
        }
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the barriers, as the copy engine sees them
        // Fetch this block's first weight tiles at once (no kernel writes weights): this thread made the
        // barriers and is the producer, so it need not wait for the block's set-up, and the kernel before
        // this one may still be running. The activations, the residual and the split-K scratch are
        // touched only after griddep_wait().
        if ((int)blockIdx.x < n_units) {
            Unit w = unit_of(blockIdx.x, tiles_a, splits);
            int kb_begin = w.split * kblocks_per_split;
            int kb_end = min(n_kblocks, kb_begin + kblocks_per_split);
            early = (uint32_t)min(stages, kb_end - kb_begin);
            for (uint32_t i = 0; i < early; ++i) {
                uint32_t bar = smem_u32(&full_bar[i]);
                mbar_expect_tx(bar, A_BYTES + B_BYTES);
                if (swap) tma_load_2d(smem_u32(a_tiles + (size_t)i * A_BYTES), &map_a, bar, (kb_begin + i) * BK, w.tile_a * BM);
                else tma_load_2d(smem_u32(b_tiles + (size_t)i * B_BYTES), &map_b, bar, (kb_begin + i) * BK, w.tile_b * BN);
            }
        }
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
    LLMB_STAMP(1, 0);                                           // barriers and tensor memory are set up
    griddep_wait();
    LLMB_STAMP(2, 0);                                           // the kernel before this one has completed

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;                                    // k-blocks issued so far, over all units
            int s = 0;                                          // the stage of k-block `it`, and how often
            uint32_t round = 0;                                 // the ring has been walked through (no division here)
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                Unit w = unit_of(u, tiles_a, splits);
                int kb_begin = w.split * kblocks_per_split;
                int kb_end = min(n_kblocks, kb_begin + kblocks_per_split);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it, s = (s + 1 == stages ? 0 : s + 1), round += (s == 0)) {
                    uint32_t bar = smem_u32(&full_bar[s]);
                    if (it < early) {                           // armed above, the weight tile is in flight
                        if (swap) tma_load_2d(smem_u32(b_tiles + (size_t)s * B_BYTES), &map_b, bar, kb * BK, w.tile_b * BN);
                        else tma_load_2d(smem_u32(a_tiles + (size_t)s * A_BYTES), &map_a, bar, kb * BK, w.tile_a * BM);
                        continue;
                    }
                    ok = mbar_wait(smem_u32(&empty_bar[s]), (round & 1) ^ 1, abort_flag, status, 1);
                    if (!ok) break;
                    mbar_expect_tx(bar, A_BYTES + B_BYTES);
                    tma_load_2d(smem_u32(a_tiles + (size_t)s * A_BYTES), &map_a, bar, kb * BK, w.tile_a * BM);
                    tma_load_2d(smem_u32(b_tiles + (size_t)s * B_BYTES), &map_b, bar, kb * BK, w.tile_b * BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D 32-bit, A and B bfloat16, both K-major, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // (this thread's instructions are the products' pace: the stage and its phase are counted, the
            // descriptors of stage 0 are made once, and the k-block that overwrites the accumulator is
            // peeled off: see gemm_tc_pair_kernel)
            uint32_t n_done = 0;
            int s = 0;
            uint32_t phase = 0;
            bool first = true;
            const uint64_t a_desc0 = smem_desc(smem_u32(a_tiles)), b_desc0 = smem_desc(smem_u32(b_tiles));
            const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++n_done) {
                Unit w = unit_of(u, tiles_a, splits);
                int kb_begin = w.split * kblocks_per_split;
                int kb_end = min(n_kblocks, kb_begin + kblocks_per_split);
                uint32_t buffer = n_done & 1, use = n_done >> 1;
                // the epilogue must have drained this buffer (its previous use)
                ok = mbar_wait(smem_u32(&acc_empty_bar[buffer]), (use & 1) ^ 1, abort_flag, status, 4);
                if (!ok) break;
                tcgen05_fence_after();
                uint32_t d_tmem = tmem_base + buffer * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = mbar_wait(full0 + 8 * s, phase, abort_flag, status, 2);
                    if (!ok) break;
                    if (first) { LLMB_STAMP(3, 32); first = false; }    // the first operand tiles have landed
                    tcgen05_fence_after();
                    uint64_t a_desc = a_desc0 + (uint64_t)(s * (A_BYTES >> 4));
                    uint64_t b_desc = b_desc0 + (uint64_t)(s * (B_BYTES >> 4));
                    // 16 k-values = 32 bytes further inside the swizzled row: +2 in 16-byte units
                    if (kb == kb_begin) {
                        tcgen05_mma(d_tmem, a_desc, b_desc, idesc, 0u);
#pragma unroll
                        for (int k = 1; k < BK / UMMA_K; ++k) tcgen05_mma(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, 1u);
                    } else {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) tcgen05_mma(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, 1u);
                    }
                    tcgen05_commit(empty0 + 8 * s);
                    if (++s == stages) { s = 0; phase ^= 1; }
                }
                if (ok) tcgen05_commit(smem_u32(&acc_full_bar[buffer]));
                LLMB_STAMP(4, 32);                              // the unit's last product is issued
            }
        }
    } else {
        int quarter = warp & 3;                          // the 32 lanes of tensor memory this warp may read
        int row = quarter * 32 + lane;                   // row of the tile = row of A
        uint32_t n_done = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++n_done) {
            Unit w = unit_of(u, tiles_a, splits);
            uint32_t buffer = n_done & 1, use = n_done >> 1;
            // a folded norm: the scales of this tile's token rows, computed while the products run
            // (two buffers in turn and one barrier a unit: a warp that runs ahead writes the other one)
            const float* rstd = nullptr;
            if (ep.f.norm_sumsq) {
                tile_rstd(ep, rstd_s[n_done & 1], quarter, swap ? w.tile_b * BN : w.tile_a * BM,
                          swap ? (BN < BM ? BN : BM) : BM);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                rstd = rstd_s[n_done & 1];
            }
            // a fused rotation: positions, pages and angles of the tile's tokens into shared memory
            // (read again only after this unit's epilogue, which ends with a barrier of these warps)
            if (BN == 16 && swap && splits > 1 && ep.f.rope) stage_rope(ep, rope_stage, w.tile_b * BN);
            ok = mbar_wait(smem_u32(&acc_full_bar[buffer]), use & 1, abort_flag, status, 3);
            if (!ok) break;
            tcgen05_fence_after();
            uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buffer * BN;
            int a_row = w.tile_a * BM + row;             // swap: output column; else: token
            size_t tile_id = (size_t)w.tile_b * tiles_a + w.tile_a;
            if (splits == 1 && ep.glu && !swap) {
                float r = rstd ? rstd[row] : 1.f;
                // columns alternate 16 gate, 16 up: this thread's row gets 16 activations per pair
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(ep.out);
#pragma unroll 1
                for (int c = 0; c + 32 <= BN; c += 32) {
                    uint32_t g[16], u[16];
                    tmem_ld16(taddr + c, g);
                    tmem_ld16(taddr + c + 16, u);
                    int n0 = w.tile_b * BN + c;                      // first weight row of the pair
                    if (a_row < ep.tokens && n0 + 32 <= ep.outs) {
                        uint4 packed[2];
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            h[j] = __floats2bfloat162_rn(
                                silu_mul(__uint_as_float(g[2 * j]) * r, __uint_as_float(u[2 * j]) * r),
                                silu_mul(__uint_as_float(g[2 * j + 1]) * r, __uint_as_float(u[2 * j + 1]) * r));
                        __nv_bfloat16* dst = o + (size_t)a_row * ep.ldo + n0 / 2;
                        if ((ep.ldo & 7) == 0) {
                            reinterpret_cast<uint4*>(dst)[0] = packed[0];
                            reinterpret_cast<uint4*>(dst)[1] = packed[1];
                        } else {
                            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(packed);
#pragma unroll
                            for (int j = 0; j < 16; ++j) dst[j] = e[j];
                        }
                    }
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[buffer]));
                continue;
            }
            if (splits == 1) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    uint32_t r[16];
                    float v[16];
                    tmem_ld16(taddr + c, r);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                    store_columns<BN>(ep, swap, a_row, w.tile_b, c, v, nullptr, rstd, row);
                }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[buffer]));
                continue;
            }
            // split K: park the partial tile [BN columns][128 rows], free the accumulator, and
            // let the block that arrives last add all partials in split order
            float* mine = partials + (tile_id * splits + w.split) * (size_t)(BN * BM);
            int cols = swap ? min(BN, ep.tokens - w.tile_b * BN) : BN;      // columns that hold tokens: the rest is padding that nobody reads
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c, r);
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (c + j < cols) __stcg(mine + (size_t)(c + j) * BM + row, __uint_as_float(r[j]));
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[buffer]));
            if (sum_later) {
                LLMB_STAMP(5, 64);
                continue;                                           // the kernel's end publishes the partials
            }
            __threadfence();
            LLMB_STAMP(5, 64);                                      // the partial tile is written and fenced
            asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps
            if (threadIdx.x == 64) {
                unsigned arrived = atomicAdd(&counters[tile_id], 1u);
                *last_flag = arrived == (unsigned)(splits - 1);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            bool last = *last_flag != 0;     // the flag is next written after the next unit's first barrier
            LLMB_STAMP(6, 64);                                      // the tile's counter has answered
            if (!last) continue;
            __threadfence();
            const float* first = partials + tile_id * splits * (size_t)(BN * BM) + row;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16], old[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.f;
                // columns that hold tokens (swapped products: the rest of the 16 is padding)
                int valid = swap ? min(16, ep.tokens - (w.tile_b * BN + c)) : 16;
                // the residual's values first: their latency runs under the partials' loads
                bool preload = swap && ep.residual && !ep.glu && a_row < ep.outs;
                if (preload) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        old[j] = j < valid ? ep.residual[(size_t)(w.tile_b * BN + c + j) * ep.ldo + a_row] : 0.f;
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) old[j] = 0.f;
                }
                // Partials are added in split order. With at most 8 valid columns, 8 splits' loads
                // are in flight at once (a decode step of up to 8 sequences sums 9 splits in two
                // rounds of loads instead of three over all 16 columns); else 4 splits of 16 columns.
                if (valid <= 8) {
                    for (int s0 = 0; s0 < splits; s0 += 8) {
                        float t[8][8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            bool live = s0 + i < splits;
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                t[i][j] = (live && j < valid) ? __ldcg(first + (size_t)(s0 + i) * (BN * BM) + (size_t)(c + j) * BM) : 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i)
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] += t[i][j];
                    }
                } else {
                    for (int s0 = 0; s0 < splits; s0 += 4) {
                        float t[4][16];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            bool live = s0 + i < splits;
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                t[i][j] = (live && j < valid) ? __ldcg(first + (size_t)(s0 + i) * (BN * BM) + (size_t)(c + j) * BM) : 0.f;
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i)
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] += t[i][j];
                    }
                }
                if (swap && (ep.f.rope || ep.f.emit_rows)) {
                    // the fused decode epilogues (tiles of 16 tokens: this loop runs once)
                    if (rstd) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] *= rstd[c + j];
                    }
                    if (ep.f.rope) finish_rope(ep, a_row, row, w.tile_b * BN + c, valid, v, exch, rope_stage);
                    else finish_emit(ep, a_row, w.tile_a, w.tile_b * BN + c, valid, v, old, exch);
                } else {
                    store_columns<BN>(ep, swap, a_row, w.tile_b, c, v, preload ? old : nullptr, rstd, row);
                }
            }
            if (threadIdx.x == 64) counters[tile_id] = 0u;
            LLMB_STAMP(7, 64);                                      // the last arriver has summed and stored
        }
    }

    // teardown: everyone meets, then the allocating warp frees the tensor memory
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // let copies that are still in flight land before shared memory is given up
        for (int i = 0; i < 100; ++i) __nanosleep(10000);
        __syncthreads();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Sums the partial tiles of a swapped split-K product: one thread per (token, output feature),
// the splits added in order, then scale / bias / residual / store as the product's epilogue would;
// with a residual it can also leave the next norm's input (bfloat16 rows and one partial sum of
// squares per block of 256 features).
// Partials: [tile_b][tile_a][split][BN columns = tokens][128 rows = features].
__device__ __forceinline__ float split_sum(const float* partials, int tiles_a, int splits, int bn, int token,
                                           int weight_row) {
    size_t tile_floats = (size_t)bn * BM;
    int tile_a = weight_row / BM, row = weight_row % BM, tile_b = token / bn, col = token % bn;
    const float* p = partials + ((size_t)tile_b * tiles_a + tile_a) * splits * tile_floats + (size_t)col * BM + row;
    float v = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = s0 + i < splits ? __ldcg(p + (size_t)(s0 + i) * tile_floats) : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) v += t[i];
    }
    return v;
}

__global__ void __launch_bounds__(256)
splitk_sum_kernel(const float* __restrict__ partials, Epilogue ep, int tiles_a, int splits, int bn) {
    griddep_launch();
    griddep_wait();
    __shared__ float scale_s;
    __shared__ float squares[8];
    int token = blockIdx.y;
    int feature = blockIdx.x * 256 + threadIdx.x;                  // with glu: the activated column
    int n_features = ep.glu ? ep.outs / 2 : ep.outs;
    if (ep.f.norm_sumsq) {
        if (threadIdx.x < 32) {
            float r = warp_row_rstd(ep.f, token);
            if (threadIdx.x == 0) scale_s = r;
        }
        __syncthreads();
    }
    float scale = ep.f.norm_sumsq ? scale_s : 1.f;
    float updated = 0.f;
    if (feature < n_features) {
        if (ep.glu) {
            // weight rows alternate 16 gate rows, 16 up rows
            int gate_row = (feature / LLMB_GLU_BLOCK) * 2 * LLMB_GLU_BLOCK + feature % LLMB_GLU_BLOCK;
            float gate = split_sum(partials, tiles_a, splits, bn, token, gate_row) * scale;
            float up = split_sum(partials, tiles_a, splits, bn, token, gate_row + LLMB_GLU_BLOCK) * scale;
            reinterpret_cast<__nv_bfloat16*>(ep.out)[(size_t)token * ep.ldo + feature] = __float2bfloat16_rn(silu_mul(gate, up));
        } else {
            float v = split_sum(partials, tiles_a, splits, bn, token, feature) * scale + (ep.bias ? ep.bias[feature] : 0.f);
            size_t at = (size_t)token * ep.ldo + feature;
            if (ep.residual) {
                updated = ep.residual[at] + v;
                ep.residual[at] = updated;
                if (ep.f.emit_rows) reinterpret_cast<__nv_bfloat16*>(ep.f.emit_rows)[at] = __float2bfloat16_rn(updated);
            } else if (ep.out_is_bf16) {
                reinterpret_cast<__nv_bfloat16*>(ep.out)[at] = __float2bfloat16_rn(v);
            } else {
                reinterpret_cast<float*>(ep.out)[at] = v;
            }
        }
    }
    if (ep.f.emit_sumsq) {                                          // uniform over the block
        float sq = warp_sum(updated * updated);
        if ((threadIdx.x & 31) == 0) squares[threadIdx.x >> 5] = sq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float total = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) total += squares[i];
            ep.f.emit_sumsq[(size_t)token * LLMB_SUMSQ_LD + blockIdx.x] = total;
        }
    }
}

// The same sum, four neighbouring features a thread and four tokens a block (rows and strides that
// allow 16-byte accesses): every thread has its shares' loads and its residual in flight together, and a
// quarter of the blocks pass through the GPU. With one value a thread the sum of a 512 x 4,096 product
// took 27 us for 34 MB, each of its 8,192 small blocks a chain of three trips to memory.
__device__ __forceinline__ float4 split_sum4(const float* partials, int tiles_a, int splits, int bn, int token,
                                             int weight_row) {
    size_t tile_floats = (size_t)bn * BM;
    int tile_a = weight_row / BM, row = weight_row % BM, tile_b = token / bn, col = token % bn;
    const float4* p = reinterpret_cast<const float4*>(
        partials + ((size_t)tile_b * tiles_a + tile_a) * splits * tile_floats + (size_t)col * BM + row);
    size_t stride = tile_floats / 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 8) {
        float4 t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t[i] = s0 + i < splits ? __ldcg(p + (size_t)(s0 + i) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v.x += t[i].x;
            v.y += t[i].y;
            v.z += t[i].z;
            v.w += t[i].w;
        }
    }
    return v;
}

__device__ __forceinline__ uint2 pack4(float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 r;
    r.x = *reinterpret_cast<uint32_t*>(&lo);
    r.y = *reinterpret_cast<uint32_t*>(&hi);
    return r;
}

__global__ void __launch_bounds__(256)
splitk_sum4_kernel(const float* __restrict__ partials, Epilogue ep, int tiles_a, int splits, int bn) {
    griddep_launch();
    griddep_wait();
    __shared__ float scale_s[4];
    __shared__ float squares[4][2];
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int slot = threadIdx.x >> 6;                                   // which of the block's four tokens
    int token = blockIdx.y * 4 + slot;
    int feature = blockIdx.x * 256 + (threadIdx.x & 63) * 4;       // with glu: the activated column
    int n_features = ep.glu ? ep.outs / 2 : ep.outs;
    if (ep.f.norm_sumsq) {
        if (warp < 4) {
            int t = blockIdx.y * 4 + warp;
            float r = t < ep.tokens ? warp_row_rstd(ep.f, t) : 1.f;
            if (lane == 0) scale_s[warp] = r;
        }
        __syncthreads();
    }
    float scale = ep.f.norm_sumsq ? scale_s[slot] : 1.f;
    float sq = 0.f;
    if (token < ep.tokens && feature < n_features) {
        if (ep.glu) {
            // weight rows alternate 16 gate rows, 16 up rows; four neighbours stay inside a block of 16
            int gate_row = (feature / LLMB_GLU_BLOCK) * 2 * LLMB_GLU_BLOCK + feature % LLMB_GLU_BLOCK;
            float4 g = split_sum4(partials, tiles_a, splits, bn, token, gate_row);
            float4 u = split_sum4(partials, tiles_a, splits, bn, token, gate_row + LLMB_GLU_BLOCK);
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ep.out) + (size_t)token * ep.ldo + feature) =
                pack4(silu_mul(g.x * scale, u.x * scale), silu_mul(g.y * scale, u.y * scale),
                      silu_mul(g.z * scale, u.z * scale), silu_mul(g.w * scale, u.w * scale));
        } else {
            float4 v = split_sum4(partials, tiles_a, splits, bn, token, feature);
            float4 b = ep.bias ? *reinterpret_cast<const float4*>(ep.bias + feature) : make_float4(0.f, 0.f, 0.f, 0.f);
            v.x = v.x * scale + b.x;
            v.y = v.y * scale + b.y;
            v.z = v.z * scale + b.z;
            v.w = v.w * scale + b.w;
            size_t at = (size_t)token * ep.ldo + feature;
            if (ep.residual) {
                float4 r = *reinterpret_cast<const float4*>(ep.residual + at);
                r.x += v.x;
                r.y += v.y;
                r.z += v.z;
                r.w += v.w;
                *reinterpret_cast<float4*>(ep.residual + at) = r;
                if (ep.f.emit_rows)
                    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ep.f.emit_rows) + at) = pack4(r.x, r.y, r.z, r.w);
                sq = fmaf(r.w, r.w, fmaf(r.z, r.z, fmaf(r.y, r.y, r.x * r.x)));
            } else if (ep.out_is_bf16) {
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ep.out) + at) = pack4(v.x, v.y, v.z, v.w);
            } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(ep.out) + at) = v;
            }
        }
    }
    if (ep.f.emit_sumsq) {                                          // uniform over the block
        sq = warp_sum(sq);
        if (lane == 0) squares[slot][warp & 1] = sq;
        __syncthreads();
        if (threadIdx.x < 4 && blockIdx.y * 4 + threadIdx.x < ep.tokens)
            ep.f.emit_sumsq[(size_t)(blockIdx.y * 4 + threadIdx.x) * LLMB_SUMSQ_LD + blockIdx.x] =
                squares[threadIdx.x][0] + squares[threadIdx.x][1];
    }
}

// The same sum for the q/k/v product with the rotation and the cache write behind it (see finish_rope):
// one thread per (token, item); an item is a rotation pair of a query or key head, or one value of a v head.
__global__ void __launch_bounds__(256)
splitk_sum_rope_kernel(const float* __restrict__ partials, Epilogue ep, int tiles_a, int splits, int bn) {
    griddep_launch();
    griddep_wait();
    __shared__ float scale_s;
    const llmb_gemm_fusion& f = ep.f;
    int token = blockIdx.y;
    int dim = f.head_dim, half = dim >> 1;
    int n_pairs = (f.n_heads + f.n_kv_heads) * half;
    int n_items = n_pairs + f.n_kv_heads * dim;
    int item = blockIdx.x * 256 + threadIdx.x;
    if (f.norm_sumsq) {
        if (threadIdx.x < 32) {
            float r = warp_row_rstd(f, token);
            if (threadIdx.x == 0) scale_s = r;
        }
        __syncthreads();
    }
    float scale = f.norm_sumsq ? scale_s : 1.f;
    if (item >= n_items) return;
    int pos = f.tok_pos[token];
    size_t cache_row = 0;
    if (f.write_cache) {
        int page = f.block_table[(size_t)f.tok_seq[token] * f.table_stride + ((pos / LLMB_PAGE) % f.ring_pages)];
        cache_row = ((size_t)page * f.n_kv_heads) * LLMB_PAGE + (pos % LLMB_PAGE);      // + kv_head * 64, times dim
    }
    __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(ep.out) + (size_t)token * ep.ldo;
    if (item < n_pairs) {
        int head = item / half, pair = item - head * half;
        int e0 = f.interleaved ? 2 * pair : pair, e1 = f.interleaved ? 2 * pair + 1 : pair + half;
        int row0 = head * dim + e0, row1 = head * dim + e1;
        float lo = split_sum(partials, tiles_a, splits, bn, token, row0) * scale + (ep.bias ? ep.bias[row0] : 0.f);
        float hi = split_sum(partials, tiles_a, splits, bn, token, row1) * scale + (ep.bias ? ep.bias[row1] : 0.f);
        if (f.rope_table) {
            float c = f.rope_table[(size_t)pos * dim + pair], s = f.rope_table[(size_t)pos * dim + half + pair];
            float a = lo * c - hi * s, b = lo * s + hi * c;
            lo = a;
            hi = b;
        }
        if (head < f.n_heads) {
            q_out[row0] = __float2bfloat16_rn(lo);
            q_out[row1] = __float2bfloat16_rn(hi);
        } else if (f.write_cache) {
            __nv_bfloat16* k = reinterpret_cast<__nv_bfloat16*>(f.k_cache) +
                               (cache_row + (size_t)(head - f.n_heads) * LLMB_PAGE) * dim;
            k[e0] = __float2bfloat16_rn(lo);
            k[e1] = __float2bfloat16_rn(hi);
        }
    } else if (f.write_cache) {
        int rest = item - n_pairs;
        int kv_head = rest / dim, e = rest - kv_head * dim;
        int row = (f.n_heads + f.n_kv_heads + kv_head) * dim + e;
        float v = split_sum(partials, tiles_a, splits, bn, token, row) * scale + (ep.bias ? ep.bias[row] : 0.f);
        reinterpret_cast<__nv_bfloat16*>(f.v_cache)[(cache_row + (size_t)kv_head * LLMB_PAGE) * dim + e] = __float2bfloat16_rn(v);
    }
}

// The same with four neighbouring rotation pairs (or four values of a v head) a thread and four tokens a
// block, as splitk_sum4_kernel (head sizes that are multiples of 8, rows that allow 8-byte stores).
__global__ void __launch_bounds__(256)
splitk_sum_rope4_kernel(const float* __restrict__ partials, Epilogue ep, int tiles_a, int splits, int bn) {
    griddep_launch();
    griddep_wait();
    __shared__ float scale_s[4];
    const llmb_gemm_fusion& f = ep.f;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int slot = threadIdx.x >> 6;
    int token = blockIdx.y * 4 + slot;
    int dim = f.head_dim, half = dim >> 1;
    int n_pair_quads = (f.n_heads + f.n_kv_heads) * half / 4;
    int n_quads = n_pair_quads + f.n_kv_heads * dim / 4;
    int quad = blockIdx.x * 64 + (threadIdx.x & 63);
    if (f.norm_sumsq) {
        if (warp < 4) {
            int t = blockIdx.y * 4 + warp;
            float r = t < ep.tokens ? warp_row_rstd(f, t) : 1.f;
            if (lane == 0) scale_s[warp] = r;
        }
        __syncthreads();
    }
    float scale = f.norm_sumsq ? scale_s[slot] : 1.f;
    if (token >= ep.tokens || quad >= n_quads) return;
    int pos = f.tok_pos[token];
    size_t cache_row = 0;
    if (f.write_cache) {
        int page = f.block_table[(size_t)f.tok_seq[token] * f.table_stride + ((pos / LLMB_PAGE) % f.ring_pages)];
        cache_row = ((size_t)page * f.n_kv_heads) * LLMB_PAGE + (pos % LLMB_PAGE);      // + kv_head * 64, times dim
    }
    auto biased = [&](float4 v, int row) {
        float4 b = ep.bias ? *reinterpret_cast<const float4*>(ep.bias + row) : make_float4(0.f, 0.f, 0.f, 0.f);
        return make_float4(v.x * scale + b.x, v.y * scale + b.y, v.z * scale + b.z, v.w * scale + b.w);
    };
    __nv_bfloat16* q_out = reinterpret_cast<__nv_bfloat16*>(ep.out) + (size_t)token * ep.ldo;
    if (quad < n_pair_quads) {
        int item = quad * 4;                                         // the first of four pairs of one head
        int head = item / half, pair = item - head * half;
        // rows of the four pairs: (pair .. pair + 3) and the same half a head on, or 2 pair .. 2 pair + 7
        int row0 = head * dim + (f.interleaved ? 2 * pair : pair);
        int row1 = f.interleaved ? row0 + 4 : row0 + half;
        float4 a = biased(split_sum4(partials, tiles_a, splits, bn, token, row0), row0);
        float4 b = biased(split_sum4(partials, tiles_a, splits, bn, token, row1), row1);
        float lo[4], hi[4];
        if (f.interleaved) {
            lo[0] = a.x; hi[0] = a.y; lo[1] = a.z; hi[1] = a.w;
            lo[2] = b.x; hi[2] = b.y; lo[3] = b.z; hi[3] = b.w;
        } else {
            lo[0] = a.x; lo[1] = a.y; lo[2] = a.z; lo[3] = a.w;
            hi[0] = b.x; hi[1] = b.y; hi[2] = b.z; hi[3] = b.w;
        }
        if (f.rope_table) {
            float4 c4 = *reinterpret_cast<const float4*>(f.rope_table + (size_t)pos * dim + pair);
            float4 s4 = *reinterpret_cast<const float4*>(f.rope_table + (size_t)pos * dim + half + pair);
            const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float x = lo[i] * c[i] - hi[i] * sn[i], y = lo[i] * sn[i] + hi[i] * c[i];
                lo[i] = x;
                hi[i] = y;
            }
        }
        __nv_bfloat16* dst = nullptr;
        if (head < f.n_heads) dst = q_out + (size_t)head * dim;
        else if (f.write_cache)
            dst = reinterpret_cast<__nv_bfloat16*>(f.k_cache) + (cache_row + (size_t)(head - f.n_heads) * LLMB_PAGE) * dim;
        if (dst) {
            if (f.interleaved) {
                *reinterpret_cast<uint2*>(dst + 2 * pair) = pack4(lo[0], hi[0], lo[1], hi[1]);
                *reinterpret_cast<uint2*>(dst + 2 * pair + 4) = pack4(lo[2], hi[2], lo[3], hi[3]);
            } else {
                *reinterpret_cast<uint2*>(dst + pair) = pack4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint2*>(dst + half + pair) = pack4(hi[0], hi[1], hi[2], hi[3]);
            }
        }
    } else if (f.write_cache) {
        int rest = (quad - n_pair_quads) * 4;
        int kv_head = rest / dim, e = rest - kv_head * dim;
        int row = (f.n_heads + f.n_kv_heads + kv_head) * dim + e;
        float4 v = biased(split_sum4(partials, tiles_a, splits, bn, token, row), row);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(f.v_cache) + (cache_row + (size_t)kv_head * LLMB_PAGE) * dim + e) =
            pack4(v.x, v.y, v.z, v.w);
    }
}

// ------------------------------------------------------------------------- two SMs on one tile
// For large token counts the 128 x 256 tile above is held back by shared-memory fill: per
// k-block it loads 48 KB for 524 tensor-core cycles. Two blocks of a cluster (a CTA pair on
// neighbouring SMs) computing one 256 x 256 tile with tcgen05.mma.cta_group::2 halve the
// weight traffic per SM: each block loads its own 128 token rows and only half (128 rows) of
// the weight tile, and the instruction reads both halves. Block 0 of the pair issues the
// instructions for both; each block keeps its 128 x 256 half of the accumulator in its own
// tensor memory and runs its own epilogue.
//
// Barriers: both producers' TMA loads report their bytes to block 0's `full` barrier (the
// .cta_group::2 form of the load allows a barrier in the partner block); tcgen05.commit with
// a multicast mask frees the stage in both blocks and announces the accumulator to both
// epilogues; all eight epilogue warps of the pair arrive on block 0's `acc_empty`.

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate),
          "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}

constexpr int PAIR_BN = 256;        // columns of the pair's tile; each block loads half of them

// The order in which the pairs take the tiles. The 74 tiles that run at the same time read their
// operands' k-blocks at about the same time, so an operand tile that several of them share comes from
// HBM once. With the token tile running fastest over all tiles (unit_of) a long prompt's 74 tiles
// share ONE weight tile and read 74 different token tiles: at 65,536 tokens and K = 2,048 that is
// 74 MB per 10 us, more than HBM delivers (products of a 263,000-token prefill ran at half their
// rate). So the token tiles are taken in panels of 8: inside a panel the token tile runs fastest,
// then the weight tile, then the next panel. A round of 74 tiles then reads 8 token tiles and about 9
// weight tiles.
constexpr int PANEL = 8;
__device__ __forceinline__ Unit pair_unit_of(int u, int tiles_a, int tiles_b) {
    Unit w;
    w.split = 0;
    int per_panel = PANEL * tiles_b;
    int panel = u / per_panel;
    int first = panel * PANEL;
    int width = min(PANEL, tiles_a - first);          // the last panel may be narrower
    int r = u - panel * per_panel;
    w.tile_b = r / width;
    w.tile_a = first + (r - w.tile_b * width);
    return w;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_residual, Epilogue ep, int n_kblocks, int tiles_a,
                    int n_units, int* status, int stages, int residual_by_tma) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = (PAIR_BN / 2) * BK * 2;
    constexpr int TMEM_COLS = 2 * PAIR_BN;
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = base;
    unsigned char* b_tiles = base + (size_t)stages * A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_tiles + (size_t)stages * B_BYTES);
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + stages;
    uint64_t* acc_full_bar = bars + 2 * stages;
    uint64_t* acc_empty_bar = bars + 2 * stages + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * stages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    __shared__ float rstd_s[2][BM];                   // scales of this block's 128 token rows (a folded norm)
    // Adding into the residual: accumulator pieces of 128 rows x 32 columns leave through two 16 KB
    // staging buffers behind the ring, and the copy engine adds them into the 32-bit matrix
    // (cp.reduce.async.bulk.tensor). Reading the old values into registers, 64 bytes a lane and one
    // chunk after the other, cost the last tile of every block some 16 us of load latency.
    float* staging = reinterpret_cast<float*>(base + (size_t)stages * (A_BYTES + B_BYTES) + 1024);

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank = cluster_rank();
    int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full_bar[b]), 1);
            mbar_init(smem_u32(&acc_empty_bar[b]), 8);          // four epilogue warps in each block
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();                                   // the partner's barriers exist from here on
    tcgen05_fence_after();
    uint32_t tmem_base = *tmem_slot;

    // As in gemm_tc_kernel: the first weight tiles (operand B here) are fetched while the kernel
    // before this one may still be running; the tokens only after griddep_wait().
    griddep_launch();
    uint32_t early = 0;
    if (warp == 0 && lane == 0 && pair < n_units) {
        Unit w = pair_unit_of(pair, tiles_a, n_units / tiles_a);
        early = (uint32_t)min(stages, n_kblocks);
        for (uint32_t i = 0; i < early; ++i) {
            if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[i]), 2 * (A_BYTES + B_BYTES));
            uint32_t bar = map_to_rank(smem_u32(&full_bar[i]), 0);
            tma_load_2d_pair(smem_u32(b_tiles + (size_t)i * B_BYTES), &map_b, bar, (int)i * BK,
                             w.tile_b * PAIR_BN + (int)rank * (PAIR_BN / 2));
        }
    }
    griddep_wait();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            int s = 0;
            uint32_t round = 0;                                 // how often the ring has been walked through
            bool ok = true;
            for (int u = pair; u < n_units && ok; u += n_pairs) {
                Unit w = pair_unit_of(u, tiles_a, n_units / tiles_a);
                for (int kb = 0; kb < n_kblocks; ++kb, ++it, s = (s + 1 == stages ? 0 : s + 1), round += (s == 0)) {
                    if (it < early) {                           // armed above, the weight tile is in flight
                        tma_load_2d_pair(smem_u32(a_tiles + (size_t)s * A_BYTES), &map_a,
                                         map_to_rank(smem_u32(&full_bar[s]), 0), kb * BK,
                                         w.tile_a * 2 * BM + (int)rank * BM);
                        continue;
                    }
                    ok = mbar_wait(smem_u32(&empty_bar[s]), (round & 1) ^ 1, abort_flag, status, 1);
                    if (!ok) break;
                    // both blocks' bytes are counted on block 0's barrier
                    if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * (A_BYTES + B_BYTES));
                    uint32_t bar = map_to_rank(smem_u32(&full_bar[s]), 0);
                    tma_load_2d_pair(smem_u32(a_tiles + (size_t)s * A_BYTES), &map_a, bar, kb * BK,
                                     w.tile_a * 2 * BM + (int)rank * BM);
                    tma_load_2d_pair(smem_u32(b_tiles + (size_t)s * B_BYTES), &map_b, bar, kb * BK,
                                     w.tile_b * PAIR_BN + (int)rank * (PAIR_BN / 2));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // D 32-bit, A and B bfloat16, both K-major, N = 256, M = 256 over the pair
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                       ((uint32_t)(PAIR_BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            // This one thread's instructions are the products' pace: per k-block it waits for a barrier and
            // issues four instructions and a commit. Nothing in the loop divides, reads a clock or builds a
            // descriptor from scratch: the stage and its phase are counted, the descriptors of stage 0
            // are made once and a stage adds a constant, and the first k-block (which overwrites the
            // accumulator) is peeled off so that the others accumulate unconditionally.
            uint32_t n_done = 0;
            int s = 0;
            uint32_t phase = 0;
            const uint64_t a_desc0 = smem_desc(smem_u32(a_tiles)), b_desc0 = smem_desc(smem_u32(b_tiles));
            const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
            bool ok = true;
            for (int u = pair; u < n_units && ok; u += n_pairs, ++n_done) {
                uint32_t buffer = n_done & 1, use = n_done >> 1;
                ok = mbar_wait(smem_u32(&acc_empty_bar[buffer]), (use & 1) ^ 1, abort_flag, status, 4);
                if (!ok) break;
                tcgen05_fence_after();
                uint32_t d_tmem = tmem_base + buffer * PAIR_BN;
                for (int kb = 0; kb < n_kblocks; ++kb) {
                    ok = mbar_wait(full0 + 8 * s, phase, abort_flag, status, 2);
                    if (!ok) break;
                    tcgen05_fence_after();
                    uint64_t a_desc = a_desc0 + (uint64_t)(s * (A_BYTES >> 4));
                    uint64_t b_desc = b_desc0 + (uint64_t)(s * (B_BYTES >> 4));
                    if (kb == 0) {
                        tcgen05_mma_pair(d_tmem, a_desc, b_desc, idesc, 0u);
#pragma unroll
                        for (int k = 1; k < BK / UMMA_K; ++k) tcgen05_mma_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, 1u);
                    } else {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) tcgen05_mma_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, 1u);
                    }
                    tcgen05_commit_pair(empty0 + 8 * s);               // frees the stage in both blocks
                    if (++s == stages) { s = 0; phase ^= 1; }
                }
                if (ok) tcgen05_commit_pair(smem_u32(&acc_full_bar[buffer]));
            }
        }
    } else {
        int quarter = warp & 3;
        int row = quarter * 32 + lane;
        uint32_t n_done = 0;
        bool ok = true;
        for (int u = pair; u < n_units && ok; u += n_pairs, ++n_done) {
            Unit w = pair_unit_of(u, tiles_a, n_units / tiles_a);
            uint32_t buffer = n_done & 1, use = n_done >> 1;
            const float* rstd = nullptr;
            if (ep.f.norm_sumsq) {                    // as in gemm_tc_kernel: while the products run
                tile_rstd(ep, rstd_s[n_done & 1], quarter, w.tile_a * 2 * BM + (int)rank * BM, BM);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                rstd = rstd_s[n_done & 1];
            }
            ok = mbar_wait(smem_u32(&acc_full_bar[buffer]), use & 1, abort_flag, status, 3);
            if (!ok) break;
            tcgen05_fence_after();
            uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buffer * PAIR_BN;
            int a_row = w.tile_a * 2 * BM + (int)rank * BM + row;
            if (ep.glu) {
                float r = rstd ? rstd[row] : 1.f;
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(ep.out);
#pragma unroll 1
                for (int c = 0; c < PAIR_BN; c += 32) {
                    uint32_t g[16], uu[16];
                    tmem_ld16(taddr + c, g);
                    tmem_ld16(taddr + c + 16, uu);
                    int n0 = w.tile_b * PAIR_BN + c;
                    if (a_row < ep.tokens && n0 + 32 <= ep.outs) {
                        uint4 packed[2];
                        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(packed);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            h[j] = __floats2bfloat162_rn(
                                silu_mul(__uint_as_float(g[2 * j]) * r, __uint_as_float(uu[2 * j]) * r),
                                silu_mul(__uint_as_float(g[2 * j + 1]) * r, __uint_as_float(uu[2 * j + 1]) * r));
                        __nv_bfloat16* dst = o + (size_t)a_row * ep.ldo + n0 / 2;
                        if ((ep.ldo & 7) == 0) {
                            reinterpret_cast<uint4*>(dst)[0] = packed[0];
                            reinterpret_cast<uint4*>(dst)[1] = packed[1];
                        } else {
                            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(packed);
#pragma unroll
                            for (int j = 0; j < 16; ++j) dst[j] = e[j];
                        }
                    }
                }
            } else if (residual_by_tma) {
                float scale = rstd ? rstd[row] : 1.f;
                int tile_row0 = w.tile_a * 2 * BM + (int)rank * BM;
#pragma unroll 1
                for (int c = 0; c < PAIR_BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    int n0 = w.tile_b * PAIR_BN + c;
                    float* buffer_s = staging + ((c >> 5) & 1) * (BM * 32);
                    // the copy that last read this buffer (two pieces ago) must be done with it
                    if (threadIdx.x == 64) bulk_wait_read<1>();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (n0 < ep.outs) {
                        // row `row` of the piece: eight 16-byte chunks, chunk q at place q ^ (row % 8)
                        // (the 128-byte swizzle of the tensor map; also spreads the lanes over the banks)
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            float4 piece;
                            piece.x = __uint_as_float(r[4 * q]) * scale;
                            piece.y = __uint_as_float(r[4 * q + 1]) * scale;
                            piece.z = __uint_as_float(r[4 * q + 2]) * scale;
                            piece.w = __uint_as_float(r[4 * q + 3]) * scale;
                            if (ep.bias) {
                                int n = n0 + 4 * q;
                                piece.x += n < ep.outs ? ep.bias[n] : 0.f;
                                piece.y += n + 1 < ep.outs ? ep.bias[n + 1] : 0.f;
                                piece.z += n + 2 < ep.outs ? ep.bias[n + 2] : 0.f;
                                piece.w += n + 3 < ep.outs ? ep.bias[n + 3] : 0.f;
                            }
                            *reinterpret_cast<float4*>(buffer_s + row * 32 + ((q ^ (row & 7)) << 2)) = piece;
                        }
                    }
                    fence_async_shared();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (threadIdx.x == 64) {
                        if (n0 < ep.outs && tile_row0 < ep.tokens)
                            tma_reduce_add_2d(&map_residual, smem_u32(buffer_s), n0, tile_row0);
                        bulk_commit();
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < PAIR_BN; c += 16) {
                    uint32_t r[16];
                    float v[16];
                    tmem_ld16(taddr + c, r);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
                    store_columns<PAIR_BN>(ep, 0, a_row, w.tile_b, c, v, nullptr, rstd, row);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_rank(smem_u32(&acc_empty_bar[buffer]), 0));
        }
    }

    if (threadIdx.x == 64) bulk_wait<0>();            // the copy engine is done with the staging buffers
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 100; ++i) __nanosleep(10000);
        __syncthreads();
    }
    cluster_sync();                                   // nobody leaves while the partner may still signal it
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------- host side

// rows x K bfloat16, K contiguous with `ld` elements between rows; box 64 x box_rows, 128-byte swizzle
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long k, long long ld, int box_rows) {
    return make_map_2d(map, ptr, rows, k, ld, BK, box_rows);
}

// Whether a swapped split-K product leaves the sum to splitk_sum_kernel: from 17 tokens. Up to 16
// tokens both ways measured the same on a decode step (4.87 ms at batch 8), at 64 tokens the
// kernel of its own is far ahead (O projection 21.8 -> 12.0 us).
inline int sums_later(int swap, int splits, int bn) { return (swap && splits > 1 && bn >= 32) ? 1 : 0; }

template <int BN>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const Epilogue& ep, int swap,
           int tiles_a, int tiles_b, int n_kblocks, int per_split, int splits, float* partials,
           unsigned* counters, cudaStream_t stream) {
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    int stages = (200 * 1024) / (A_BYTES + B_BYTES);
    if (stages > 8) stages = 8;
    int blocks_per_sm = 1;
    // the fused decode epilogues exchange values through shared memory behind the control words:
    // 64 floats for the sums of squares, 16 x 128 for rotation pairs that sit half a head apart
    size_t exchange = 256;
    if (swap && BN == 16 && splits > 1 && ep.f.rope) exchange = (size_t)16 * BM * 4 + sizeof(RopeStage);
    if (swap) {                                         // two blocks per SM for the decode stream
        stages = (int)((110 * 1024 - (exchange > 256 ? exchange : 0)) / (A_BYTES + B_BYTES));
        if (stages > 6) stages = 6;
        blocks_per_sm = 2;
    }
    size_t smem = 1024 + (size_t)stages * (A_BYTES + B_BYTES) + (2 * stages + 4) * 8 + 16 + exchange;
    static size_t configured = 0;
    if (smem > configured) {
        LLMB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    static int n_sms = 0;
    if (n_sms == 0) {
        int device = 0;
        LLMB_CUDA(cudaGetDevice(&device));
        LLMB_CUDA(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device));
    }
    int* status = status_word();
    int* status_dev = nullptr;
    if (status) cudaHostGetDevicePointer((void**)&status_dev, status, 0);
    int n_units = tiles_a * tiles_b * splits;
    int grid = n_units < n_sms * blocks_per_sm ? n_units : n_sms * blocks_per_sm;
    int sum_later = sums_later(swap, splits, BN);
    llmb::launch(gemm_tc_kernel<BN>, grid, THREADS, smem, stream, true, map_a, map_b, ep, swap, n_kblocks, per_split,
                 splits, tiles_a, n_units, partials, counters, status_dev, stages, sum_later);
    int code = check_launch("gemm_tc");
    if (code || !sum_later) return code;
    auto aligned = [](const void* p, uintptr_t to) { return (reinterpret_cast<uintptr_t>(p) & (to - 1)) == 0; };
    if (ep.f.rope) {
        int n_items = (ep.f.n_heads + ep.f.n_kv_heads) * (ep.f.head_dim / 2) + ep.f.n_kv_heads * ep.f.head_dim;
        if (ep.f.head_dim % 8 == 0 && ep.ldo % 4 == 0 && aligned(ep.out, 8) && aligned(ep.bias, 16) &&
            aligned(ep.f.k_cache, 8) && aligned(ep.f.v_cache, 8) && aligned(ep.f.rope_table, 16)) {
            llmb::launch(splitk_sum_rope4_kernel, dim3((n_items / 4 + 63) / 64, (ep.tokens + 3) / 4), 256, 0, stream, true,
                         (const float*)partials, ep, tiles_a, splits, BN);
            return check_launch("gemm_tc (split-K sum with rotation, four pairs a thread)");
        }
        llmb::launch(splitk_sum_rope_kernel, dim3((n_items + 255) / 256, ep.tokens), 256, 0, stream, true,
                     (const float*)partials, ep, tiles_a, splits, BN);
        return check_launch("gemm_tc (split-K sum with rotation)");
    }
    int n_features = ep.glu ? ep.outs / 2 : ep.outs;
    bool by_fours = n_features % 4 == 0 && ep.ldo % 4 == 0 && aligned(ep.out, ep.out_is_bf16 ? 8 : 16) &&
                    aligned(ep.residual, 16) && aligned(ep.bias, 16) && aligned(ep.f.emit_rows, 8);
    if (by_fours) {
        llmb::launch(splitk_sum4_kernel, dim3((n_features + 255) / 256, (ep.tokens + 3) / 4), 256, 0, stream, true,
                     (const float*)partials, ep, tiles_a, splits, BN);
        return check_launch("gemm_tc (split-K sum, four features a thread)");
    }
    llmb::launch(splitk_sum_kernel, dim3((n_features + 255) / 256, ep.tokens), 256, 0, stream, true,
                 (const float*)partials, ep, tiles_a, splits, BN);
    return check_launch("gemm_tc (split-K sum)");
}

int launch_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, const Epilogue& ep, int tiles_a,
                int tiles_b, int n_kblocks, cudaStream_t stream) {
    constexpr int STAGE_BYTES = BM * BK * 2 + (PAIR_BN / 2) * BK * 2;
    int stages = (192 * 1024) / STAGE_BYTES;
    if (stages > 8) stages = 8;
    // ring | 1 KB: barriers and control words | two staging buffers of 128 rows x 32 floats for the
    // residual epilogue (1024-byte aligned, as the swizzle wants)
    size_t smem = 1024 + (size_t)stages * STAGE_BYTES + 1024 + 2 * (size_t)BM * 32 * 4;
    static bool configured = false;
    if (!configured) {
        LLMB_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    // the residual through the copy engine where a tensor map can describe it
    CUtensorMap map_residual = map_a;
    int residual_by_tma = 0;
    if (ep.residual && !ep.glu && ep.ldo % 4 == 0 && (reinterpret_cast<uintptr_t>(ep.residual) & 15) == 0) {
        int code = make_map_2d_f32(&map_residual, ep.residual, ep.tokens, ep.outs, ep.ldo, BM);
        if (code) return code;
        residual_by_tma = 1;
    }
    static int n_sms = 0;
    if (n_sms == 0) {
        int device = 0;
        LLMB_CUDA(cudaGetDevice(&device));
        LLMB_CUDA(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device));
    }
    int* status = status_word();
    int* status_dev = nullptr;
    if (status) cudaHostGetDevicePointer((void**)&status_dev, status, 0);
    int n_units = tiles_a * tiles_b;
    int pairs = n_units < n_sms / 2 ? n_units : n_sms / 2;
    llmb::launch(gemm_tc_pair_kernel, 2 * pairs, THREADS, smem, stream, true, map_a, map_b, map_residual, ep,
                 n_kblocks, tiles_a, n_units, status_dev, stages, residual_by_tma);
    return check_launch("gemm_tc_pair");
}

struct Plan {
    int swap, bn, tiles_a, tiles_b, n_kblocks, per_split, splits;
};

// The weights take the 128-row side of the tiles (tokens in tiles of up to 128 on the other) and K
// is split whenever the 256 x 256 tiles of the pair kernel would fill less than 0.6 of the GPU's 74
// pairs of SMs: always up to 128 tokens, and up to 1,024 tokens for products with few output
// columns. (With the tokens on the 128-row side a 128 x 4096 x 4096 product has 16 tiles and took
// 38 us, a 256 x 4096 x 14336 product 103 us; this way they take 16 and 44 us. At 512 x 6144 x 4096
// the 48 pair tiles are faster again: 28 against 34 us.)
constexpr int SWAP_TOKENS = 128, SWAP_TOKENS_MOST = 1024, PAIRS = 74;

Plan make_plan(int M, int N, int K) {
    Plan p;
    p.n_kblocks = (K + BK - 1) / BK;
    long long pair_tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    // (a pair's tile of 64 k-blocks takes 26 us alone, whatever fills the other pairs: with a short K the
    // pairs win from 24 tiles on, 256 x 6144 x 4096 in 25.9 against 30.5 us, 512 x 4096 x 4096 in 26.1 against 38.3;
    // with a long K the split products stay ahead until the pairs are well filled)
    bool few_tiles = p.n_kblocks <= 64 ? pair_tiles < 24 : pair_tiles * 5 < PAIRS * 3;
    p.swap = M <= SWAP_TOKENS || (M <= SWAP_TOKENS_MOST && few_tiles);
    if (p.swap) {
        p.bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        p.tiles_a = (N + BM - 1) / BM;
        p.tiles_b = (M + p.bn - 1) / p.bn;
        // all blocks resident at once (two per SM): a second, partly filled wave would
        // double the time of a product this short
        int want = (2 * 148) / (p.tiles_a * p.tiles_b);
        int most = p.n_kblocks / 4 > 0 ? p.n_kblocks / 4 : 1; // at least four k-blocks a block
        if (want > most) want = most;
        if (want > 32) want = 32;
        if (want == 9 || want == 10) want = 8;      // the last block of a tile sums eight splits in one round of loads
        if (want < 1) want = 1;
        p.per_split = (p.n_kblocks + want - 1) / want;
        p.splits = (p.n_kblocks + p.per_split - 1) / p.per_split;
    } else {
        p.bn = N >= 256 ? 256 : N > 64 ? 128 : 64;
        p.tiles_a = (M + BM - 1) / BM;
        p.tiles_b = (N + p.bn - 1) / p.bn;
        p.per_split = p.n_kblocks;
        p.splits = 1;
    }
    return p;
}

}  // namespace

// 0 if nothing went wrong since the last call of this function; else the code of the
// wait that ran out (1 producer, 2 mma, 3 epilogue). Call after a synchronisation.
// The stamps of the last launches (a build with -DLLMB_TRACE): LLMB_TRACE_BLOCKS rows of
// LLMB_TRACE_SLOTS global-timer values, 0 where nothing was stamped. Returns 1 in a build without.
LLMB_EXPORT int llmb_gemm_tc_trace(unsigned long long* out, int clear) { return llmb_read_trace(out, clear); }

LLMB_EXPORT int llmb_gemm_tc_status() {
    int* s = status_word();
    if (!s) return -1;
    int v = *s;
    *s = 0;
    return v;
}

// Floats of partial-sum scratch and counters a call needs (0 when it does not split K).
LLMB_EXPORT long long llmb_gemm_tc_scratch_floats(int M, int N, int K) {
    Plan p = make_plan(M, N, K);
    return p.splits > 1 ? (long long)p.tiles_a * p.tiles_b * p.splits * p.bn * BM : 0;
}
LLMB_EXPORT int llmb_gemm_tc_counters(int M, int N, int K) {
    Plan p = make_plan(M, N, K);
    return p.tiles_a * p.tiles_b;
}

// Kernels a call launches (1, or 2 where the split-K sum is a kernel of its own).
LLMB_EXPORT int llmb_gemm_tc_kernels(int M, int N, int K) {
    Plan p = make_plan(M, N, K);
    return 1 + sums_later(p.swap, p.splits, p.bn);
}

// Partial sums of squares per row that a call with emit_rows / emit_sumsq writes inside its kernels
// (0: the shape's kernels do not, and the caller runs llmb_cast_sumsq behind the product).
LLMB_EXPORT int llmb_gemm_tc_emit_parts(int M, int N, int K) {
    Plan p = make_plan(M, N, K);
    if (!p.swap || p.splits <= 1) return 0;
    int parts = sums_later(p.swap, p.splits, p.bn) ? (N + 255) / 256 : p.tiles_a;
    return parts <= LLMB_SUMSQ_LD ? parts : 0;
}

// Whether a call with `rope` rotates and writes the cache inside its kernels.
LLMB_EXPORT int llmb_gemm_tc_fuses_rope(int M, int N, int K, int n_heads, int n_kv_heads, int head_dim) {
    Plan p = make_plan(M, N, K);
    return p.swap && p.splits > 1 && head_dim >= 2 && head_dim % 2 == 0 && BM % head_dim == 0 &&
           (long long)(n_heads + 2 * n_kv_heads) * head_dim == N;
}

// out[M, N] = x[M, K] . w[N, K]^T (+ bias[N]); or residual[M, N] += the same.
// allow_pair != 0: products with more than 128 rows run 256 x 256 tiles on pairs of SMs.
// glu != 0: w holds gate and up rows alternating in blocks of 16 (N = 2 F rows, N % 32 == 0) and
// out is bfloat16 [M, ldo] with F columns silu(gate) * up; no bias, no residual.
// fusion (optional): see fusion.h. *applied (optional) tells which parts ran inside the kernels:
// a folded norm always does; the rows and sums for the next norm and the rotation with the cache
// write only where the shape's kernels have them, else the caller runs them as kernels of their own.
LLMB_EXPORT int llmb_gemm_tc_ex(const void* x, int ldx, const void* w, const float* bias, void* out,
                                int out_dtype, float* residual, float* partials, long long partial_floats,
                                unsigned* counters, int n_counters, int M, int N, int K, int ldo, int glu,
                                int allow_pair, const llmb_gemm_fusion* fusion, int* applied,
                                cudaStream_t stream) {
    if (applied) *applied = 0;
    if (M == 0 || N == 0) return LLMB_OK;
    LLMB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes");
    LLMB_REQUIRE(K % 8 == 0 && ldx % 8 == 0,
                 "gemm_tc: K %d and the row stride %d must be multiples of 8 (TMA strides of 16 bytes)", K, ldx);
    LLMB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                 "gemm_tc: operands must be 16-byte aligned");
    LLMB_REQUIRE((out != nullptr) != (residual != nullptr), "gemm_tc: give out or residual");
    LLMB_REQUIRE(residual || out_dtype == LLMB_DTYPE_BF16 || out_dtype == LLMB_DTYPE_F32,
                 "gemm_tc: unknown output dtype %d", out_dtype);
    if (glu) {
        LLMB_REQUIRE(N % 32 == 0 && !bias && !residual && out_dtype == LLMB_DTYPE_BF16 && ldo >= N / 2,
                     "gemm_tc: the gated epilogue needs N %% 32 == 0, a bfloat16 output and no bias");
    } else {
        LLMB_REQUIRE(ldo >= N, "gemm_tc: bad output stride");
    }
    Plan p = make_plan(M, N, K);
    LLMB_REQUIRE((long long)p.tiles_a * p.tiles_b * p.splits < (1ll << 30), "gemm_tc: too many tiles");
    if (p.splits > 1) {
        LLMB_REQUIRE(partials && counters && partial_floats >= llmb_gemm_tc_scratch_floats(M, N, K) &&
                     n_counters >= p.tiles_a * p.tiles_b, "gemm_tc: scratch is missing or too small");
    }
    Epilogue ep{bias, out, residual, out_dtype == LLMB_DTYPE_BF16, ldo, M, N, glu != 0, {}};
    int did = 0;
    if (fusion) {
        llmb_gemm_fusion f = *fusion;
        if (f.norm_sumsq) {
            LLMB_REQUIRE(f.norm_parts >= 1 && f.norm_parts <= LLMB_SUMSQ_LD && f.norm_width > 0.f,
                         "gemm_tc: a folded norm needs 1 to %d partial sums a row", LLMB_SUMSQ_LD);
            did |= LLMB_FUSED_NORM;
        } else {
            f.norm_parts = 0;
        }
        if (f.emit_rows && f.emit_sumsq && residual && llmb_gemm_tc_emit_parts(M, N, K) > 0) {
            did |= LLMB_FUSED_EMIT;
        } else {
            f.emit_rows = nullptr;
            f.emit_sumsq = nullptr;
        }
        if (f.rope) {
            LLMB_REQUIRE(out && out_dtype == LLMB_DTYPE_BF16 && !glu && !residual && f.tok_pos && f.tok_seq &&
                         f.block_table && f.k_cache && f.v_cache && f.ring_pages > 0,
                         "gemm_tc: the rotation needs a bfloat16 output, positions, a page table and the cache");
            if (llmb_gemm_tc_fuses_rope(M, N, K, f.n_heads, f.n_kv_heads, f.head_dim)) did |= LLMB_FUSED_ROPE;
            else f.rope = 0;
        }
        ep.f = f;
    }
    if (applied) *applied = did;
    CUtensorMap map_a, map_b;
    int code;
    if (allow_pair && !p.swap && M > 128 && N >= 256) {
        // 256 x 256 tiles over pairs of SMs; each block's boxes are 128 rows
        if ((code = make_map(&map_a, x, M, K, ldx, BM))) return code;
        if ((code = make_map(&map_b, w, N, K, K, PAIR_BN / 2))) return code;
        return launch_pair(map_a, map_b, ep, (M + 2 * BM - 1) / (2 * BM), (N + PAIR_BN - 1) / PAIR_BN,
                           p.n_kblocks, stream);
    }
    if (p.swap) {
        if ((code = make_map(&map_a, w, N, K, K, BM))) return code;
        if ((code = make_map(&map_b, x, M, K, ldx, p.bn))) return code;
    } else {
        if ((code = make_map(&map_a, x, M, K, ldx, BM))) return code;
        if ((code = make_map(&map_b, w, N, K, K, p.bn))) return code;
    }
#define GO(BN) return launch<BN>(map_a, map_b, ep, p.swap, p.tiles_a, p.tiles_b, p.n_kblocks, \
                                 p.per_split, p.splits, partials, counters, stream)
    switch (p.bn) {
        case 16: GO(16);
        case 32: GO(32);
        case 64: GO(64);
        case 128: GO(128);
        default: GO(256);
    }
#undef GO
}

LLMB_EXPORT int llmb_gemm_tc(const void* x, int ldx, const void* w, const float* bias, void* out,
                             int out_dtype, float* residual, float* partials, long long partial_floats,
                             unsigned* counters, int n_counters, int M, int N, int K, int ldo, int glu,
                             int allow_pair, cudaStream_t stream) {
    return llmb_gemm_tc_ex(x, ldx, w, bias, out, out_dtype, residual, partials, partial_floats, counters,
                           n_counters, M, N, K, ldo, glu, allow_pair, nullptr, nullptr, stream);
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_gemm_tc_ex)
LLMB_PACKED(llmb_gemm_tc)
