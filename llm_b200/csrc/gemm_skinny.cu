// y[M, N] = x[M, K] . W[N, K]^T for a handful of rows (decode: M = live
// sequences <= 64), bfloat16 operands, 32-bit accumulation.
//
// The step is bound by reading W once from HBM, so the kernel is shaped around
// the stream of W (the role of q8_matmul_decode in MythEclipse/llm,
// apps/engine/kernels/gpu.cu:186-261: one warp per output row, 128-bit loads,
// residual in the epilogue), with the arithmetic on the tensor cores so that
// it stays hidden up to M = 64:
//
// * a warp owns 16 consecutive rows of W (one m16 tile of mma.sync.m16n8k16)
//   and a slice of K; the M tokens are the n dimension (padded to 8 * NT);
// * operands go from global memory straight into fragment registers with
//   128-bit loads. A lane with quad index t = lane % 4 loads 16 consecutive
//   elements of its row at k0 + 16 t; mma number j of the four that cover 64
//   k-values takes elements 4j..4j+3 of every lane. The x fragments are loaded
//   with the same rule, so both operands agree on which physical k a fragment
//   slot means and the dot product is only reordered;
// * K is split over `splits` warps per row tile so that even N = 4096 fills
//   148 SMs. Every warp writes its partial sums to scratch [splits, Mpad, N];
//   the warp that arrives last at the tile's counter adds the partials in
//   split order 0, 1, 2 ... (a fixed order, whichever warp is last) and
//   applies the epilogue: bias, then store as 32-bit or bfloat16 or add to the
//   32-bit residual. The counter is left at zero for the next call.
//
// Scratch (partials and counters) is passed in by the caller and may be shared
// by all calls on one stream; calls that overlap on the GPU must not share it.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_gemm_skinny)

constexpr int WARPS = 8;
constexpr int KSTEP = 64;           // k-values per fragment load
constexpr int UNROLL = 2;           // fragment loads in flight per row half

struct Frag {                       // 16 consecutive bf16 of one row: four mma k16 slices
    uint4 lo, hi;
};

__device__ __forceinline__ uint32_t frag_reg(const Frag& f, int i) {
    switch (i) {
        case 0: return f.lo.x; case 1: return f.lo.y; case 2: return f.lo.z; case 3: return f.lo.w;
        case 4: return f.hi.x; case 5: return f.hi.y; case 6: return f.hi.z; default: return f.hi.w;
    }
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                   const float* __restrict__ bias, void* __restrict__ out, int out_is_bf16,
                   float* __restrict__ residual, float* __restrict__ partials,
                   unsigned* __restrict__ counters, int M, int N, int K, int ldo, int splits,
                   int k_per_split, int n_tasks) {
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int task = blockIdx.x * WARPS + warp;
    if (task >= n_tasks) return;
    int row_tile = task / splits, split = task - row_tile * splits;
    int g = lane >> 2, t = lane & 3;
    int row_lo = row_tile * 16 + g, row_hi = row_lo + 8;
    int k_begin = split * k_per_split;
    int k_end = min(K, k_begin + k_per_split);
    const __nv_bfloat16* w_lo = w + (size_t)row_lo * K + t * 16;
    const __nv_bfloat16* w_hi = w + (size_t)row_hi * K + t * 16;
    bool lo_ok = row_lo < N, hi_ok = row_hi < N;

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

    // K is a multiple of 8 and every lane's 16 elements start at a multiple of 16,
    // so a lane's slice is whole, half (8 elements) or empty at the end of K.
    auto load_w = [&](const __nv_bfloat16* base, bool row_ok, int k) {
        Frag f;
        int at = k + t * 16;
        bool first = row_ok && at + 8 <= k_end, second = row_ok && at + 16 <= k_end;
        f.lo = first ? __ldg(reinterpret_cast<const uint4*>(base + k)) : make_uint4(0, 0, 0, 0);
        f.hi = second ? __ldg(reinterpret_cast<const uint4*>(base + k) + 1) : make_uint4(0, 0, 0, 0);
        return f;
    };

    Frag cur_lo[UNROLL], cur_hi[UNROLL], nxt_lo[UNROLL], nxt_hi[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        nxt_lo[u] = load_w(w_lo, lo_ok, k_begin + u * KSTEP);
        nxt_hi[u] = load_w(w_hi, hi_ok, k_begin + u * KSTEP);
    }
    for (int k0 = k_begin; k0 < k_end; k0 += KSTEP * UNROLL) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) { cur_lo[u] = nxt_lo[u]; cur_hi[u] = nxt_hi[u]; }
        int k_next = k0 + KSTEP * UNROLL;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            nxt_lo[u] = load_w(w_lo, lo_ok, k_next + u * KSTEP);
            nxt_hi[u] = load_w(w_hi, hi_ok, k_next + u * KSTEP);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            int k = k0 + u * KSTEP;
            int at = k + t * 16;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                int token = n * 8 + g;
                const __nv_bfloat16* xp = x + (size_t)token * ldx + at;
                Frag xf;
                bool tok_ok = token < M;
                xf.lo = (tok_ok && at + 8 <= k_end) ? __ldg(reinterpret_cast<const uint4*>(xp)) : make_uint4(0, 0, 0, 0);
                xf.hi = (tok_ok && at + 16 <= k_end) ? __ldg(reinterpret_cast<const uint4*>(xp) + 1) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    mma_bf16(acc[n], frag_reg(cur_lo[u], 2 * j), frag_reg(cur_hi[u], 2 * j),
                             frag_reg(cur_lo[u], 2 * j + 1), frag_reg(cur_hi[u], 2 * j + 1),
                             frag_reg(xf, 2 * j), frag_reg(xf, 2 * j + 1));
            }
        }
    }

    // element i of acc[n]: row (i < 2 ? row_lo : row_hi), token n * 8 + 2 t + (i & 1)
    if (splits > 1) {
        int m_pad = NT * 8;
        float* mine = partials + (size_t)split * m_pad * N;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int row = i < 2 ? row_lo : row_hi;
                int token = n * 8 + 2 * t + (i & 1);
                if (row < N) __stcg(mine + (size_t)token * N + row, acc[n][i]);
            }
        __threadfence();
        __syncwarp();
        unsigned arrived = 0;
        if (lane == 0) arrived = atomicAdd(&counters[row_tile], 1u);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        if (arrived != (unsigned)(splits - 1)) return;
        __threadfence();
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int row = i < 2 ? row_lo : row_hi;
                int token = n * 8 + 2 * t + (i & 1);
                float sum = 0.f;
                if (row < N)
                    for (int s = 0; s < splits; ++s)
                        sum += __ldcg(partials + ((size_t)s * m_pad + token) * N + row);
                acc[n][i] = sum;
            }
        if (lane == 0) counters[row_tile] = 0u;
    }
    if (residual) {
        // loads first, then stores: a load after a store would wait for it
        float old[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int row = i < 2 ? row_lo : row_hi;
                int token = n * 8 + 2 * t + (i & 1);
                old[n][i] = (row < N && token < M) ? residual[(size_t)token * ldo + row] : 0.f;
            }
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int row = i < 2 ? row_lo : row_hi;
                int token = n * 8 + 2 * t + (i & 1);
                if (row < N && token < M)
                    residual[(size_t)token * ldo + row] = old[n][i] + (acc[n][i] + (bias ? bias[row] : 0.f));
            }
        return;
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int row = i < 2 ? row_lo : row_hi;
            int token = n * 8 + 2 * t + (i & 1);
            if (row >= N || token >= M) continue;
            float v = acc[n][i] + (bias ? bias[row] : 0.f);
            size_t at = (size_t)token * ldo + row;
            if (out_is_bf16) reinterpret_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(out)[at] = v;
        }
}

// How many k-splits a call uses: enough warps to fill the GPU, each with at
// least two fragment loads of work.
LLMB_EXPORT int llmb_gemm_skinny_splits(int N, int K) {
    int row_tiles = (N + 15) / 16;
    int want = (148 * 20 + row_tiles - 1) / row_tiles;
    int most = (K + KSTEP * UNROLL - 1) / (KSTEP * UNROLL);
    if (want > most) want = most;
    if (want > 64) want = 64;
    if (want < 1) want = 1;
    int per = ((K + want - 1) / want + KSTEP * UNROLL - 1) / (KSTEP * UNROLL) * (KSTEP * UNROLL);
    return (K + per - 1) / per;
}

// Bytes of scratch a call needs: partials [splits, Mpad, N] floats, then one
// counter per row tile. The counters must be zero before the first call and are
// left at zero by every call.
LLMB_EXPORT long long llmb_gemm_skinny_scratch_bytes(int M, int N, int K) {
    int nt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
    int splits = llmb_gemm_skinny_splits(N, K);
    long long partial = splits > 1 ? (long long)splits * nt * 8 * N * 4 : 0;
    return partial;
}

LLMB_EXPORT int llmb_gemm_skinny(const void* x, int ldx, const void* w, const float* bias, void* out,
                                 int out_dtype, float* residual, float* partials,
                                 long long partial_bytes, unsigned* counters, int n_counters,
                                 int M, int N, int K, int ldo, cudaStream_t stream) {
    if (M == 0 || N == 0) return LLMB_OK;
    LLMB_REQUIRE(M > 0 && M <= 64, "gemm_skinny: %d rows (serves 1 to 64)", M);
    LLMB_REQUIRE(K > 0 && K % 8 == 0 && ldx % 8 == 0,
                 "gemm_skinny: K %d and the row stride %d must be multiples of 8 (16-byte loads)", K, ldx);
    LLMB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                 "gemm_skinny: operands must be 16-byte aligned");
    LLMB_REQUIRE((out != nullptr) != (residual != nullptr), "gemm_skinny: give out or residual");
    LLMB_REQUIRE(ldo >= N, "gemm_skinny: bad output stride");
    int splits = llmb_gemm_skinny_splits(N, K);
    int per = ((K + splits - 1) / splits + KSTEP * UNROLL - 1) / (KSTEP * UNROLL) * (KSTEP * UNROLL);
    int row_tiles = (N + 15) / 16;
    if (splits > 1) {
        LLMB_REQUIRE(partials != nullptr && counters != nullptr, "gemm_skinny: scratch is missing");
        LLMB_REQUIRE(partial_bytes >= llmb_gemm_skinny_scratch_bytes(M, N, K) && n_counters >= row_tiles,
                     "gemm_skinny: scratch too small (%lld bytes, %d counters)", partial_bytes, n_counters);
    }
    int n_tasks = row_tiles * splits;
    int blocks = (n_tasks + WARPS - 1) / WARPS;
    int is_bf16 = out_dtype == LLMB_DTYPE_BF16;
    LLMB_REQUIRE(residual || out_dtype == LLMB_DTYPE_BF16 || out_dtype == LLMB_DTYPE_F32,
                 "gemm_skinny: unknown output dtype %d", out_dtype);
#define LAUNCH(NT)                                                                               \
    gemm_skinny_kernel<NT><<<blocks, WARPS * 32, 0, stream>>>(                                   \
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, bias, out, is_bf16, residual,     \
        partials, counters, M, N, K, ldo, splits, per, n_tasks)
    if (M <= 8) LAUNCH(1);
    else if (M <= 16) LAUNCH(2);
    else if (M <= 32) LAUNCH(4);
    else LAUNCH(8);
#undef LAUNCH
    return check_launch("gemm_skinny");
}

// ------------------------------------------------------------------------- no allocation
// llmb_gemm_skinny_static (declared and described in gemm_skinny_static.h): the same
// product with its scratch in this library's own device memory instead of buffers
// the caller allocates.
#include "gemm_skinny_static.h"

static __device__ __align__(256) float static_partials[LLMB_GEMM_SKINNY_STATIC_FLOATS];
static __device__ __align__(256) unsigned static_counters[LLMB_GEMM_SKINNY_STATIC_COUNTERS];

namespace {
constexpr int MAX_DEVICES = 64;
float* static_partials_at[MAX_DEVICES] = {nullptr};      // device addresses, found once per device
unsigned* static_counters_at[MAX_DEVICES] = {nullptr};
}  // namespace

LLMB_EXPORT int llmb_gemm_skinny_static(const void* x, int ldx, const void* w, const float* bias,
                                        void* out, int out_dtype, float* residual, int M, int N,
                                        int K, int ldo, cudaStream_t stream) {
    if (M == 0 || N == 0) return LLMB_OK;
    LLMB_REQUIRE(M > 0 && M <= 64 && N > 0 && K > 0, "gemm_skinny_static: bad sizes");
    long long need = llmb_gemm_skinny_scratch_bytes(M, N, K);
    int row_tiles = (N + 15) / 16;
    LLMB_REQUIRE(need <= (long long)LLMB_GEMM_SKINNY_STATIC_FLOATS * 4,
                 "gemm_skinny_static: %d x %d x %d needs %lld bytes of partial sums, the built-in "
                 "scratch holds %lld; use llmb_gemm_skinny with scratch of your own",
                 M, N, K, need, (long long)LLMB_GEMM_SKINNY_STATIC_FLOATS * 4);
    LLMB_REQUIRE(row_tiles <= LLMB_GEMM_SKINNY_STATIC_COUNTERS,
                 "gemm_skinny_static: %d output rows need %d tile counters, the built-in scratch "
                 "holds %d", N, row_tiles, LLMB_GEMM_SKINNY_STATIC_COUNTERS);
    int device = 0;
    LLMB_CUDA(cudaGetDevice(&device));
    LLMB_REQUIRE(device >= 0 && device < MAX_DEVICES, "gemm_skinny_static: device %d", device);
    if (static_partials_at[device] == nullptr) {
        // Set-up, once per device, with that device current. In host code the names of the
        // arrays are host-side stand-ins, not device addresses: ask the runtime for the
        // addresses and hand those to the kernel.
        float* partials = nullptr;
        unsigned* counters = nullptr;
        LLMB_CUDA(cudaGetSymbolAddress((void**)&partials, static_partials));
        LLMB_CUDA(cudaGetSymbolAddress((void**)&counters, static_counters));
        // the counters must start at zero (every call leaves them at zero again)
        LLMB_CUDA(cudaMemsetAsync(counters, 0, sizeof(unsigned) * LLMB_GEMM_SKINNY_STATIC_COUNTERS, stream));
        static_counters_at[device] = counters;
        static_partials_at[device] = partials;
    }
    return llmb_gemm_skinny(x, ldx, w, bias, out, out_dtype, residual, static_partials_at[device],
                            (long long)LLMB_GEMM_SKINNY_STATIC_FLOATS * 4, static_counters_at[device],
                            LLMB_GEMM_SKINNY_STATIC_COUNTERS, M, N, K, ldo, stream);
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_gemm_skinny)
