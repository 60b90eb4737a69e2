// C[M, N] = A[M, K] . W[N, K]^T (+ bias[N]), stored or added to a 32-bit
// residual: the matrix product of every projection, on the CUDA cores.
//
// This is the kernel of the true 32-bit path (IEEE fused multiply-add, no
// reduced-precision matrix mode) and the fallback of the bfloat16 path for
// shapes the tensor-core kernels refuse (a row stride that is no multiple of 16
// bytes, for instance). Weights are row-major [out, in] as in MythEclipse/llm
// (apps/engine/src/tensor.rs:14,91: y[t,o] = sum_i x[t,i] W[o,i]); the residual
// is added in the epilogue as its matmul_add does (apps/engine/src/compute.rs:537-581).
//
// Every output element is summed over k = 0 .. K-1 in that order by one thread,
// whatever the tile shape, so a row's result does not depend on how many other
// rows the call has.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_gemm_simt)

// Loads rows [row0, row0 + ROWS) x columns [k0, k0 + BK) of a row-major matrix into `held`: every
// thread takes items of four consecutive k (one 16-byte load where `vector` holds: 32-bit elements,
// rows that start on 16-byte boundaries, K a multiple of 4); outside the matrix the value is 0.
template <typename TIn, int ROWS, int BK, int THREADS, int ITEMS>
__device__ __forceinline__ void fetch_tile(const TIn* __restrict__ base, int n_rows, int K, int ld, int row0, int k0,
                                           bool vector, float (&held)[ITEMS][4]) {
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        int item = threadIdx.x + it * THREADS;            // item = (row, group of four k)
        int r = item / (BK / 4), kk = (item % (BK / 4)) * 4;
        int row = row0 + r, k = k0 + kk;
        bool inside = item < ROWS * (BK / 4) && row < n_rows;
        if (inside && vector && k + 3 < K) {
            float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + (size_t)row * ld + k);
            held[it][0] = v.x; held[it][1] = v.y; held[it][2] = v.z; held[it][3] = v.w;
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                held[it][q] = (inside && k + q < K) ? to_float(base[(size_t)row * ld + k + q]) : 0.f;
        }
    }
}

template <int ROWS, int BK, int THREADS, int ITEMS, int LD>
__device__ __forceinline__ void park_tile(float (*tile)[LD], const float (&held)[ITEMS][4]) {
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        int item = threadIdx.x + it * THREADS;
        if (item >= ROWS * (BK / 4)) continue;
        int r = item / (BK / 4), kk = (item % (BK / 4)) * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) tile[kk + q][r] = held[it][q];
    }
}

// The next tiles are on their way from memory (into registers) while the current ones, in shared
// memory, are multiplied; the order of a thread's additions is k = 0, 1, 2, ... as before.
template <typename TIn, typename TOut, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const TIn* __restrict__ a, const TIn* __restrict__ w,
                 const float* __restrict__ bias, TOut* __restrict__ out,
                 float* __restrict__ residual, int M, int N, int K, int lda, int ldc, int vector) {
    constexpr int THREADS = (BM / TM) * (BN / TN);
    constexpr int A_ITEMS = (BM * BK / 4 + THREADS - 1) / THREADS, W_ITEMS = (BN * BK / 4 + THREADS - 1) / THREADS;
    __shared__ float a_tile[BK][BM + 4];
    __shared__ float w_tile[BK][BN + 4];
    int tid = threadIdx.x;
    int tx = tid % (BN / TN), ty = tid / (BN / TN);
    int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    float a_held[A_ITEMS][4], w_held[W_ITEMS][4];
    fetch_tile<TIn, BM, BK, THREADS, A_ITEMS>(a, M, K, lda, m0, 0, vector != 0, a_held);
    fetch_tile<TIn, BN, BK, THREADS, W_ITEMS>(w, N, K, K, n0, 0, vector != 0, w_held);
    for (int k0 = 0; k0 < K; k0 += BK) {
        park_tile<BM, BK, THREADS, A_ITEMS, BM + 4>(a_tile, a_held);
        park_tile<BN, BK, THREADS, W_ITEMS, BN + 4>(w_tile, w_held);
        __syncthreads();
        if (k0 + BK < K) {
            fetch_tile<TIn, BM, BK, THREADS, A_ITEMS>(a, M, K, lda, m0, k0 + BK, vector != 0, a_held);
            fetch_tile<TIn, BN, BK, THREADS, W_ITEMS>(w, N, K, K, n0, k0 + BK, vector != 0, w_held);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = a_tile[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = w_tile[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j] + (bias ? bias[n] : 0.f);
            size_t at = (size_t)m * ldc + n;
            if (residual) residual[at] += v;
            else out[at] = from_float<TOut>(v);
        }
    }
}

template <typename TIn, typename TOut>
static int launch(const void* a, const void* w, const float* bias, void* out, float* residual,
                  int M, int N, int K, int lda, int ldc, cudaStream_t stream) {
    // 16-byte loads: 32-bit elements, every row of both operands on a 16-byte boundary
    int vector = sizeof(TIn) == 4 && K % 4 == 0 && lda % 4 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    if (M > 64) {
        dim3 grid(ceil_div(N, 128), ceil_div(M, 128));
        gemm_simt_kernel<TIn, TOut, 128, 128, 8, 8, 8><<<grid, 256, 0, stream>>>(
            (const TIn*)a, (const TIn*)w, bias, (TOut*)out, residual, M, N, K, lda, ldc, vector);
    } else {
        dim3 grid(ceil_div(N, 64), ceil_div(M, 32));
        gemm_simt_kernel<TIn, TOut, 32, 64, 16, 2, 4><<<grid, 256, 0, stream>>>(
            (const TIn*)a, (const TIn*)w, bias, (TOut*)out, residual, M, N, K, lda, ldc, vector);
    }
    return check_launch("gemm_simt");
}

// in_dtype: element type of a and w. out_dtype: element type of `out` (ignored
// when `residual` is given: then the product is added to residual[M, N], 32-bit).
LLMB_EXPORT int llmb_gemm_simt(const void* a, const void* w, const float* bias, void* out,
                               float* residual, int in_dtype, int out_dtype, int M, int N, int K,
                               int lda, int ldc, cudaStream_t stream) {
    if (M == 0 || N == 0) return LLMB_OK;
    LLMB_REQUIRE(M > 0 && N > 0 && K > 0 && lda >= K && ldc >= N, "gemm_simt: bad sizes");
    LLMB_REQUIRE((out != nullptr) != (residual != nullptr), "gemm_simt: give out or residual");
    LLMB_REQUIRE(ceil_div(M, 32) <= 65535, "gemm_simt: too many rows");
    if (in_dtype == LLMB_DTYPE_F32) {
        if (residual || out_dtype == LLMB_DTYPE_F32)
            return launch<float, float>(a, w, bias, out, residual, M, N, K, lda, ldc, stream);
        return fail(LLMB_ERR_ARGUMENT, "gemm_simt: 32-bit inputs need a 32-bit output");
    }
    if (in_dtype == LLMB_DTYPE_BF16) {
        if (residual || out_dtype == LLMB_DTYPE_F32)
            return launch<__nv_bfloat16, float>(a, w, bias, out, residual, M, N, K, lda, ldc, stream);
        if (out_dtype == LLMB_DTYPE_BF16)
            return launch<__nv_bfloat16, __nv_bfloat16>(a, w, bias, out, residual, M, N, K, lda, ldc, stream);
    }
    return fail(LLMB_ERR_ARGUMENT, "gemm_simt: unknown dtypes %d -> %d", in_dtype, out_dtype);
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_gemm_simt)
