// Row-wise kernels of the decoder: embedding gather, RMSNorm, rotary encoding
// fused with the write of keys and values into the paged cache, and the gated
// activation. Every kernel exists for 32-bit and for bfloat16 activations;
// sums, angles and the residual stream are 32-bit in both.
#include "common.cuh"
#include "fusion.h"
#include "random_normal.h"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_elementwise)

// ----------------------------------------------------------------------------- embedding
// x[t, :] = table[token[t], :], widened to 32-bit (the residual stream).
// Formula: apps/engine/kernels/gpu.cu:1752-1766 of MythEclipse/llm (one thread per
// (token, column)); here one block per token, columns strided over the threads.
// `scale` multiplies every value (1 for Llama; an architecture's embedding scale otherwise).
// With `rows` and `sumsq` the kernel also leaves the first norm's input: the row as bfloat16 and the
// sum of its squares (one partial sum, see fusion.h).
__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) total += scratch[i];               // the same order in every thread
    return total;
}

template <typename T>
__global__ void __launch_bounds__(256)
embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ x, int hidden,
             int vocab, int vector, float scale, __nv_bfloat16* __restrict__ rows, float* __restrict__ sumsq) {
    __shared__ float scratch[8];
    int t = blockIdx.x;
    int token = tokens[t];
    griddep_launch();
    if (token < 0 || token >= vocab) token = 0;   // host checks ids; device-sampled ids are in range
    const T* row = table + (size_t)token * hidden;
    float* out = x + (size_t)t * hidden;
    if (rows) {                                   // any width; the row is short enough to take element by element
        float sq = 0.f;
        for (int e = threadIdx.x; e < hidden; e += blockDim.x) {
            float v = to_float(row[e]) * scale;
            out[e] = v;
            rows[(size_t)t * hidden + e] = __float2bfloat16_rn(v);
            sq = fmaf(v, v, sq);
        }
        float total = block_sum_256(sq, scratch);
        if (threadIdx.x == 0) sumsq[(size_t)t * LLMB_SUMSQ_LD] = total;
        return;
    }
    if (vector) {
        // 16 bytes of the table per load (hidden is a multiple of 16 / sizeof(T), rows are aligned)
        constexpr int PER = 16 / sizeof(T);
        const uint4* src = reinterpret_cast<const uint4*>(row);
        for (int v = threadIdx.x; v < hidden / PER; v += blockDim.x) {
            uint4 raw = src[v];
            const T* e = reinterpret_cast<const T*>(&raw);
            float4* dst = reinterpret_cast<float4*>(out + (size_t)v * PER);
#pragma unroll
            for (int q = 0; q < PER / 4; ++q)
                dst[q] = make_float4(to_float(e[4 * q]) * scale, to_float(e[4 * q + 1]) * scale,
                                     to_float(e[4 * q + 2]) * scale, to_float(e[4 * q + 3]) * scale);
        }
        return;
    }
    for (int e = threadIdx.x; e < hidden; e += blockDim.x) out[e] = to_float(row[e]) * scale;
}

LLMB_EXPORT int llmb_embed(const int* tokens, const void* table, int table_dtype, float* x,
                           int n_tokens, int hidden, int vocab, float scale, void* rows, float* sumsq,
                           cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embed: bad sizes");
    LLMB_REQUIRE((rows != nullptr) == (sumsq != nullptr), "embed: give both the bfloat16 rows and the sums, or neither");
    int aligned = (reinterpret_cast<uintptr_t>(table) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (table_dtype == LLMB_DTYPE_F32)
        embed_kernel<float><<<n_tokens, 256, 0, stream>>>(tokens, (const float*)table, x, hidden, vocab,
                                                         aligned && hidden % 4 == 0, scale,
                                                         (__nv_bfloat16*)rows, sumsq);
    else if (table_dtype == LLMB_DTYPE_BF16)
        embed_kernel<__nv_bfloat16><<<n_tokens, 256, 0, stream>>>(tokens, (const __nv_bfloat16*)table, x, hidden,
                                                                 vocab, aligned && hidden % 8 == 0, scale,
                                                                 (__nv_bfloat16*)rows, sumsq);
    else
        return fail(LLMB_ERR_ARGUMENT, "embed: unknown dtype %d", table_dtype);
    return check_launch("embed");
}

// ----------------------------------------------------------------------------- RMSNorm
// out[r, :] = x[row(r), :] * (1 / sqrt(mean(x^2) + eps)) * gain, eps inside the root
// (apps/engine/src/ops.rs:4-12, apps/engine/kernels/gpu.cu:266-316). One block per
// row; the sum of squares is 32-bit and is reduced in a fixed order, so a row's
// result does not depend on the batch it is in. `rows` (optional) gathers rows.
// Four consecutive results in one store (the address is a multiple of the store's size).
__device__ __forceinline__ void store_quad(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store_quad(__nv_bfloat16* p, float a, float b, float c, float d) {
    uint2 packed;
    *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(a, b);
    *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = packed;
}

template <typename TOut, int PER_THREAD>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
               const int* __restrict__ rows, TOut* __restrict__ out, int hidden, float eps) {
    // PER_THREAD > 0: hidden is a multiple of 4 and at most 1024 * PER_THREAD; every thread
    // keeps its PER_THREAD float4 of the row in registers (all loads in flight at once).
    // PER_THREAD == 0: any width, the row is read twice.
    griddep_launch();
    griddep_wait();
    int r = blockIdx.x;
    int src = rows ? rows[r] : r;
    const float* in = x + (size_t)src * hidden;
    float sum = 0.f;
    float4 held[PER_THREAD > 0 ? PER_THREAD : 1];
    if (PER_THREAD > 0) {
        int quads = hidden >> 2;
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            int q = threadIdx.x + i * 256;
            held[i] = q < quads ? reinterpret_cast<const float4*>(in)[q] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // the same order of additions for every row: element order inside a thread
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            sum = fmaf(held[i].x, held[i].x, sum);
            sum = fmaf(held[i].y, held[i].y, sum);
            sum = fmaf(held[i].z, held[i].z, sum);
            sum = fmaf(held[i].w, held[i].w, sum);
        }
    } else {
        for (int e = threadIdx.x; e < hidden; e += blockDim.x) {
            float v = in[e];
            sum = fmaf(v, v, sum);
        }
    }
    __shared__ float partial[32];
    __shared__ float scale_shared;
    sum = warp_sum(sum);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) partial[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        int n_warps = blockDim.x >> 5;
        float v = lane < n_warps ? partial[lane] : 0.f;
        v = warp_sum(v);
        if (lane == 0) scale_shared = 1.0f / sqrtf(v / (float)hidden + eps);
    }
    __syncthreads();
    float scale = scale_shared;
    TOut* o = out + (size_t)r * hidden;
    if (PER_THREAD > 0) {
        int quads = hidden >> 2;
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            int q = threadIdx.x + i * 256;
            if (q >= quads) continue;
            float4 g = reinterpret_cast<const float4*>(gain)[q];
            float4 v = held[i];
            store_quad(o + 4 * q, v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        }
    } else {
        for (int e = threadIdx.x; e < hidden; e += blockDim.x)
            o[e] = from_float<TOut>(in[e] * scale * gain[e]);
    }
}

template <typename TOut>
static void launch_rmsnorm(const float* x, const float* gain, const int* rows, TOut* out, int n_rows,
                           int hidden, float eps, cudaStream_t stream) {
    bool vector = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(gain) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (vector && hidden <= 1024) llmb::launch(rmsnorm_kernel<TOut, 1>, n_rows, 256, 0, stream, true, x, gain, rows, out, hidden, eps);
    else if (vector && hidden <= 2048) llmb::launch(rmsnorm_kernel<TOut, 2>, n_rows, 256, 0, stream, true, x, gain, rows, out, hidden, eps);
    else if (vector && hidden <= 4096) llmb::launch(rmsnorm_kernel<TOut, 4>, n_rows, 256, 0, stream, true, x, gain, rows, out, hidden, eps);
    else if (vector && hidden <= 8192) llmb::launch(rmsnorm_kernel<TOut, 8>, n_rows, 256, 0, stream, true, x, gain, rows, out, hidden, eps);
    else llmb::launch(rmsnorm_kernel<TOut, 0>, n_rows, 256, 0, stream, true, x, gain, rows, out, hidden, eps);
}

LLMB_EXPORT int llmb_rmsnorm(const float* x, const float* gain, const int* rows, void* out,
                             int out_dtype, int n_rows, int hidden, float eps,
                             cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(n_rows > 0 && hidden > 0, "rmsnorm: bad sizes");
    if (out_dtype == LLMB_DTYPE_F32)
        launch_rmsnorm<float>(x, gain, rows, (float*)out, n_rows, hidden, eps, stream);
    else if (out_dtype == LLMB_DTYPE_BF16)
        launch_rmsnorm<__nv_bfloat16>(x, gain, rows, (__nv_bfloat16*)out, n_rows, hidden, eps, stream);
    else
        return fail(LLMB_ERR_ARGUMENT, "rmsnorm: unknown dtype %d", out_dtype);
    return check_launch("rmsnorm");
}

// ----------------------------------------------------------------------------- a norm's input without the norm
// rows[t, :] = bfloat16(x[t, :]) and sumsq[t, 0] = sum of x[t, :]^2: what a product with a folded norm reads
// (fusion.h) when no product's epilogue has left it. One block per row, the sum in a fixed order.
__global__ void __launch_bounds__(256)
cast_sumsq_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ rows, float* __restrict__ sumsq,
                  int hidden, int vector) {
    griddep_launch();
    griddep_wait();
    __shared__ float scratch[8];
    int t = blockIdx.x;
    const float* in = x + (size_t)t * hidden;
    __nv_bfloat16* out = rows + (size_t)t * hidden;
    float sq = 0.f;
    if (vector) {
        for (int q = threadIdx.x; q < hidden / 4; q += blockDim.x) {
            float4 v = reinterpret_cast<const float4*>(in)[q];
            sq = fmaf(v.x, v.x, sq);
            sq = fmaf(v.y, v.y, sq);
            sq = fmaf(v.z, v.z, sq);
            sq = fmaf(v.w, v.w, sq);
            store_quad(out + 4 * q, v.x, v.y, v.z, v.w);
        }
    } else {
        for (int e = threadIdx.x; e < hidden; e += blockDim.x) {
            float v = in[e];
            sq = fmaf(v, v, sq);
            out[e] = __float2bfloat16_rn(v);
        }
    }
    float total = block_sum_256(sq, scratch);
    if (threadIdx.x == 0) sumsq[(size_t)t * LLMB_SUMSQ_LD] = total;
}

LLMB_EXPORT int llmb_cast_sumsq(const float* x, void* rows, float* sumsq, int n_rows, int hidden,
                                cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(n_rows > 0 && hidden > 0, "cast_sumsq: bad sizes");
    int vector = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(rows) & 7) == 0;
    llmb::launch(cast_sumsq_kernel, n_rows, 256, 0, stream, true, x, (__nv_bfloat16*)rows, sumsq, hidden, vector);
    return check_launch("cast_sumsq");
}

// out[t, :] = out[t, :] * rstd(t) + bias: the folded norm's scale for a product whose kernel does not
// apply it itself (rstd from the partial sums of squares as in fusion.h).
template <typename T>
__global__ void scale_rows_kernel(T* __restrict__ out, int width, const float* __restrict__ sumsq, int parts,
                                  float eps, float norm_width, const float* __restrict__ bias) {
    __shared__ float scale_s;
    int t = blockIdx.x;
    if (threadIdx.x < 32) {
        // the order of the products' epilogues (warp_row_rstd in gemm_tc.cu): lane i takes parts i and
        // i + 32, then a butterfly over the lanes
        int lane = threadIdx.x;
        const float* p = sumsq + (size_t)t * LLMB_SUMSQ_LD;
        float v = (lane < parts ? p[lane] : 0.f) + (lane + 32 < parts ? p[lane + 32] : 0.f);
        v = warp_sum(v);
        if (lane == 0) scale_s = 1.0f / sqrtf(v / norm_width + eps);
    }
    __syncthreads();
    float scale = scale_s;
    for (int e = threadIdx.x; e < width; e += blockDim.x)
        out[(size_t)t * width + e] = from_float<T>(to_float(out[(size_t)t * width + e]) * scale + (bias ? bias[e] : 0.f));
}

LLMB_EXPORT int llmb_scale_rows(void* out, int dtype, int n_rows, int width, const float* sumsq, int parts,
                                float eps, float norm_width, const float* bias, cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(n_rows > 0 && width > 0 && parts >= 1 && parts <= LLMB_SUMSQ_LD, "scale_rows: bad sizes");
    if (dtype == LLMB_DTYPE_F32)
        scale_rows_kernel<float><<<n_rows, 256, 0, stream>>>((float*)out, width, sumsq, parts, eps, norm_width, bias);
    else if (dtype == LLMB_DTYPE_BF16)
        scale_rows_kernel<__nv_bfloat16><<<n_rows, 256, 0, stream>>>((__nv_bfloat16*)out, width, sumsq, parts, eps,
                                                                   norm_width, bias);
    else
        return fail(LLMB_ERR_ARGUMENT, "scale_rows: unknown dtype %d", dtype);
    return check_launch("scale_rows");
}

// ----------------------------------------------------------------------------- rotary + cache write
// One launch per layer: rotate the queries in place, rotate the keys and store
// them into the paged cache, copy the values into the cache (the job of
// rope_append, apps/engine/kernels/gpu.cu:525-581). Only the first n_rot
// elements of a head are rotated, the rest passes through (the rope dimension
// count that MythEclipse/llm reads beside the head size, apps/engine/src/model.rs:93-95).
// Angles come from a 32-bit table [max_positions, n_rot] (cos in the first half
// of a row, sin in the second) built once on the host; `interleaved` chooses the
// pairs (2p, 2p+1) of MythEclipse/llm (apps/engine/src/ops.rs:152-165), otherwise
// (p, p + n_rot/2). With table == nullptr nothing is rotated (a mixer without
// position encoding). A token's position and sequence come from device arrays;
// position p of sequence b lives in page block_table[b][(p / 64) % ring_pages],
// row p % 64.
template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const float* __restrict__ table,
                                  const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                  const int* __restrict__ block_table, int table_stride,
                                  int ring_pages, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  int n_heads, int n_kv_heads, int head_dim, int n_rot, int interleaved,
                                  int write_cache) {
    int t = blockIdx.x;
    int head = blockIdx.y;               // [0, Hq): q; [Hq, Hq+Hkv): k; then v
    int pos = tok_pos[t];
    int half = n_rot >> 1;
    size_t row_stride = (size_t)(n_heads + 2 * n_kv_heads) * head_dim;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * head_dim;
    bool is_q = head < n_heads;
    bool is_k = !is_q && head < n_heads + n_kv_heads;
    T* dst = nullptr;
    if (!is_q) {
        if (!write_cache) return;
        int kv_head = is_k ? head - n_heads : head - n_heads - n_kv_heads;
        int b = tok_seq[t];
        int page = block_table[(size_t)b * table_stride + ((pos / LLMB_PAGE) % ring_pages)];
        size_t offset = (((size_t)page * n_kv_heads + kv_head) * LLMB_PAGE + (pos % LLMB_PAGE)) * head_dim;
        dst = (is_k ? k_cache : v_cache) + offset;
    }
    if (is_q || is_k) {
        const float* angles = table ? table + (size_t)pos * n_rot : nullptr;
        T* out = is_q ? src : dst;
        for (int p = threadIdx.x; p < half; p += blockDim.x) {
            int i0 = interleaved ? 2 * p : p;
            int i1 = interleaved ? 2 * p + 1 : p + half;
            float low = to_float(src[i0]), high = to_float(src[i1]);
            float c = angles ? angles[p] : 1.f, s = angles ? angles[half + p] : 0.f;
            out[i0] = from_float<T>(low * c - high * s);
            out[i1] = from_float<T>(low * s + high * c);
        }
        if (is_k)                                                      // the part that is not rotated
            for (int d = n_rot + threadIdx.x; d < head_dim; d += blockDim.x) dst[d] = src[d];
    } else {
        for (int d = threadIdx.x; d < head_dim; d += blockDim.x) dst[d] = src[d];
    }
}

// The same work for bfloat16 with 16-byte accesses (head_dim and n_rot multiples of 16): one
// block per token, every thread takes items of 8 rotation pairs (two 16-byte pieces of a head)
// or 8 values that are only copied (a key's elements beyond n_rot, a v head).
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ table,
                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                      const int* __restrict__ block_table, int table_stride, int ring_pages,
                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                      int n_heads, int n_kv_heads, int head_dim, int n_rot, int interleaved, int write_cache) {
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x;
    int pos = tok_pos[t];
    int half = n_rot >> 1;
    int items_rot = n_rot >> 4;                          // items of 8 pairs per rotated head
    int items_tail = (head_dim - n_rot) >> 3;            // items of 8 values of a key beyond n_rot
    int items_copy = head_dim >> 3;                      // items of 8 values per v head
    int n_rot_heads = n_heads + n_kv_heads;
    int rot_total = n_rot_heads * items_rot;
    int tail_total = write_cache ? n_kv_heads * items_tail : 0;
    int total = rot_total + tail_total + (write_cache ? n_kv_heads * items_copy : 0);
    __nv_bfloat16* row = qkv + (size_t)t * (n_heads + 2 * n_kv_heads) * head_dim;
    size_t page_base = 0;
    if (write_cache) {
        int page = block_table[(size_t)tok_seq[t] * table_stride + ((pos / LLMB_PAGE) % ring_pages)];
        page_base = (size_t)page * n_kv_heads * LLMB_PAGE * head_dim + (size_t)(pos % LLMB_PAGE) * head_dim;
    }
    const float* angles = table ? table + (size_t)pos * n_rot : nullptr;
    for (int item = threadIdx.x; item < total; item += blockDim.x) {
        if (item < rot_total) {
            int head = item / items_rot, piece = item - head * items_rot;
            bool is_q = head < n_heads;
            if (!is_q && !write_cache) continue;
            __nv_bfloat16* src = row + (size_t)head * head_dim;
            __nv_bfloat16* dst = is_q ? src
                                      : k_cache + page_base + (size_t)(head - n_heads) * LLMB_PAGE * head_dim;
            int p0 = piece * 8;                           // first of this item's 8 pairs
            int at_lo = interleaved ? 2 * p0 : p0, at_hi = interleaved ? 2 * p0 + 8 : p0 + half;
            uint4 raw_lo = *reinterpret_cast<const uint4*>(src + at_lo);
            uint4 raw_hi = *reinterpret_cast<const uint4*>(src + at_hi);
            __nv_bfloat16* lo = reinterpret_cast<__nv_bfloat16*>(&raw_lo);
            __nv_bfloat16* hi = reinterpret_cast<__nv_bfloat16*>(&raw_hi);
            float c[8], s[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                c[i] = angles ? angles[p0 + i] : 1.f;
                s[i] = angles ? angles[half + p0 + i] : 0.f;
            }
            if (interleaved) {
                // pair i of this item is elements (2i, 2i+1) of the 16 loaded values
                __nv_bfloat16 all[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) { all[i] = lo[i]; all[8 + i] = hi[i]; }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a = __bfloat162float(all[2 * i]), b = __bfloat162float(all[2 * i + 1]);
                    all[2 * i] = __float2bfloat16_rn(a * c[i] - b * s[i]);
                    all[2 * i + 1] = __float2bfloat16_rn(a * s[i] + b * c[i]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) { lo[i] = all[i]; hi[i] = all[8 + i]; }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a = __bfloat162float(lo[i]), b = __bfloat162float(hi[i]);
                    lo[i] = __float2bfloat16_rn(a * c[i] - b * s[i]);
                    hi[i] = __float2bfloat16_rn(a * s[i] + b * c[i]);
                }
            }
            *reinterpret_cast<uint4*>(dst + at_lo) = raw_lo;
            *reinterpret_cast<uint4*>(dst + at_hi) = raw_hi;
        } else if (item < rot_total + tail_total) {
            int rest = item - rot_total;
            int kv_head = rest / items_tail, piece = rest - kv_head * items_tail;
            const __nv_bfloat16* src = row + (size_t)(n_heads + kv_head) * head_dim + n_rot + piece * 8;
            __nv_bfloat16* dst = k_cache + page_base + (size_t)kv_head * LLMB_PAGE * head_dim + n_rot + piece * 8;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        } else {
            int rest = item - rot_total - tail_total;
            int kv_head = rest / items_copy, piece = rest - kv_head * items_copy;
            const __nv_bfloat16* src = row + (size_t)(n_rot_heads + kv_head) * head_dim + piece * 8;
            __nv_bfloat16* dst = v_cache + page_base + (size_t)kv_head * LLMB_PAGE * head_dim + piece * 8;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        }
    }
}

LLMB_EXPORT int llmb_rope_cache_write(void* qkv, int dtype, const float* table,
                                      const int* tok_pos, const int* tok_seq,
                                      const int* block_table, int table_stride, int ring_pages,
                                      void* k_cache, void* v_cache, int n_tokens, int n_heads,
                                      int n_kv_heads, int head_dim, int n_rot, int interleaved,
                                      int write_cache, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "rope: head_dim %d must be even", head_dim);
    LLMB_REQUIRE(n_rot >= 0 && n_rot <= head_dim && n_rot % 2 == 0,
                 "rope: the rotated part %d must be even and at most head_dim %d", n_rot, head_dim);
    LLMB_REQUIRE(n_heads > 0 && n_kv_heads > 0 && ring_pages > 0, "rope: bad sizes");
    LLMB_REQUIRE(n_heads + 2 * n_kv_heads <= 65535, "rope: too many heads");
    if (dtype == LLMB_DTYPE_BF16 && head_dim % 16 == 0 && n_rot % 16 == 0 &&
        ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) |
          reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0) {
        llmb::launch(rope_cache_vec_kernel, n_tokens, 256, 0, stream, true,
                     (__nv_bfloat16*)qkv, table, tok_pos, tok_seq, block_table, table_stride, ring_pages,
                     (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_heads, n_kv_heads, head_dim, n_rot,
                     interleaved, write_cache);
        return check_launch("rope_cache_write");
    }
    dim3 grid(n_tokens, n_heads + 2 * n_kv_heads);
    int threads = head_dim / 2 >= 64 ? 64 : 32;
    if (dtype == LLMB_DTYPE_F32)
        rope_cache_kernel<float><<<grid, threads, 0, stream>>>(
            (float*)qkv, table, tok_pos, tok_seq, block_table, table_stride, ring_pages,
            (float*)k_cache, (float*)v_cache, n_heads, n_kv_heads, head_dim, n_rot, interleaved, write_cache);
    else if (dtype == LLMB_DTYPE_BF16)
        rope_cache_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
            (__nv_bfloat16*)qkv, table, tok_pos, tok_seq, block_table, table_stride, ring_pages,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_heads, n_kv_heads, head_dim, n_rot,
            interleaved, write_cache);
    else
        return fail(LLMB_ERR_ARGUMENT, "rope: unknown dtype %d", dtype);
    return check_launch("rope_cache_write");
}

// ----------------------------------------------------------------------------- scaling in place
// x *= scale over n 32-bit values (the logits of an architecture with a logit scale).
__global__ void scale_kernel(float* __restrict__ x, long long n, float scale) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] *= scale;
}

LLMB_EXPORT int llmb_scale(float* x, long long n, float scale, cudaStream_t stream) {
    if (n <= 0) return LLMB_OK;
    int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    scale_kernel<<<blocks, 256, 0, stream>>>(x, n, scale);
    return check_launch("scale");
}

// ----------------------------------------------------------------------------- gated activation
// act[t, f] = silu(gu[t, f]) * gu[t, F + f], silu(z) = z / (1 + exp(-z))
// (apps/engine/kernels/gpu.cu:409-418, apps/engine/src/ops.rs:33-35). The gate
// and up projections are one matrix product whose row holds [gate | up].
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, long long total,
                              int width) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        long long t = i / width;
        int f = (int)(i - t * width);
        float g = to_float(gu[t * 2 * width + f]);
        float u = to_float(gu[t * 2 * width + width + f]);
        act[i] = from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 rows whose width is a multiple of 8: 16 bytes of gate and of up per thread and step
__global__ void swiglu_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act,
                                  long long total_vectors, int vectors_per_row) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total_vectors; i += stride) {
        long long t = i / vectors_per_row;
        int f = (int)(i - t * vectors_per_row);
        const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * vectors_per_row * 8);
        uint4 raw_g = row[f], raw_u = row[vectors_per_row + f];
        const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&raw_g);
        const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&raw_u);
        uint4 packed;
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&packed);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float gate = __bfloat162float(g[j]);
            o[j] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * __bfloat162float(u[j]));
        }
        reinterpret_cast<uint4*>(act)[i] = packed;
    }
}

LLMB_EXPORT int llmb_swiglu(const void* gu, void* act, int dtype, int n_tokens, int width,
                            cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(n_tokens > 0 && width > 0, "swiglu: bad sizes");
    long long total = (long long)n_tokens * width;
    if (dtype == LLMB_DTYPE_BF16 && width % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(act)) & 15) == 0) {
        long long vectors = total / 8;
        int blocks = (int)((vectors + 255) / 256 < 148 * 16 ? (vectors + 255) / 256 : 148 * 16);
        swiglu_vec_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act,
                                                      vectors, width / 8);
        return check_launch("swiglu");
    }
    int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == LLMB_DTYPE_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, (float*)act, total, width);
    else if (dtype == LLMB_DTYPE_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act, total, width);
    else
        return fail(LLMB_ERR_ARGUMENT, "swiglu: unknown dtype %d", dtype);
    return check_launch("swiglu");
}

// ----------------------------------------------------------------------------- random weights
// out[i] = mean + deviation * N(0, 1) keyed by (key, i): the formulas of random_normal.h, the same
// bits as the host library's llmh_random_normal gives.
template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, float mean,
                                     float deviation) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) out[i] = from_float<T>(llmb_random::value(key, (uint64_t)i, mean, deviation));
}

LLMB_EXPORT int llmb_random_normal(void* out, int dtype, long long n, unsigned long long key, float mean,
                                   float deviation, cudaStream_t stream) {
    if (n <= 0) return LLMB_OK;
    int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == LLMB_DTYPE_F32)
        random_normal_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, n, key, mean, deviation);
    else if (dtype == LLMB_DTYPE_BF16)
        random_normal_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, n, key, mean, deviation);
    else
        return fail(LLMB_ERR_ARGUMENT, "random_normal: unknown dtype %d", dtype);
    return check_launch("random_normal");
}

// the packed doors of the launching entry points (common.cuh)
LLMB_PACKED(llmb_embed)
LLMB_PACKED(llmb_rmsnorm)
LLMB_PACKED(llmb_cast_sumsq)
LLMB_PACKED(llmb_scale_rows)
LLMB_PACKED(llmb_rope_cache_write)
LLMB_PACKED(llmb_scale)
LLMB_PACKED(llmb_swiglu)
