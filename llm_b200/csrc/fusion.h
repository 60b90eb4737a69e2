// What a matrix product can do besides the product, so that a decode layer is five kernels
// instead of nine. MythEclipse/llm fuses the same neighbours into its products: the norm into
// the consumer's input format (apps/engine/kernels/gpu.cu:351-407), the rotation and the cache
// append into one kernel behind the projections (gpu.cu:525-581), the activation into the next
// product's input (gpu.cu:812-853). Here all of them ride in the product's epilogue.
//
// * norm_sumsq: the product's input rows were NOT normalised: they are the bfloat16 copy of the
//   32-bit residual rows, and the norm's gain is already folded into the weight columns. Row t of
//   the result is scaled by 1 / sqrt(sum_p norm_sumsq[t * LLMB_SUMSQ_LD + p] / norm_width + norm_eps),
//   p < norm_parts, before the bias is added: y = rstd(x) * (x . (g * W)^T) = (rstd(x) * g * x) . W^T.
// * emit_rows / emit_sumsq (products that add into the residual): the updated residual rows are also
//   written as bfloat16 [tokens, ldo] and their squares are summed per row into emit_sumsq
//   [tokens, LLMB_SUMSQ_LD], one partial sum per block of output columns: the next norm's input.
//   How many partials a call writes per row is told by llmb_gemm_tc_emit_parts().
// * rope (the q/k/v product): output columns are heads of head_dim values: n_heads query heads,
//   n_kv_heads key heads, n_kv_heads value heads. Query and key heads are rotated by the angles of
//   rope_table[position] (cos in the first half of a row of head_dim values, sin in the second;
//   pairs (p, p + head_dim/2), or (2p, 2p+1) with `interleaved`; nullptr: no rotation); queries go
//   to `out`, keys and values of token t go to row tok_pos[t] % 64 of page
//   block_table[tok_seq[t]][(tok_pos[t] / 64) % ring_pages] of the cache (unless write_cache == 0).
#pragma once

#define LLMB_SUMSQ_LD 64        // floats per row of a sum-of-squares array (most partial sums a row can have)

struct llmb_gemm_fusion {
    const float* norm_sumsq;
    int norm_parts;
    float norm_eps;
    float norm_width;
    void* emit_rows;            // bfloat16 [tokens, ldo]
    float* emit_sumsq;          // [tokens, LLMB_SUMSQ_LD]
    int rope;                   // 0: none
    int interleaved;
    int write_cache;
    int n_heads, n_kv_heads, head_dim;
    const float* rope_table;    // [positions, head_dim] or nullptr
    const int* tok_pos;
    const int* tok_seq;
    const int* block_table;
    int table_stride, ring_pages;
    void* k_cache;
    void* v_cache;
};

// bits of what a call did inside its kernels (the caller does the rest with kernels of their own)
#define LLMB_FUSED_NORM 1
#define LLMB_FUSED_EMIT 2
#define LLMB_FUSED_ROPE 4
