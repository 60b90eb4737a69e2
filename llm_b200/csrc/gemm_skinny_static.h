// llmb_gemm_skinny_static: the decode matrix product for callers that cannot allocate.
//
// This entry point has no counterpart in MythEclipse/llm; it is an addition of this
// library.
//
// Who it is for. llmb_gemm_skinny (gemm_skinny.cu) splits K over many warps and needs
// scratch for their partial sums and for one counter per tile of 16 output rows; its
// caller passes that scratch in, which means the caller has to own device memory
// beyond the product's inputs and outputs. Some callers have no way to get any: code
// that runs inside a region where cudaMalloc is forbidden or would stall everything
// (a plug-in called from another engine's step with a fixed memory budget, a callback
// on a stream whose owner has already handed out all device memory, a host program
// written in a language binding that exposes kernel launches but no allocator). For
// them this function keeps the scratch inside the library: two file-scope
// `static __device__` arrays in gemm_skinny.cu, 4 MiB of partial sums and 8192
// counters. Every GPU that loads the library holds those 4 MiB + 32 KiB until the
// process exits, whether the function is called or not.
//
// What the caller still passes: x [M, K] and w [N, K] (bfloat16, K contiguous, 16-byte
// aligned, K and ldx multiples of 8), optionally bias [N] (32-bit), and either `out`
// ([M, ldo], 32-bit or bfloat16 by out_dtype) or `residual` ([M, ldo] 32-bit, added
// into). Nothing is allocated or freed, here or in anything this calls: no cudaMalloc,
// no cudaFree, no allocating library routine.
//
// Limits. 1 <= M <= 64. The partial sums of a call (llmb_gemm_skinny_scratch_bytes(M,
// N, K)) must fit the 4 MiB and N must be at most 16 * 8192 = 131072; a call beyond
// either is refused with LLMB_ERR_ARGUMENT and a text that names both numbers
// (llmb_gemm_skinny_last_error()). Every decode product of a Llama-3.1-8B at up to 8
// rows fits; at 64 rows the wide ones do not.
//
// First call on a device. It looks the two arrays' device addresses up with
// cudaGetSymbolAddress (with that device current) and clears the counters once; make
// this first call before any stream capture begins on that device. Later calls only
// launch the kernel. The clearing repeats what loading the library has done already
// (`__device__` arrays start as zeros): it is there so that the counters' starting value
// does not rest on that, and it is the only reason why the first call has to come before
// a capture. The set-up is not guarded against two host threads making a device's first
// call at the same moment: both would look up the same two addresses, store the same
// values and clear the same counters, which is harmless as long as neither has a kernel
// of this entry point in flight yet; callers that share a device between threads should
// make the first call from one of them.
//
// Sharing. All calls on a device use the same arrays, and the arrays keep whatever the
// last call left: the partial sums are overwritten before they are read, and the
// counters are returned to zero by the block that finishes each tile, so calls that
// run one after the other (the same stream, or streams ordered by events) need no
// clearing in between. Two calls that overlap on the GPU race on both arrays and
// give wrong sums; so does a call that overlaps with nothing but was preceded by a
// call that was torn down half way (its counters may be non-zero).
#pragma once

#include <cuda_runtime.h>

#define LLMB_GEMM_SKINNY_STATIC_FLOATS (1 << 20)       /* 4 MiB of partial sums */
#define LLMB_GEMM_SKINNY_STATIC_COUNTERS 8192          /* one per 16 output rows */

extern "C" int llmb_gemm_skinny_static(const void* x, int ldx, const void* w, const float* bias,
                                       void* out, int out_dtype, float* residual, int M, int N,
                                       int K, int ldo, cudaStream_t stream);
