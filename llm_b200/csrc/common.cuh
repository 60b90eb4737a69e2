// Shared helpers of every kernel file: element types, error reporting, launch checks.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and
// a stream, and returns 0 or an LLMB_ERR_* code; the text of the last error of
// the calling thread is read with <file prefix>_last_error(). Kernels read
// positions, lengths and page tables from device arrays, never from launch
// arguments, so that a captured step replays on new values (the device-side
// [position, visible] words of MythEclipse/llm, apps/engine/src/cuda/mod.rs:184-195,
// generalised to arrays).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <type_traits>
#include <utility>

#define LLMB_OK 0
#define LLMB_ERR_ARGUMENT 1    // a size or option this kernel refuses
#define LLMB_ERR_CUDA 2        // a CUDA call failed
#define LLMB_ERR_TIMEOUT 3     // a bounded device-side wait ran out

#define LLMB_DTYPE_F32 0
#define LLMB_DTYPE_BF16 1

#include "plan.h"              // LLMB_PAGE and the other constants shared with the host library

namespace llmb {

inline char* error_buffer() {
    static thread_local char buffer[512] = {0};
    return buffer;
}

template <typename... Args>
inline int fail(int code, const char* format, Args... args) {
    snprintf(error_buffer(), 512, format, args...);
    return code;
}
inline int fail(int code, const char* text) {
    snprintf(error_buffer(), 512, "%s", text);
    return code;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(LLMB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return LLMB_OK;
}

#define LLMB_REQUIRE(cond, ...)                                              \
    do {                                                                     \
        if (!(cond)) return llmb::fail(LLMB_ERR_ARGUMENT, __VA_ARGS__);      \
    } while (0)

#define LLMB_CUDA(call)                                                      \
    do {                                                                     \
        cudaError_t e_ = (call);                                             \
        if (e_ != cudaSuccess)                                               \
            return llmb::fail(LLMB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// Programmatic dependent launch: a kernel launched with `dependent` may begin while the kernel
// before it in the stream is still running, once every block of that kernel has called
// griddep_launch() (or has exited). Everything it does before its own griddep_wait() overlaps the
// predecessor, so that part may only touch what no kernel of a step writes: weights and its own
// shared memory. griddep_wait() returns when the predecessor has completed and its writes are
// visible. Both calls do nothing in a kernel launched the plain way. LLMB_NO_PDL=1 turns every
// launch into a plain one.
inline bool pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* off = std::getenv("LLMB_NO_PDL");
        enabled = (off && off[0] && off[0] != '0') ? 0 : 1;
    }
    return enabled == 1;
}

template <typename... Params, typename... Args>
inline cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          bool dependent, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = (dependent && pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, Params(args)...);
}

}  // namespace llmb

// Built with -DLLMB_TRACE (LLMB_NVCC_FLAGS=-DLLMB_TRACE), a kernel stamps the GPU's global timer
// (nanoseconds) at the phases it names with LLMB_STAMP(slot, thread): thread `thread` of each of the
// first LLMB_TRACE_BLOCKS blocks (numbered x fastest) writes slot `slot` of its block's row. Otherwise the
// macro is empty. llmb_read_trace copies the rows to the host (and zeroes them if `clear`): 0, or 1 in a
// build without stamps, 2 on a CUDA error. Each library has a buffer of its own.
#define LLMB_TRACE_BLOCKS 296
#define LLMB_TRACE_SLOTS 12
#ifdef LLMB_TRACE
__device__ unsigned long long llmb_trace_buffer[LLMB_TRACE_BLOCKS * LLMB_TRACE_SLOTS];
__device__ __forceinline__ unsigned long long llmb_global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define LLMB_STAMP(slot, thread)                                                          \
    do {                                                                                  \
        unsigned block_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;  \
        if (threadIdx.x == (thread) && block_ < LLMB_TRACE_BLOCKS)                        \
            llmb_trace_buffer[block_ * LLMB_TRACE_SLOTS + (slot)] = llmb_global_timer();  \
    } while (0)
inline int llmb_read_trace(unsigned long long* out, int clear) {
    size_t bytes = sizeof(unsigned long long) * LLMB_TRACE_BLOCKS * LLMB_TRACE_SLOTS;
    if (cudaMemcpyFromSymbol(out, llmb_trace_buffer, bytes) != cudaSuccess) return 2;
    if (clear) {
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, llmb_trace_buffer) != cudaSuccess || cudaMemset(address, 0, bytes) != cudaSuccess)
            return 2;
    }
    return 0;
}
#else
#define LLMB_STAMP(slot, thread) do { } while (0)
inline int llmb_read_trace(unsigned long long*, int) { return 1; }
#endif

#define LLMB_EXPORT extern "C" __attribute__((visibility("default")))

// A second door to every launching entry point: `name`_packed(const llmb_slot* args) takes the same
// arguments as `name`, one 8-byte slot each in the order of the signature (pointers, and the stream,
// as addresses; integers widened to 64 bits; floating point as double). A recorded pass is a list
// of such (function, argument block) pairs that the native host library walks with one call per
// launch and none of the caller's marshalling (llmh_plan_run in csrc/host/plan_run.cpp), in the way
// MythEclipse/llm's layer loop calls its kernels from native code (apps/engine/src/model.rs:755-825).
union llmb_slot {
    void* p;
    long long i;
    double f;
};

namespace llmb {
template <typename T>
inline T slot_as(const llmb_slot& s) {
    if constexpr (std::is_pointer<T>::value) return reinterpret_cast<T>(s.p);
    else if constexpr (std::is_floating_point<T>::value) return static_cast<T>(s.f);
    else return static_cast<T>(s.i);
}
template <typename R, typename... A, size_t... I>
inline R call_packed(R (*fn)(A...), const llmb_slot* a, std::index_sequence<I...>) {
    return fn(slot_as<A>(a[I])...);
}
template <typename R, typename... A>
inline R call_packed(R (*fn)(A...), const llmb_slot* a) {
    return call_packed(fn, a, std::index_sequence_for<A...>{});
}
}  // namespace llmb

#define LLMB_PACKED(name) \
    LLMB_EXPORT int name##_packed(const llmb_slot* args) { return llmb::call_packed(name, args); }

// Each .cu file is built into a library of its own and defines its own reader
// of the calling thread's last error text.
#define LLMB_DEFINE_LAST_ERROR(prefix) \
    LLMB_EXPORT const char* prefix##_last_error() { return llmb::error_buffer(); }
