// Shared declarations of the kernel library: dtype codes, error reporting, conversions, reductions.
// Every exported function returns 0 on success; otherwise ts_last_error() holds the reason.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

enum { TS_F32 = 0, TS_BF16 = 1 };

#define TS_API extern "C" __attribute__((visibility("default")))

char* ts_error_buffer();

static inline int ts_fail(const char* fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(ts_error_buffer(), 512, fmt, args);
    va_end(args);
    return 1;
}

#define TS_REQUIRE(cond, ...)                \
    do {                                     \
        if (!(cond)) return ts_fail(__VA_ARGS__); \
    } while (0)

#define TS_LAUNCH_CHECK(name)                                                         \
    do {                                                                              \
        cudaError_t e_ = cudaGetLastError();                                          \
        if (e_ != cudaSuccess) return ts_fail("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round to the activation dtype and come back: where the model materialises a tensor.
template <typename T>
__device__ __forceinline__ float round_to(float v) { return to_float<T>(from_float<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block in a fixed order (lane tree, then warps in index order): every thread gets it.
// One barrier: every thread adds up the warps' sums itself, in the same order.  `scratch` must not be
// in use by other threads when the call begins.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nwarps; ++w) t += scratch[w];
    return t;
}

// Programmatic dependent launch.  A kernel launched through launch_chained() may start while the
// kernel before it on the stream is still running: it may read what no kernel on the stream writes
// (weights, tables) at once, and must call chain_wait() before it reads anything an earlier kernel
// produced and before its first write to global memory; chain_wait() returns when every earlier
// kernel has finished and its writes are visible.  chain_release() lets the next kernel on the
// stream start in the same way.  Launched normally, both calls do nothing.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool ts_chaining_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ts_chaining_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define TS_CHAINED_CHECK(name, expr)                                                              \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess) return ts_fail("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    } while (0)

// Geometry of one cache entry inside a layer group's key (or value) pool.  The pool is laid out
// [page][entry][kv head][token in page][head_dim]; offsets are in elements.
struct KVGeometry {
    long long page_stride;    // entries * kv_heads * page_tokens * head_dim
    long long entry_offset;   // index of the entry in its group * kv_heads * page_tokens * head_dim
    int page_tokens;
    int num_pages;
};
