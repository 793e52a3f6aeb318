// Shared by every kernel module: the C ABI conventions, error reporting, and small
// device helpers.  Each module is compiled into its own shared library, so the
// `static` objects below exist once per module.
//
// ABI: every exported function returns 0 on success; on a refused size or a failed
// launch it returns non-zero and `mlr_last_error()` of the same module gives the
// reason.  Pointers are device pointers unless a parameter comment says otherwise;
// `stream` is a cudaStream_t.  Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#define MLR_API extern "C" __attribute__((visibility("default")))

static thread_local char mlr_error_text[512];

static int mlr_fail(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(mlr_error_text, sizeof(mlr_error_text), format, args);
    va_end(args);
    return 1;
}

MLR_API const char* mlr_last_error() { return mlr_error_text; }

// After a launch: reports a launch failure without synchronising.
static int mlr_launched(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return mlr_fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

#define MLR_REQUIRE(condition, ...) \
    do {                            \
        if (!(condition)) return mlr_fail(__VA_ARGS__); \
    } while (0)

// Status bits kernels may set in a device status word instead of trapping.
enum : int { MLR_STATUS_BAD_INDEX = 1, MLR_STATUS_BAD_PAGE = 2, MLR_STATUS_NONFINITE = 4 };

// ---- element access in either precision; arithmetic is always float ----
__device__ __forceinline__ float mlr_load(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float mlr_load(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void mlr_store(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void mlr_store(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float mlr_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float mlr_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed reduction tree (the result does not depend on timing).
// `scratch` holds at least 32 floats of shared memory.  Every thread gets the sum.
__device__ __forceinline__ float mlr_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = mlr_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = lane < warps ? scratch[lane] : 0.0f;
    total = mlr_warp_sum(total);
    return total;
}

__device__ __forceinline__ float mlr_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = mlr_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = lane < warps ? scratch[lane] : -INFINITY;
    total = mlr_warp_max(total);
    return total;
}
