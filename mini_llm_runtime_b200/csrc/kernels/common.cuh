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
#include <cstdlib>
#include <utility>

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

// ---- programmatic dependent launch ----
// Every kernel of the package is launched with the attribute that lets the NEXT kernel of
// the stream be set up and scheduled while this one still runs.  In exchange each kernel
//   * calls mlr_grid_dependents_may_start() at its top: once all blocks of a grid have done
//     so, the blocks of the following grid may be placed on free SM resources, and
//   * calls mlr_grid_wait() before it first reads or writes memory that earlier kernels
//     touch: the call returns when all earlier grids have finished and their writes are
//     visible.  What a kernel does before that call (barrier set-up, tensor memory, loads of
//     weights, which no kernel writes) overlaps the tail of its predecessor.
// MLR_PDL=0 in the environment launches kernels the ordinary way (both calls are then no-ops
// in effect).
__device__ __forceinline__ void mlr_grid_dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void mlr_grid_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

static bool mlr_pdl_enabled() {
    static const bool enabled = [] {
        const char* v = getenv("MLR_PDL");
        return !(v && v[0] == '0');
    }();
    return enabled;
}

template <typename... KArgs, typename... Args>
static void mlr_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = mlr_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);   // an error shows in mlr_launched()
}

// The same for a kernel whose blocks form clusters of `cluster` consecutive blocks.
template <typename... KArgs, typename... Args>
static void mlr_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster, size_t smem, cudaStream_t stream,
                               Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[2];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = mlr_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);   // an error shows in mlr_launched()
}

// Number of SMs of the current device (asked once per device and thread); grid-stride kernels
// size their grids as a multiple of it.
static int mlr_sm_count() {
    static thread_local int cached_device = -1, cached_count = 0;
    int device = 0;
    cudaGetDevice(&device);
    if (device != cached_device) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) count = 1;
        cached_device = device;
        cached_count = count;
    }
    return cached_count;
}

// Blocks of a grid-stride kernel over `units` work items of one block each: all of them, up to
// `per_sm` resident blocks on every SM.
static int mlr_grid_stride_blocks(size_t units, int per_sm) {
    const size_t limit = static_cast<size_t>(mlr_sm_count()) * per_sm;
    return static_cast<int>(units < 1 ? 1 : (units < limit ? units : limit));
}

#define MLR_REQUIRE(condition, ...) \
    do {                            \
        if (!(condition)) return mlr_fail(__VA_ARGS__); \
    } while (0)

// Status bits kernels may set in a device status word instead of trapping.
enum : int { MLR_STATUS_BAD_INDEX = 1, MLR_STATUS_BAD_PAGE = 2, MLR_STATUS_NONFINITE = 4, MLR_STATUS_TIMEOUT = 8 };

// ---- layout of a token's row in the paged cache ----
// A layer's cache is [page][K|V][kv_head][token_in_page][head_dim].  In bfloat16 caches
// with a head size of 64, 128 or 256 the 16-byte chunks of a token's row are stored
// permuted: chunk c of the token at absolute position p lives at chunk c ^ (p & 7).  A
// page block copied to shared memory byte for byte is then already laid out so that the
// eight rows of an ldmatrix fall into different banks.  Other caches store rows plainly.
// Every kernel that touches the cache derives the rule from (precision, head size) here.
__host__ __device__ inline bool mlr_cache_swizzled(bool bf16, int head_dim) {
    return bf16 && (head_dim == 64 || head_dim == 128 || head_dim == 256);
}
// Column (element index within the row) at which element `col` of the token at `position` is stored.
__host__ __device__ inline int mlr_cache_col(int col, int position, bool swizzled) {
    return swizzled ? col ^ ((position & 7) << 3) : col;
}

// ---- element access in either precision; arithmetic is always float ----
__device__ __forceinline__ float mlr_load(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float mlr_load(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void mlr_store(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void mlr_store(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// ---- 2 consecutive elements (the address must be aligned to the pair) ----
__device__ __forceinline__ void mlr_load2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x;
    b = v.y;
}
__device__ __forceinline__ void mlr_load2(const __nv_bfloat16* p, float& a, float& b) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
    a = __low2float(v);
    b = __high2float(v);
}
__device__ __forceinline__ void mlr_store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void mlr_store2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// ---- 4 and 8 consecutive elements with 8- or 16-byte accesses (the address must be aligned to the access) ----
__device__ __forceinline__ void mlr_load4(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
__device__ __forceinline__ void mlr_load4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&q.x), b = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void mlr_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void mlr_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 q;
    q.x = *reinterpret_cast<const uint32_t*>(&lo);
    q.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = q;
}
__device__ __forceinline__ void mlr_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void mlr_load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
        v[2 * i] = __low2float(h);
        v[2 * i + 1] = __high2float(h);
    }
}
__device__ __forceinline__ void mlr_store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void mlr_store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

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
