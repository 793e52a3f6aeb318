// Matrix-vector products for decode steps of one to four rows: out[M, N] = f(x[M, K] W[N, K]^T).
//
// With so few rows a product is a pass over the weight matrix and nothing else: 2 M flops per
// 2 bytes, far below what any arithmetic unit needs to be busy, so the tensor cores have nothing
// to add and the kernel is built around the memory system instead.  Every warp owns pairs of
// output rows; its lanes read 16 contiguous bytes of a weight row each (512 bytes per warp and
// load, streaming past L1), several loads in flight per lane, and multiply them with the step's
// activations, which the block keeps in shared memory as float32.  A row's sum is made by one
// warp in a fixed order (lane-wise partial sums, then a shuffle tree), so the result does not
// depend on the grid or on timing.  The blocks are persistent (a few per SM) and walk the row
// pairs with a fixed stride.
//
// What else would be a launch of its own is folded in:
//  * prologue: the RMS norm of the rows of the float32 residual stream that feed the product
//    (`(h * 1/sqrt(mean(h^2) + eps)) * w`, rounded to bfloat16 as the norm kernel rounds it), on
//    all rows or on the rows an index names (the final norm before the output head);
//  * epilogue: store as bfloat16 or float32, ADD into the float32 residual stream (each element
//    has one owner, so the add is a plain read-modify-write), or the SiLU gate of a stacked
//    gate/up matrix (blocks of 128 gate rows followed by their 128 "up" rows): a warp's pair of
//    rows is then (gate row, its up row) and it stores silu(gate) * up.
// Before it waits for the kernels before it, a block already asks for the first weights of its
// first rows: they are weights, nobody writes them.
//
// The reference sends these products to cuBLAS gemv kernels (src/minillm/cuda/matrix.cpp:30-36) and
// runs norm, gate and residual add as kernels of their own (src/minillm/cuda/layer.cpp:42-70).
#include "common.cuh"

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kUnroll = 4;          // 16-byte loads in flight per lane and row
constexpr int kGateBlock = 128;

enum Mode : int { kStoreBf16 = 0, kStoreF32 = 1, kAddF32 = 2, kSiluGateBf16 = 3 };

struct Params {
    const __nv_bfloat16* W;
    long long ldw;
    int N, K;
    const void* x;              // bfloat16 activations [M, K], or the float32 stream when `norm`
    long long ldx;
    int norm;
    const void* norm_weight;
    int norm_weight_bf16;
    float eps;
    const int* row_index;       // with `norm`: row r of the product is row row_index[r] of the stream (null: r)
    void* out;
    long long ldo;
    int mode;
};

__device__ __forceinline__ uint4 load_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }
// Two bfloat16 values of one 32-bit word as a pair of floats in one 64-bit register, for the packed
// float32 multiply-add of sm_100 (two sums per instruction).
__device__ __forceinline__ unsigned long long pair_of(uint32_t packed) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "r"(packed << 16), "r"(packed & 0xffff0000u));
    return r;
}
__device__ __forceinline__ void fma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;\n" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ float sum_of(unsigned long long pair) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(pair));
    return lo + hi;
}

// Which two rows of W unit `u` stands for.
__device__ __forceinline__ void rows_of_unit(int u, int mode, int& r0, int& r1) {
    if (mode == kSiluGateBf16) {
        r0 = (u / kGateBlock) * 2 * kGateBlock + u % kGateBlock;
        r1 = r0 + kGateBlock;
    } else {
        r0 = 2 * u;
        r1 = 2 * u + 1;
    }
}

template <int M>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const Params p) {
    // [M][2][K / 2] float32 (bfloat16 values): of every 8 consecutive values of a row, the first four
    // lie in the first half and the last four in the second, so that the 16-byte reads of a warp's
    // lanes fall on consecutive addresses (no bank conflicts).
    extern __shared__ __align__(16) float xs[];
    auto at = [K = p.K](int m, int k) { return m * K + ((k >> 2) & 1) * (K >> 1) + ((k >> 3) << 2) + (k & 3); };
    __shared__ float reduce_scratch[32];
    mlr_grid_dependents_may_start();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = p.K, chunks = K >> 3;                    // 16-byte chunks per row
    const int units = p.mode == kSiluGateBf16 ? p.N / 2 : (p.N + 1) / 2;
    const int first_unit = blockIdx.x * kWarps + warp, unit_stride = gridDim.x * kWarps;

    // The first weights of the first pair of rows are asked for (into L2) before anything else: weights
    // have no writer, so this may overlap the kernels before this one.
    int r0 = 0, r1 = 0;
    if (first_unit < units) {
        rows_of_unit(first_unit, p.mode, r0, r1);
        const uint4* w0 = reinterpret_cast<const uint4*>(p.W + static_cast<size_t>(r0) * p.ldw);
        const uint4* w1 = reinterpret_cast<const uint4*>(p.W + static_cast<size_t>(r1 < p.N ? r1 : r0) * p.ldw);
        const int c = lane * 8;                              // one request per 128 bytes: the first 4 KB of each row
        if (c < chunks) {
            prefetch_l2(w0 + c);
            prefetch_l2(w1 + c);
        }
    }
    mlr_grid_wait();

    // ---- the activations of the step, into shared memory
    if (p.norm) {
        const float* h = static_cast<const float*>(p.x);
        for (int m = 0; m < M; ++m) {
            const float* row = h + static_cast<size_t>(p.row_index ? p.row_index[m] : m) * p.ldx;
            float sum = 0.0f;
            for (int k = threadIdx.x * 4; k < K; k += kThreads * 4) {
                const float4 v = *reinterpret_cast<const float4*>(row + k);
                *reinterpret_cast<float4*>(xs + at(m, k)) = v;
                sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            sum = mlr_block_sum(sum, reduce_scratch);
            const float scale = 1.0f / sqrtf(sum / static_cast<float>(K) + p.eps);
            for (int k = threadIdx.x; k < K; k += kThreads) {
                const float w = p.norm_weight_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.norm_weight)[k])
                                                   : static_cast<const float*>(p.norm_weight)[k];
                xs[at(m, k)] = __bfloat162float(__float2bfloat16_rn((xs[at(m, k)] * scale) * w));
            }
        }
    } else {
        const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.x);
        for (int m = 0; m < M; ++m)
            for (int k = threadIdx.x * 8; k < K; k += kThreads * 8) {
                float v[8];
                mlr_load8(x + static_cast<size_t>(m) * p.ldx + k, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) xs[at(m, k + i)] = v[i];
            }
    }
    __syncthreads();

    // ---- the rows
    for (int unit = first_unit; unit < units; unit += unit_stride) {
        if (unit != first_unit) rows_of_unit(unit, p.mode, r0, r1);
        const bool second = r1 < p.N;
        const uint4* w0 = reinterpret_cast<const uint4*>(p.W + static_cast<size_t>(r0) * p.ldw);
        const uint4* w1 = reinterpret_cast<const uint4*>(p.W + static_cast<size_t>(second ? r1 : r0) * p.ldw);
        // Two sums per row and activation row: over the even and over the odd elements (one packed
        // multiply-add handles a word of two weights); they are added at the end, always in this order.
        unsigned long long acc2[M][2];
#pragma unroll
        for (int m = 0; m < M; ++m) acc2[m][0] = acc2[m][1] = 0ull;
        uint4 a[kUnroll], b[kUnroll];
        for (int base = 0; base < chunks; base += 32 * kUnroll) {
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int c = base + lane + 32 * u;
                a[u] = c < chunks ? load_stream(w0 + c) : make_uint4(0, 0, 0, 0);
                b[u] = c < chunks ? load_stream(w1 + c) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int c = base + lane + 32 * u;
                if (c < chunks) {
                    const unsigned long long aw[4] = {pair_of(a[u].x), pair_of(a[u].y), pair_of(a[u].z), pair_of(a[u].w)};
                    const unsigned long long bw[4] = {pair_of(b[u].x), pair_of(b[u].y), pair_of(b[u].z), pair_of(b[u].w)};
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const ulonglong2 x0 = *reinterpret_cast<const ulonglong2*>(xs + m * K + c * 4);
                        const ulonglong2 x1 = *reinterpret_cast<const ulonglong2*>(xs + m * K + (K >> 1) + c * 4);
                        const unsigned long long xv[4] = {x0.x, x0.y, x1.x, x1.y};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            fma2(acc2[m][0], aw[i], xv[i]);
                            fma2(acc2[m][1], bw[i], xv[i]);
                        }
                    }
                }
            }
        }
        float acc[M][2];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            acc[m][0] = mlr_warp_sum(sum_of(acc2[m][0]));
            acc[m][1] = mlr_warp_sum(sum_of(acc2[m][1]));
        }
        if (lane < M) {
            // Lane m writes row m of the result (every lane holds every sum after the shuffle tree).
            float y0 = 0.0f, y1 = 0.0f;
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (lane == m) { y0 = acc[m][0]; y1 = acc[m][1]; }
            const size_t row = static_cast<size_t>(lane) * p.ldo;
            if (p.mode == kSiluGateBf16) {
                const int column = (r0 / (2 * kGateBlock)) * kGateBlock + r0 % kGateBlock;
                static_cast<__nv_bfloat16*>(p.out)[row + column] = __float2bfloat16_rn((y0 / (1.0f + expf(-y0))) * y1);
            } else if (p.mode == kStoreBf16) {
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + row;
                out[r0] = __float2bfloat16_rn(y0);
                if (second) out[r1] = __float2bfloat16_rn(y1);
            } else {
                float* out = static_cast<float*>(p.out) + row;
                if (p.mode == kAddF32) {
                    out[r0] += y0;
                    if (second) out[r1] += y1;
                } else {
                    out[r0] = y0;
                    if (second) out[r1] = y1;
                }
            }
        }
    }
}

int sm_limit_bytes() {
    int device = 0, bytes = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&bytes, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    return bytes;
}

template <int M>
int launch(const Params& p, cudaStream_t stream) {
    const size_t bytes = sizeof(float) * M * static_cast<size_t>(p.K);
    static size_t allowed = 0;
    if (bytes > allowed) {
        if (cudaFuncSetAttribute(gemv_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess) {
            cudaGetLastError();
            return mlr_fail("gemv_bf16: %zu bytes of shared memory for %d rows of %d values were refused", bytes, M, p.K);
        }
        allowed = bytes;
    }
    const int units = p.mode == kSiluGateBf16 ? p.N / 2 : (p.N + 1) / 2;
    const int per_sm = bytes <= 100 * 1024 ? 2 : 1;
    const int wanted = (units + kWarps - 1) / kWarps;
    const int grid = wanted < mlr_sm_count() * per_sm ? wanted : mlr_sm_count() * per_sm;
    mlr_launch((gemv_kernel<M>), dim3(grid), dim3(kThreads), bytes, stream, p);
    return mlr_launched("gemv_bf16");
}

}  // namespace

// Whether mlr_gemv_bf16 takes a product of `M` rows over K values (its activations must fit shared memory).
MLR_API int mlr_gemv_bf16_fits(int M, int K) {
    return M >= 1 && M <= 4 && K >= 8 && K % 8 == 0 && sizeof(float) * static_cast<size_t>(M) * K + 1024 <= static_cast<size_t>(sm_limit_bytes());
}

// out = f(x W^T) for 1 <= M <= 4 rows.  W: [N, K] bfloat16, rows `ldw` elements apart (a multiple of 8),
// 16-byte aligned.  `norm` = 0: x is bfloat16 [M, K], rows `ldx` apart; `norm` = 1: x is the float32
// residual stream, rows `ldx` apart, and the product's row r is the RMS norm (weight `norm_weight`,
// bfloat16 or float32, `eps`) of its row row_index[r] (r when row_index is null), rounded to bfloat16.
// mode 0: out bfloat16 [M, N]; 1: out float32 [M, N]; 2: out float32 [M, N] += the product; 3: W is a
// stacked gate/up matrix (blocks of 128 gate rows, each followed by its 128 "up" rows; N a multiple of
// 256) and out is bfloat16 [M, N / 2] = silu(gate) * up.  `ldo`: elements between rows of out.
MLR_API int mlr_gemv_bf16(const void* W, long long ldw, int N, int K, const void* x, long long ldx, int norm,
                          const void* norm_weight, int norm_weight_bf16, float eps, const int* row_index, int M, void* out,
                          long long ldo, int mode, cudaStream_t stream) {
    MLR_REQUIRE(N >= 1 && K >= 8 && K % 8 == 0, "gemv_bf16: bad sizes N=%d K=%d (K must be a multiple of 8)", N, K);
    MLR_REQUIRE(M >= 1 && M <= 4, "gemv_bf16: takes 1 to 4 rows, got %d", M);
    MLR_REQUIRE(mode >= kStoreBf16 && mode <= kSiluGateBf16, "gemv_bf16: unknown mode %d", mode);
    MLR_REQUIRE(mode != kSiluGateBf16 || N % (2 * kGateBlock) == 0, "gemv_bf16: a stacked gate/up matrix has a multiple of 256 rows, got %d", N);
    MLR_REQUIRE(ldw % 8 == 0 && reinterpret_cast<uintptr_t>(W) % 16 == 0, "gemv_bf16: the weight rows must be 16-byte aligned");
    MLR_REQUIRE(norm ? (ldx % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && K % 4 == 0 && norm_weight != nullptr)
                     : (ldx % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0),
                "gemv_bf16: the activation rows must be 16-byte aligned (and a norm needs its weight)");
    MLR_REQUIRE(mlr_gemv_bf16_fits(M, K), "gemv_bf16: %d rows of %d values do not fit shared memory", M, K);
    Params p{static_cast<const __nv_bfloat16*>(W), ldw, N, K, x, ldx, norm, norm_weight, norm_weight_bf16, eps, row_index, out, ldo, mode};
    switch (M) {
        case 1: return launch<1>(p, stream);
        case 2: return launch<2>(p, stream);
        case 3: return launch<3>(p, stream);
        default: return launch<4>(p, stream);
    }
}
