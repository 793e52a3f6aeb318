// Matrix products for a few tokens (decode): out[M, N] = x[M, K] W[N, K]^T with M <= 16,
// bfloat16 inputs, float32 accumulation.  With so few rows the product reads every weight
// once and does almost no arithmetic: the kernel is a weight streamer.
//
//   * Thread blocks are persistent: block b walks the 16-row tiles b, b + grid, ... of W and
//     never drains its pipeline between tiles.
//   * Warp 4 copies: for every (tile, 1024-wide slice of K) it waits for a free stage and
//     issues one bulk copy (cp.async.bulk, completion counted on an mbarrier) per weight
//     row, 2 KB each, into rows padded by 64 bytes (16-byte shared loads of 8 rows x 4
//     threads then touch every bank once).
//   * Warps 0-3 multiply: each takes every fourth 32-wide block of the slice.  The weights
//     are the A operand of mma.sync m16n8k16 (16 weight rows x 16 k), the tokens the B
//     operand (16 k x 8 tokens), so a tile of 16 outputs for up to 16 tokens costs two
//     mma per 16 k.  Within a 32-wide block the k index is permuted so that a thread's
//     fragments for two mma steps are one 16-byte load of a weight row (from shared
//     memory) and one of a token row (from global memory, cached): no ldmatrix.
//   * At the end of a tile the four warps' partial sums are added in a fixed order through
//     shared memory and written: as bfloat16, as float32, or, for the stacked gate/up
//     matrix, as silu(gate) * up (rows 0-7 of a tile are 8 gate rows, rows 8-15 the 8 up
//     rows of the same outputs, so the gate is applied in registers).
//
// The reference sends these products to cublasGemmEx like all others
// (src/minillm/cuda/matrix.cpp:30-36; on its GPU they resolve to gemv kernels,
// benchmarks/results/cuda-model-profiler/analysis.md:15-35).  Every wait is bounded.
#include "common.cuh"

namespace {

constexpr int kThreads = 160;          // 4 multiply warps + 1 copy warp
constexpr int kStages = 3;
constexpr int kSliceK = 1024;          // k values per stage
constexpr int kRowPitch = kSliceK * 2 + 64;
constexpr int kStageBytes = 16 * kRowPitch;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Waits for a phase, but gives up after about two seconds.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > 4000000000LL) return false;
    }
    return true;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

enum Epilogue : int { kStoreBf16 = 0, kStoreF32 = 1, kSwigluBf16 = 2 };

// Row of W that row r (0..15) of tile `tile` reads.  Plain: 16 consecutive rows.  Gate/up:
// rows 0-7 are gate rows 8*tile .., rows 8-15 the up rows of the same outputs.
__device__ __forceinline__ int weight_row(int tile, int r, int n_rows, int epilogue) {
    if (epilogue == kSwigluBf16) {
        const int inter = n_rows >> 1;
        const int column = min(tile * 8 + (r & 7), inter - 1);
        return r < 8 ? column : inter + column;
    }
    return min(tile * 16 + r, n_rows - 1);
}

// NT: token tiles of 8 (1 for M <= 8, 2 for M <= 16).
template <int NT>
__global__ void __launch_bounds__(kThreads) gemv_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int M,
                                                        const __nv_bfloat16* __restrict__ W, int ldw, int n_rows,
                                                        int K, void* __restrict__ out, int ldo, int epilogue,
                                                        int tiles, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long barriers[2 * kStages];
    __shared__ float reduce[2][4][16][8 * NT];
    __shared__ int fault;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t smem_base = smem_u32(smem), bar_base = smem_u32(barriers);
    auto stage_at = [&](int s) { return smem_base + s * kStageBytes; };
    auto full_bar = [&](int s) { return bar_base + s * 8; };
    auto empty_bar = [&](int s) { return bar_base + (kStages + s) * 8; };
    if (threadIdx.x == 0) {
        fault = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();
    const int slices = (K + kSliceK - 1) / kSliceK;

    if (warp == 4) {
        // ---------------- the copy warp
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const int row = weight_row(tile, lane & 15, n_rows, epilogue);
            const __nv_bfloat16* src_row = W + static_cast<size_t>(row) * ldw;
            for (int slice = 0; slice < slices; ++slice, ++it) {
                const int stage = it % kStages;
                if (it >= kStages) ok = mbar_wait(empty_bar(stage), ((it / kStages) - 1) & 1);
                if (!ok) break;
                const int k0 = slice * kSliceK;
                const uint32_t bytes = static_cast<uint32_t>(min(kSliceK, K - k0)) * 2;
                if (lane == 0) mbar_expect_tx(full_bar(stage), bytes * 16);
                __syncwarp();
                if (lane < 16) bulk_copy(stage_at(stage) + lane * kRowPitch, src_row + k0, bytes, full_bar(stage));
            }
        }
        if (!ok) fault = 2;
    } else {
        // ---------------- multiply warps
        const int g = lane >> 2, t = lane & 3;
        // Token rows this thread supplies as the B operand: token g of each token tile.
        const __nv_bfloat16* xrow[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xrow[nt] = nt * 8 + g < M ? x + static_cast<size_t>(nt * 8 + g) * ldx : nullptr;
        bool ok = true;
        int it = 0, parity_buffer = 0;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, parity_buffer ^= 1) {
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
            for (int slice = 0; slice < slices; ++slice, ++it) {
                const int stage = it % kStages;
                ok = mbar_wait(full_bar(stage), (it / kStages) & 1);
                if (!ok) break;
                const int k0 = slice * kSliceK;
                const int blocks = (min(kSliceK, K - k0)) >> 5;       // 32-wide blocks in this slice
                const uint32_t row_lo = stage_at(stage) + g * kRowPitch + t * 16;
                const uint32_t row_hi = row_lo + 8 * kRowPitch;
                uint4 xv[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    xv[nt] = xrow[nt] && warp < blocks ? __ldg(reinterpret_cast<const uint4*>(xrow[nt] + k0 + warp * 32 + t * 8))
                                                       : make_uint4(0u, 0u, 0u, 0u);
                for (int block = warp; block < blocks; block += 4) {
                    const uint4 lo = lds128(row_lo + block * 64), hi = lds128(row_hi + block * 64);
                    uint4 cur[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) cur[nt] = xv[nt];
                    const int next = block + 4;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                        if (next < blocks && xrow[nt])
                            xv[nt] = __ldg(reinterpret_cast<const uint4*>(xrow[nt] + k0 + next * 32 + t * 8));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        mma_bf16(acc[nt], lo.x, hi.x, lo.y, hi.y, cur[nt].x, cur[nt].y);
                        mma_bf16(acc[nt], lo.z, hi.z, lo.w, hi.w, cur[nt].z, cur[nt].w);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(stage));
            }
            if (!ok) break;
            // Partial sums of the four warps meet in shared memory (two buffers, so one
            // barrier per tile is enough).
            float(*mine)[8 * NT] = reduce[parity_buffer][warp];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mine[g][nt * 8 + 2 * t] = acc[nt][0];
                mine[g][nt * 8 + 2 * t + 1] = acc[nt][1];
                mine[g + 8][nt * 8 + 2 * t] = acc[nt][2];
                mine[g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
            }
            consumer_barrier();
            const int tid = threadIdx.x;     // 0..127
            auto total = [&](int r, int m) {
                return ((reduce[parity_buffer][0][r][m] + reduce[parity_buffer][1][r][m]) + reduce[parity_buffer][2][r][m]) +
                       reduce[parity_buffer][3][r][m];
            };
            if (epilogue == kSwigluBf16) {
                const int inter = n_rows >> 1;
                for (int idx = tid; idx < 8 * M; idx += 128) {
                    const int r = idx & 7, m = idx >> 3;
                    const int column = tile * 8 + r;
                    if (column < inter) {
                        const float gate = total(r, m), up = total(r + 8, m);
                        static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(m) * ldo + column] =
                            __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
                    }
                }
            } else {
                for (int idx = tid; idx < 16 * M; idx += 128) {
                    const int r = idx & 15, m = idx >> 4;
                    const int column = tile * 16 + r;
                    if (column < n_rows) {
                        const float v = total(r, m);
                        if (epilogue == kStoreF32)
                            static_cast<float*>(out)[static_cast<size_t>(m) * ldo + column] = v;
                        else
                            static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(m) * ldo + column] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
        if (!ok) fault = 2;
    }
    __syncthreads();
    if (fault && threadIdx.x == 0) {
        if (status) atomicOr(status, MLR_STATUS_TIMEOUT);
        for (int i = 0; i < 100; ++i) __nanosleep(1000);   // let copies in flight land before the block ends
    }
}

}  // namespace

// epilogue: 0 = out bf16 [M, n_rows]; 1 = out float32 [M, n_rows]; 2 = W is the stacked
// gate/up matrix [2 I, K] and out is bf16 [M, I] = silu(x Wgate^T) * (x Wup^T).
MLR_API int mlr_gemv_bf16(const void* x, int ldx, int M, const void* W, int ldw, int n_rows, int K, void* out, int ldo,
                          int epilogue, int* status, cudaStream_t stream) {
    MLR_REQUIRE(M >= 1 && M <= 16, "gemv_bf16: %d tokens; this kernel takes 1 to 16", M);
    MLR_REQUIRE(n_rows >= 1 && K >= 32 && K % 32 == 0, "gemv_bf16: K = %d must be a positive multiple of 32", K);
    MLR_REQUIRE(ldw >= K && ldw % 8 == 0 && ldx >= K && ldx % 8 == 0, "gemv_bf16: row strides must cover K and be multiples of 8");
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(W) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0,
                "gemv_bf16: x and W must be 16-byte aligned");
    MLR_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemv_bf16: unknown epilogue %d", epilogue);
    MLR_REQUIRE(epilogue != kSwigluBf16 || n_rows % 2 == 0, "gemv_bf16: the gate/up matrix needs an even number of rows");
    const int out_columns = epilogue == kSwigluBf16 ? n_rows / 2 : n_rows;
    MLR_REQUIRE(ldo >= out_columns, "gemv_bf16: the output row stride is smaller than the row");
    const int tiles = epilogue == kSwigluBf16 ? (n_rows / 2 + 7) / 8 : (n_rows + 15) / 16;
    const int grid = tiles < 148 * 2 ? tiles : 148 * 2;
    const size_t bytes = static_cast<size_t>(kStages) * kStageBytes;
    static thread_local bool allowed[2] = {false, false};
#define MLR_LAUNCH(NT)                                                                                             \
    do {                                                                                                           \
        if (!allowed[NT - 1]) {                                                                                    \
            const cudaError_t e = cudaFuncSetAttribute(gemv_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                       static_cast<int>(bytes));                                  \
            if (e != cudaSuccess) return mlr_fail("gemv_bf16: cannot use %zu bytes of shared memory: %s", bytes,  \
                                                  cudaGetErrorString(e));                                          \
            allowed[NT - 1] = true;                                                                                \
        }                                                                                                          \
        mlr_launch((gemv_kernel<NT>), dim3(grid), dim3(kThreads), bytes, stream, static_cast<const __nv_bfloat16*>(x), ldx, M,          \
                                                           static_cast<const __nv_bfloat16*>(W), ldw, n_rows, K,  \
                                                           out, ldo, epilogue, tiles, status);                     \
    } while (0)
    if (M <= 8) MLR_LAUNCH(1);
    else MLR_LAUNCH(2);
#undef MLR_LAUNCH
    return mlr_launched("gemv_bf16");
}
