// bfloat16 matrix product for many rows (prompt portions) on pairs of SMs:
//     out[p, q] (+)= sum_k X[p, k] * W[q, k]          (both operands row-major, K contiguous)
// Two thread blocks of a cluster share one 256 x 256 output tile.  Each loads its own 128 rows
// of X and its own 128 rows of W per 64-wide block of K (TMA, 128-byte swizzle); block 0 issues
// one tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16) per 16 of K, which both SMs' tensor
// cores execute, each reading the other's half of W from its shared memory; each block ends
// up with its 128 rows of the accumulator in its own tensor memory.  Against one block per
// 128 x 256 tile this cuts what every SM fetches from L2 per flop by a third.
//
// Per block six warps, as in the one-block kernel:
//   warp 0      one lane issues the block's TMA loads; their bytes are counted on the "full"
//               barrier of the stage in block 0, which expects both blocks' bytes;
//   warp 1      allocates tensor memory (both blocks' warps together); in block 0 one lane
//               issues the instructions, frees a stage in both blocks with a multicast
//               tcgen05.commit and hands a finished accumulator to both blocks' store warps;
//   warps 2-5   read the block's accumulator rows (tcgen05.ld), apply the epilogue, store, and
//               give the accumulator back to block 0 (a remote arrival for block 1).
// Epilogues: bfloat16 or float32 store; float32 add into `out` (a product that ends a
// sub-layer adds into the residual stream); SiLU gate, for a stacked weight matrix whose rows
// alternate 128 of the gate with the 128 of "up" that belong to the same outputs, so that
// columns c and c + 128 of a tile meet in one thread: out[p, q/2 + c] = silu(g) * u.
// Every barrier wait gives up after about two seconds, sets MLR_STATUS_TIMEOUT and lets both
// blocks leave through the common exit, which frees the tensor memory.
//
// The reference calls cublasGemmEx for every product (src/minillm/cuda/matrix.cpp:30-36).
#include "tcgen05.cuh"

namespace {

using namespace mlr_tc;

constexpr int kThreads = 192;
constexpr int kRows = 128;          // rows of X, and of W, per block and stage
constexpr int kTileK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int kTileN = 256;         // columns of the pair's tile
constexpr int kOperandBytes = kRows * kTileK * 2;
constexpr int kStageBytes = 2 * kOperandBytes;          // per block
constexpr int kStages = 7;
constexpr int kTmemColumns = 2 * kTileN;                // two accumulators
enum Epilogue : int { kStoreBf16 = 0, kStoreF32 = 1, kAddF32 = 2, kSiluGateBf16 = 3 };

// dst[0..3] += (a, b, c, d), done by the memory system: the thread does not wait for the old
// values.  Every element is added to by exactly one thread, once, so the result does not
// depend on any order (the adder flushes subnormal sums to zero).
__device__ __forceinline__ void add_to_float4(float4* dst, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__global__ void __launch_bounds__(kThreads) gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                     const __grid_constant__ CUtensorMap map_w,
                                                                     void* __restrict__ out, long long ldo, int P, int Q, int K,
                                                                     int epilogue, int* status) {
    mlr_grid_dependents_may_start();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long barriers[2 * kStages + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fault;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_u32(barriers);
    auto full_bar = [&](int s) { return bar_base + s * 8; };
    auto empty_bar = [&](int s) { return bar_base + (kStages + s) * 8; };
    auto acc_full_bar = [&](int a) { return bar_base + (2 * kStages + a) * 8; };
    auto acc_empty_bar = [&](int a) { return bar_base + (2 * kStages + 2 + a) * 8; };
    auto tile_x = [&](int s) { return smem_base + s * kStageBytes; };
    auto tile_w = [&](int s) { return smem_base + s * kStageBytes + kOperandBytes; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();          // 0 leads
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        fault = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);             // used in block 0: its loader's arrival with both blocks' bytes
            mbar_init(empty_bar(s), 1);            // in both blocks: the multicast commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);         // in both blocks: the multicast commit
            mbar_init(acc_empty_bar(a), 8);        // used in block 0: four store warps of each block
        }
        mbar_init_done();
    }
    if (warp == 1) tmem_alloc_pair(&tmem_base_slot, kTmemColumns);
    tmem_fence_before();
    cluster_sync();                                // barriers and tensor memory of both blocks exist
    tmem_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int tiles_p = (P + 2 * kRows - 1) / (2 * kRows), tiles_q = (Q + kTileN - 1) / kTileN;
    const int tiles = tiles_p * tiles_q;
    const int k_blocks = (K + kTileK - 1) / kTileK;

    if (warp == 0) {
        // ---------------- loads (each block its halves)
        if (lane == 0) {
            mlr_grid_wait();
            bool ok = true;
            int it = 0;
            for (int tile = pair; tile < tiles && ok; tile += pairs) {
                const int p0 = (tile % tiles_p) * 2 * kRows + rank * kRows;
                const int q0 = (tile / tiles_p) * kTileN + rank * kRows;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int stage = it % kStages;
                    if (it >= kStages) ok = mbar_wait(empty_bar(stage), ((it / kStages) - 1) & 1);
                    if (!ok) break;
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * kStageBytes);
                    const uint32_t leader_full = in_block_of_rank(full_bar(stage), 0);
                    tma_load_2d_pair(tile_x(stage), &map_x, kb * kTileK, p0, leader_full);
                    tma_load_2d_pair(tile_w(stage), &map_w, kb * kTileK, q0, leader_full);
                }
            }
            if (!ok) fault = 2;
        }
    } else if (warp == 1) {
        // ---------------- tensor-core instructions (block 0 only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instruction_descriptor_m256(kTileN);
            bool ok = true;
            int it = 0, local = 0;
            for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
                const int acc = local & 1;
                if (local >= 2) ok = mbar_wait(acc_empty_bar(acc), ((local >> 1) - 1) & 1);
                if (!ok) break;
                tmem_fence_after();
                const uint32_t tmem_d = tmem_base + acc * kTileN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int stage = it % kStages;
                    ok = mbar_wait(full_bar(stage), (it / kStages) & 1);
                    if (!ok) break;
                    tmem_fence_after();
                    const uint64_t desc_x = smem_descriptor(tile_x(stage)), desc_w = smem_descriptor(tile_w(stage));
#pragma unroll
                    for (int k = 0; k < kTileK / 16; ++k)
                        umma_bf16_pair(tmem_d, desc_x + 2 * k, desc_w + 2 * k, idesc, kb > 0 || k > 0);
                    umma_commit_pair(empty_bar(stage), 3);      // both blocks' loaders may refill the stage
                }
                if (!ok) break;
                umma_commit_pair(acc_full_bar(acc), 3);         // both blocks' store warps may read
            }
            if (!ok) fault = 2;
        }
    } else {
        // ---------------- stores: warp w reads lanes 32 (w % 4) .. of this block's accumulator rows
        const int quarter = warp & 3;
        mlr_grid_wait();
        const uint32_t leader_acc_empty[2] = {in_block_of_rank(acc_empty_bar(0), 0), in_block_of_rank(acc_empty_bar(1), 0)};
        bool ok = true;
        int local = 0;
        for (int tile = pair; tile < tiles; tile += pairs, ++local) {
            const int acc = local & 1;
            const int p = (tile % tiles_p) * 2 * kRows + rank * kRows + quarter * 32 + lane;
            const int q0 = (tile / tiles_p) * kTileN;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full_bar(acc), (local >> 1) & 1));     // the whole warp goes on, or none of it
            if (!ok) break;
            tmem_fence_after();
            const uint32_t row_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kTileN;
            if (epilogue == kSiluGateBf16) {
                // Columns c (gate) and c + 128 (up) of the tile give output column q0 / 2 + c.
                __nv_bfloat16* dst_row = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(p) * ldo + q0 / 2;
                const int width = Q / 2 - q0 / 2;       // output columns left from this tile's first
#pragma unroll 2
                for (int c = 0; c < kTileN / 2; c += 16) {
                    uint32_t g[16], u[16];
                    tmem_load16(row_base + c, g);
                    tmem_load16(row_base + kTileN / 2 + c, u);
                    if (p < P) {
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            // The gate is rounded to bfloat16 first, as the unfused path stores it.
                            const float gate = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j])));
                            const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j])));
                            v[j] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                        }
                        if (c + 16 <= width && (ldo & 7) == 0) {
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                                w[j] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                            uint4* dst = reinterpret_cast<uint4*>(dst_row + c);
                            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c + j < width) dst_row[c + j] = __float2bfloat16_rn(v[j]);
                        }
                    }
                }
            } else {
#pragma unroll 4
                for (int c = 0; c < kTileN; c += 16) {
                    uint32_t r[16];
                    tmem_load16(row_base + c, r);
                    if (p >= P) continue;
                    const bool whole = q0 + c + 16 <= Q && (ldo & 7) == 0;
                    if (epilogue == kStoreBf16) {
                        __nv_bfloat16* dst_row = static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(p) * ldo + q0 + c;
                        if (whole) {
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                                w[j] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                            uint4* dst = reinterpret_cast<uint4*>(dst_row);
                            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (q0 + c + j < Q) dst_row[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    } else {
                        float* dst_row = static_cast<float*>(out) + static_cast<size_t>(p) * ldo + q0 + c;
                        const bool add = epilogue == kAddF32;
                        if (whole) {
                            float4* dst = reinterpret_cast<float4*>(dst_row);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (add)
                                    add_to_float4(dst + j, __uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                                else
                                    dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                         __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (q0 + c + j < Q) dst_row[j] = __uint_as_float(r[j]) + (add ? dst_row[j] : 0.0f);
                        }
                    }
                }
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acc_empty[acc]);
        }
        if (!ok) fault = 2;
    }
    tmem_fence_before();
    __syncthreads();
    if (fault && warp == 1) {
        // Give work that may still be in flight time to finish before the memory goes back.
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
    }
    cluster_sync();                                // neither block's memory goes away under the other
    if (warp == 1) tmem_free_pair(tmem_base, kTmemColumns);
    if (fault && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_TIMEOUT);
}

int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld) {
    EncodeTiled encode = encode_tiled();
    MLR_REQUIRE(encode != nullptr, "gemm_bf16_tcgen05_pair: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {kTileK, kRows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MLR_REQUIRE(r == CUDA_SUCCESS, "gemm_bf16_tcgen05_pair: cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
    return 0;
}

}  // namespace

// out[p, q] = sum_k X[p, k] W[q, k] for X [P, K] (row stride ldx) and W [Q, K] (row stride ldw),
// bfloat16.  epilogue: 0 stores bfloat16, 1 stores float32, 2 adds into float32 `out`, 3 takes
// W as 128 gate rows alternating with their 128 "up" rows (Q a multiple of 256) and stores
// bfloat16 silu(gate) * up at out[p, Q / 2 columns].  Row stride of out: ldo elements.
MLR_API int mlr_gemm_bf16_tcgen05_pair(const void* X, long long ldx, int P, const void* W, long long ldw, int Q, int K, void* out,
                                       long long ldo, int epilogue, int* status, cudaStream_t stream) {
    MLR_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_bf16_tcgen05_pair: epilogue must be 0..3, got %d", epilogue);
    MLR_REQUIRE(P >= 1 && Q >= 1 && K >= 8, "gemm_bf16_tcgen05_pair: bad sizes P=%d Q=%d K=%d", P, Q, K);
    MLR_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldx >= K && ldw >= K,
                "gemm_bf16_tcgen05_pair: K and the operand row strides must be multiples of 8 elements (16 bytes), got K=%d", K);
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(X) % 16 == 0 && reinterpret_cast<uintptr_t>(W) % 16 == 0,
                "gemm_bf16_tcgen05_pair: the operands must be 16-byte aligned");
    MLR_REQUIRE(epilogue != kSiluGateBf16 || Q % 256 == 0, "gemm_bf16_tcgen05_pair: the gated epilogue wants Q %% 256 == 0, got %d", Q);
    MLR_REQUIRE(ldo >= (epilogue == kSiluGateBf16 ? Q / 2 : Q), "gemm_bf16_tcgen05_pair: the output row stride is smaller than the row");
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0, "gemm_bf16_tcgen05_pair: the output must be 16-byte aligned");
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    CUtensorMap map_x, map_w;
    if (int e = make_map(&map_x, X, P, K, ldx)) return e;
    if (int e = make_map(&map_w, W, Q, K, ldw)) return e;
    const size_t bytes = static_cast<size_t>(kStages) * kStageBytes + 1024;
    static thread_local bool allowed = false;
    if (!allowed) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(bytes));
        if (e != cudaSuccess) return mlr_fail("gemm_bf16_tcgen05_pair: cannot use %zu bytes of shared memory: %s", bytes, cudaGetErrorString(e));
        allowed = true;
    }
    const int tiles = ((P + 2 * kRows - 1) / (2 * kRows)) * ((Q + kTileN - 1) / kTileN);
    const int pairs = tiles < sms / 2 ? tiles : sms / 2;
    mlr_launch_cluster(gemm_tcgen05_pair_kernel, dim3(2 * pairs), dim3(kThreads), 2, bytes, stream, map_x, map_w, out, ldo, P, Q, K,
                       epilogue, status);
    return mlr_launched("gemm_bf16_tcgen05_pair");
}
