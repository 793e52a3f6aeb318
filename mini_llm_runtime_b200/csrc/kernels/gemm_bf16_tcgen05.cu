// bfloat16 matrix product on the fifth-generation tensor cores of sm_100a:
//     out[p, q] = sum_k Pm[p, k] * Qm[q, k]        (both operands row-major, K contiguous)
// written to out[p * ldo + q], or, "swapped", to out[q * ldo + p].  With Pm = activations
// and Qm = weights this is y = x W^T for prompt portions; with Pm = weights, Qm = the few
// activations of a decode step and the swapped store it is the same product arranged so
// that the weight matrix fills the 128-row side of the instruction and is streamed once.
//
// One persistent block per SM, six warps:
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of a
//               128 x 64 tile of Pm and a BN x 64 tile of Qm per stage, completion counted
//               on the stage's "full" mbarrier;
//   warp 1      allocates tensor memory (two accumulators of BN float32 columns each); one
//               lane issues tcgen05.mma (M = 128, N = BN, K = 16, four per stage) with
//               shared-memory descriptors, frees a stage with tcgen05.commit on its "empty"
//               barrier, and hands a finished accumulator over with tcgen05.commit;
//   warps 2-5   read the accumulator with tcgen05.ld (each warp its quarter of the 128
//               lanes), convert and store, and give the accumulator back.
// The main loop of the next tile overlaps the stores of the last.  Rows and columns beyond
// the operands are zero-filled by TMA on the way in and not stored on the way out; so is a
// K that is no multiple of 64.  Every barrier wait gives up after about two seconds, sets
// MLR_STATUS_TIMEOUT and lets the block leave through the common exit, which frees the
// tensor memory.
//
// The reference has no kernel of this kind: it calls cublasGemmEx for every product
// (src/minillm/cuda/matrix.cpp:30-36).
#include "tcgen05.cuh"

namespace {

using namespace mlr_tc;

constexpr int kThreads = 192;
constexpr int kTileP = 128;     // rows of Pm per tile (the M of the instruction)
constexpr int kTileK = 64;      // 64 bf16 = 128 bytes = one swizzle row
constexpr int kTilePBytes = kTileP * kTileK * 2;

template <int BN>
struct Shape {
    static constexpr int kTileQBytes = BN * kTileK * 2;
    static constexpr int kStageBytes = kTilePBytes + kTileQBytes;
    static constexpr int kStages = (200 * 1024 / kStageBytes) < 8 ? (200 * 1024 / kStageBytes) : 8;
    static constexpr int kTmemColumns = 2 * BN < 32 ? 32 : 2 * BN;      // two accumulators; a power of two >= 32
};

template <int BN>
__global__ void __launch_bounds__(kThreads) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_p,
                                                                const __grid_constant__ CUtensorMap map_q,
                                                                void* __restrict__ out_base, long long ldo, int P, int Q, int K,
                                                                int out_f32, int swapped, int k_splits,
                                                                long long split_stride, int static_operand, int* status) {
    mlr_grid_dependents_may_start();
    using S = Shape<BN>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long barriers[2 * S::kStages + 4];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int fault;
    // The tiles want 1024-byte alignment (the swizzle pattern repeats every 8 rows of 128 bytes).
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_u32(barriers);
    auto full_bar = [&](int s) { return bar_base + s * 8; };
    auto empty_bar = [&](int s) { return bar_base + (S::kStages + s) * 8; };
    auto acc_full_bar = [&](int a) { return bar_base + (2 * S::kStages + a) * 8; };
    auto acc_empty_bar = [&](int a) { return bar_base + (2 * S::kStages + 2 + a) * 8; };
    auto tile_p = [&](int s) { return smem_base + s * S::kStageBytes; };
    auto tile_q = [&](int s) { return smem_base + s * S::kStageBytes + kTilePBytes; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        fault = 0;
        for (int s = 0; s < S::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 4);
        }
        mbar_init_done();
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, S::kTmemColumns);
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    // A unit of work is an output tile and one of `k_splits` ranges of K.  With more than one
    // range, each range's sum goes to its own float32 slice of `out` (split_stride elements
    // apart); whoever reads the result adds the slices up in order.
    const int tiles_p = (P + kTileP - 1) / kTileP, tiles_q = (Q + BN - 1) / BN;
    const int tiles = tiles_p * tiles_q * k_splits;
    const int all_k_blocks = (K + kTileK - 1) / kTileK;
    auto split_of = [&](int unit) { return unit / (tiles_p * tiles_q); };
    auto first_block = [&](int split) { return static_cast<int>(static_cast<long long>(all_k_blocks) * split / k_splits); };

    if (warp == 0) {
        // ---------------- loads
        if (lane == 0) {
            // `static_operand` (1 = Pm, 2 = Qm) names an operand that no kernel writes (the
            // weights).  Its tiles for the first stages are fetched before the wait for the
            // preceding kernels, so the pipeline is full when the other operand may be read.
            int prefetched = 0;
            if (static_operand) {
                for (int unit = blockIdx.x; unit < tiles && prefetched < S::kStages; unit += gridDim.x) {
                    const int tile = unit % (tiles_p * tiles_q), split = split_of(unit);
                    const int p0 = (tile % tiles_p) * kTileP, q0 = (tile / tiles_p) * BN;
                    for (int kb = first_block(split); kb < first_block(split + 1) && prefetched < S::kStages; ++kb, ++prefetched) {
                        mbar_expect_tx(full_bar(prefetched), S::kStageBytes);
                        if (static_operand == 1) tma_load_2d(tile_p(prefetched), &map_p, kb * kTileK, p0, full_bar(prefetched));
                        else tma_load_2d(tile_q(prefetched), &map_q, kb * kTileK, q0, full_bar(prefetched));
                    }
                }
            }
            mlr_grid_wait();
            bool ok = true;
            int it = 0;
            for (int unit = blockIdx.x; unit < tiles && ok; unit += gridDim.x) {
                const int tile = unit % (tiles_p * tiles_q), split = split_of(unit);
                const int p0 = (tile % tiles_p) * kTileP, q0 = (tile / tiles_p) * BN;
                for (int kb = first_block(split); kb < first_block(split + 1); ++kb, ++it) {
                    const int stage = it % S::kStages;
                    const bool fresh = it >= prefetched;       // else the stage is announced and half loaded already
                    if (fresh && it >= S::kStages) ok = mbar_wait(empty_bar(stage), ((it / S::kStages) - 1) & 1);
                    if (!ok) break;
                    if (fresh) mbar_expect_tx(full_bar(stage), S::kStageBytes);
                    if (fresh || static_operand != 1) tma_load_2d(tile_p(stage), &map_p, kb * kTileK, p0, full_bar(stage));
                    if (fresh || static_operand != 2) tma_load_2d(tile_q(stage), &map_q, kb * kTileK, q0, full_bar(stage));
                }
            }
            if (!ok) fault = 2;
        }
    } else if (warp == 1) {
        // ---------------- tensor-core instructions
        if (lane == 0) {
            mlr_grid_wait();
            constexpr uint32_t idesc = instruction_descriptor(BN);
            bool ok = true;
            int it = 0, local = 0;
            for (int unit = blockIdx.x; unit < tiles && ok; unit += gridDim.x, ++local) {
                const int acc = local & 1;
                if (local >= 2) ok = mbar_wait(acc_empty_bar(acc), ((local >> 1) - 1) & 1);
                if (!ok) break;
                tmem_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                const int kb0 = first_block(split_of(unit)), kb1 = first_block(split_of(unit) + 1);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int stage = it % S::kStages;
                    ok = mbar_wait(full_bar(stage), (it / S::kStages) & 1);
                    if (!ok) break;
                    tmem_fence_after();
                    const uint64_t desc_p = smem_descriptor(tile_p(stage)), desc_q = smem_descriptor(tile_q(stage));
#pragma unroll
                    for (int k = 0; k < kTileK / 16; ++k)      // 16 bf16 = 32 bytes = 2 descriptor units further along K
                        umma_bf16(tmem_d, desc_p + 2 * k, desc_q + 2 * k, idesc, kb > kb0 || k > 0);
                    umma_commit(empty_bar(stage));             // the stage is free once these instructions have read it
                }
                if (!ok) break;
                umma_commit(acc_full_bar(acc));                // the accumulator is complete once all of them are done
            }
            if (!ok) fault = 2;
        }
    } else {
        // ---------------- stores: warp w reads lanes 32 (w % 4) .. of the accumulator
        const int quarter = warp & 3;
        mlr_grid_wait();
        bool ok = true;
        int local = 0;
        for (int unit = blockIdx.x; unit < tiles; unit += gridDim.x, ++local) {
            const int acc = local & 1;
            const int tile = unit % (tiles_p * tiles_q);
            const int p0 = (tile % tiles_p) * kTileP, q0 = (tile / tiles_p) * BN;
            void* out = static_cast<char*>(out_base) + static_cast<size_t>(split_of(unit)) * split_stride * (out_f32 ? 4 : 2);
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full_bar(acc), (local >> 1) & 1));     // the whole warp goes on, or none of it
            if (!ok) break;
            tmem_fence_after();
            const int p = p0 + quarter * 32 + lane;
#pragma unroll
            for (int c = 0; c < BN; c += 16) {
                uint32_t r[16];
                tmem_load16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + c, r);
                if (p < P) {
                    if (swapped) {
                        // out[q][p]: for a fixed q the 32 lanes of a warp write consecutive addresses.
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int q = q0 + c + j;
                            if (q < Q) {
                                const float v = __uint_as_float(r[j]);
                                if (out_f32) static_cast<float*>(out)[q * ldo + p] = v;
                                else static_cast<__nv_bfloat16*>(out)[q * ldo + p] = __float2bfloat16_rn(v);
                            }
                        }
                    } else if (q0 + c + 16 <= Q && (ldo & 7) == 0) {
                        // out[p][q0 + c ..]: 16 consecutive values of the thread's row.
                        if (out_f32) {
                            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(out) + p * ldo + q0 + c);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        } else {
                            uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + p * ldo + q0 + c);
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                                w[j] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int q = q0 + c + j;
                            if (q < Q) {
                                const float v = __uint_as_float(r[j]);
                                if (out_f32) static_cast<float*>(out)[p * ldo + q] = v;
                                else static_cast<__nv_bfloat16*>(out)[p * ldo + q] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                }
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
        }
        if (!ok) fault = 2;
    }
    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (fault) {
            // Give work that may still be in flight time to finish before the memory goes back.
            for (int i = 0; i < 100; ++i) __nanosleep(1000);
        }
        tmem_free(tmem_base, S::kTmemColumns);
    }
    if (fault && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_TIMEOUT);
}

// ---------------------------------------------------------------- host side
// A map over a row-major bf16 matrix [rows, cols] (row stride ld elements) that loads boxes
// of `box_rows` x 64 with the 128-byte swizzle; what lies outside the matrix reads as zero.
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    MLR_REQUIRE(encode != nullptr, "gemm_bf16_tcgen05: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {kTileK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MLR_REQUIRE(r == CUDA_SUCCESS, "gemm_bf16_tcgen05: cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
    return 0;
}

template <int BN>
int launch(const CUtensorMap& map_p, const CUtensorMap& map_q, void* out, long long ldo, int P, int Q, int K, int out_f32,
           int swapped, int k_splits, long long split_stride, int static_operand, int* status, int sms, cudaStream_t stream) {
    using S = Shape<BN>;
    const size_t bytes = static_cast<size_t>(S::kStages) * S::kStageBytes + 1024;
    static thread_local bool allowed = false;
    if (!allowed) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(bytes));
        if (e != cudaSuccess) return mlr_fail("gemm_bf16_tcgen05: cannot use %zu bytes of shared memory: %s", bytes, cudaGetErrorString(e));
        allowed = true;
    }
    const int tiles = ((P + kTileP - 1) / kTileP) * ((Q + BN - 1) / BN) * k_splits;
    const int grid = tiles < sms ? tiles : sms;
    mlr_launch((gemm_tcgen05_kernel<BN>), dim3(grid), dim3(kThreads), bytes, stream, map_p, map_q, out, ldo, P, Q, K, out_f32, swapped, k_splits,
                                                               split_stride, static_operand, status);
    return mlr_launched("gemm_bf16_tcgen05");
}

}  // namespace

// out[p, q] = sum_k Pm[p, k] Qm[q, k]; stored at out[p * ldo + q] (swapped = 0) or
// out[q * ldo + p] (swapped = 1), as bfloat16 or float32.  Pm is [P, K] with row stride ldp,
// Qm is [Q, K] with row stride ldq (elements).  tile_q: 16, 32, 64, 128 or 256 columns of Qm
// per tile (0 lets the function choose).  k_splits > 1 cuts K into that many ranges; range s
// writes its sum to the float32 slice out + s * split_stride, and the reader adds the slices.
// static_operand: 1 if no kernel in flight writes Pm (it holds weights), 2 the same for Qm, 0
// neither; the kernel fetches that operand before it waits for the kernels before it.
MLR_API int mlr_gemm_bf16_tcgen05(const void* Pm, long long ldp, int P, const void* Qm, long long ldq, int Q, int K, void* out,
                                  long long ldo, int out_f32, int swapped, int tile_q, int k_splits, long long split_stride,
                                  int static_operand, int* status, cudaStream_t stream) {
    MLR_REQUIRE(static_operand >= 0 && static_operand <= 2, "gemm_bf16_tcgen05: static_operand must be 0, 1 or 2");
    MLR_REQUIRE(k_splits >= 1 && k_splits <= (K + kTileK - 1) / kTileK, "gemm_bf16_tcgen05: %d splits of K = %d", k_splits, K);
    MLR_REQUIRE(k_splits == 1 || (out_f32 && split_stride >= 1), "gemm_bf16_tcgen05: split results are float32 slices");
    MLR_REQUIRE(P >= 1 && Q >= 1 && K >= 8, "gemm_bf16_tcgen05: bad sizes P=%d Q=%d K=%d", P, Q, K);
    MLR_REQUIRE(K % 8 == 0 && ldp % 8 == 0 && ldq % 8 == 0 && ldp >= K && ldq >= K,
                "gemm_bf16_tcgen05: K and the operand row strides must be multiples of 8 elements (16 bytes), got K=%d", K);
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(Pm) % 16 == 0 && reinterpret_cast<uintptr_t>(Qm) % 16 == 0,
                "gemm_bf16_tcgen05: the operands must be 16-byte aligned");
    MLR_REQUIRE(ldo >= (swapped ? P : Q), "gemm_bf16_tcgen05: the output row stride is smaller than the row");
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0, "gemm_bf16_tcgen05: the output must be 16-byte aligned");
    if (tile_q == 0) tile_q = Q <= 16 ? 16 : Q <= 32 ? 32 : Q <= 64 ? 64 : Q <= 128 ? 128 : 256;
    MLR_REQUIRE(tile_q == 16 || tile_q == 32 || tile_q == 64 || tile_q == 128 || tile_q == 256,
                "gemm_bf16_tcgen05: tile_q must be 16, 32, 64, 128 or 256, got %d", tile_q);
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    CUtensorMap map_p, map_q;
    if (int e = make_map(&map_p, Pm, P, K, ldp, kTileP)) return e;
    if (int e = make_map(&map_q, Qm, Q, K, ldq, tile_q)) return e;
    switch (tile_q) {
        case 16: return launch<16>(map_p, map_q, out, ldo, P, Q, K, out_f32, swapped, k_splits, split_stride, static_operand, status, sms, stream);
        case 32: return launch<32>(map_p, map_q, out, ldo, P, Q, K, out_f32, swapped, k_splits, split_stride, static_operand, status, sms, stream);
        case 64: return launch<64>(map_p, map_q, out, ldo, P, Q, K, out_f32, swapped, k_splits, split_stride, static_operand, status, sms, stream);
        case 128: return launch<128>(map_p, map_q, out, ldo, P, Q, K, out_f32, swapped, k_splits, split_stride, static_operand, status, sms, stream);
        default: return launch<256>(map_p, map_q, out, ldo, P, Q, K, out_f32, swapped, k_splits, split_stride, static_operand, status, sms, stream);
    }
}
