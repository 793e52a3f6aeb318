// True 32-bit matrix product on the CUDA cores: C[M,N] = A[M,K] * W[N,K]^T, all
// row-major float32, `y = x W^T` as the reference defines its products
// (include/minillm/cuda/matrix.h:35; it calls cublasGemmEx in pedantic FP32 mode,
// src/minillm/cuda/matrix.cpp:30-36).  No tensor cores, no TF32, no split-K.
//
// Every output element is one accumulator that adds its K products in the order
// k = 0, 1, ..., K-1 with fused multiply-adds.  The value of C[m,n] therefore depends
// only on row m of A and row n of W, not on M, on the tile the element falls in, or on
// what else is in the batch: the same token gives the same bits however the work is cut.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool kVector>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                       float* __restrict__ C, int M, int N, int K, int lda,
                                                       int ldw, int ldc) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int load_row = tid >> 2, load_k = (tid & 3) * 4;
    const int tm = (tid >> 4) * TM, tn = (tid & 15) * TN;
    float acc[TM][TN] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        const int k = k0 + load_k;
        if (m0 + load_row < M) {
            const float* src = A + static_cast<size_t>(m0 + load_row) * lda + k;
            if (kVector && k + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(src);
                a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) a[i] = src[i];
            }
        }
        if (n0 + load_row < N) {
            const float* src = W + static_cast<size_t>(n0 + load_row) * ldw + k;
            if (kVector && k + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(src);
                w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) w[i] = src[i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[load_k + i][load_row] = a[i];
            Ws[load_k + i][load_row] = w[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][tm]);
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[kk][tn]);
            const float ar[TM] = {av.x, av.y, av.z, av.w};
            const float wr[TN] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tn + j;
            if (n < N) C[static_cast<size_t>(m) * ldc + n] = acc[i][j];
        }
    }
}

}  // namespace

MLR_API int mlr_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw,
                         int ldc, cudaStream_t stream) {
    MLR_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    MLR_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_f32: a leading dimension is smaller than its row");
    if (M == 0) return 0;
    const dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    MLR_REQUIRE(grid.y <= 65535, "gemm_f32: M=%d needs more than 65535 row tiles", M);
    const bool vector = lda % 4 == 0 && ldw % 4 == 0 && reinterpret_cast<uintptr_t>(A) % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(W) % 16 == 0;
    if (vector)
        mlr_launch((gemm_f32_kernel<true>), dim3(grid), dim3(256), 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
    else
        mlr_launch((gemm_f32_kernel<false>), dim3(grid), dim3(256), 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
    return mlr_launched("gemm_f32");
}
