// Choosing the next token from float32 logits: greedy, or a draw from
// softmax(logits / temperature) by inverting the cumulative distribution.
//
// Greedy follows the reference's argmax (src/minillm/cuda/ops.cu:166-201): the largest
// value wins, ties go to the lowest id, and a row that holds a NaN or an infinity yields
// -1 and sets a status bit.  The reference samples greedily only
// (src/http_server.cpp:140-142); the temperature draw is this engine's own: with
// z_i = logit_i / T, e_i = exp(z_i - max z) in float32 and sums in float64, the token is
// the first id whose cumulative sum exceeds u * sum(e), u in [0,1) given per row by the
// host.  One block per row; every thread owns one contiguous run of ids, so the sums are
// taken in a fixed order.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

struct Best {
    float value;
    int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const float* __restrict__ logits, int ld, int vocab,
                                                          const float* __restrict__ temperature,
                                                          const double* __restrict__ uniform,
                                                          int* __restrict__ out, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    __shared__ Best best_of_warp[32];
    __shared__ double sums[kThreads];
    __shared__ int nonfinite;
    __shared__ Best winner;
    __shared__ double total;
    const int row = blockIdx.x;
    const float* x = logits + static_cast<size_t>(row) * ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int run = ((vocab + kThreads - 1) / kThreads + 3) & ~3;   // a multiple of 4: runs start on 16-byte boundaries
    const int begin = min(vocab, static_cast<int>(threadIdx.x) * run), end = min(vocab, begin + run);
    const bool vector = (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    if (threadIdx.x == 0) nonfinite = 0;
    __syncthreads();

    Best best{-INFINITY, 0x7fffffff};
    bool bad = false;
    int i = begin;
    if (vector) {
#pragma unroll 4
        for (; i + 3 < end; i += 4) {
            const float4 q = *reinterpret_cast<const float4*>(x + i);
            const float v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                bad |= !isfinite(v[k]);
                if (v[k] > best.value) best = Best{v[k], i + k};
            }
        }
    }
    for (; i < end; ++i) {
        const float v = x[i];
        bad |= !isfinite(v);
        if (v > best.value) best = Best{v, i};
    }
    if (bad) nonfinite = 1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
        best = better(best, other);
    }
    if (lane == 0) best_of_warp[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = best_of_warp[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, best.value, o), __shfl_xor_sync(0xffffffffu, best.index, o)};
            best = better(best, other);
        }
        if (lane == 0) winner = best;
    }
    __syncthreads();
    if (nonfinite) {
        if (threadIdx.x == 0) {
            out[row] = -1;
            if (status) atomicOr(status, MLR_STATUS_NONFINITE);
        }
        return;
    }
    const float t = temperature ? temperature[row] : 0.0f;
    if (!(t > 0.0f)) {
        if (threadIdx.x == 0) out[row] = winner.index;
        return;
    }
    // z = logit / T; its maximum is at the greedy winner because T > 0.
    const float zmax = winner.value / t;
    double mine = 0.0;
    for (int i = begin; i < end; ++i) mine += static_cast<double>(expf(x[i] / t - zmax));
    sums[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        double running = 0.0;
        for (int i = 0; i < kThreads; ++i) {
            const double s = sums[i];
            sums[i] = running;  // exclusive prefix
            running += s;
        }
        total = running;
    }
    __syncthreads();
    const double target = uniform[row] * total;
    const double before = sums[threadIdx.x];
    const double after = threadIdx.x + 1 < kThreads ? sums[threadIdx.x + 1] : total;
    if (threadIdx.x == 0) out[row] = vocab - 1;  // if rounding leaves the target beyond the last sum
    __syncthreads();
    if (begin < end && target >= before && target < after) {
        double running = before;
        int chosen = end - 1;
        for (int i = begin; i < end; ++i) {
            running += static_cast<double>(expf(x[i] / t - zmax));
            if (running > target) {
                chosen = i;
                break;
            }
        }
        out[row] = chosen;
    }
}

}  // namespace

// temperature: per row, 0 (or a null pointer) = greedy.  uniform: per row, in [0,1);
// may be null when every row is greedy.
MLR_API int mlr_sample(const float* logits, int ld, int rows, int vocab, const float* temperature,
                       const double* uniform, int* out, int* status, cudaStream_t stream) {
    MLR_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d ld=%d", rows, vocab, ld);
    MLR_REQUIRE(temperature == nullptr || uniform != nullptr, "sample: temperatures without uniform numbers");
    if (rows == 0) return 0;
    mlr_launch((sample_kernel), dim3(rows), dim3(kThreads), 0, stream, logits, ld, vocab, temperature, uniform, out, status);
    return mlr_launched("sample");
}
