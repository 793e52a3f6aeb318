// Choosing the next token from float32 logits: greedy, or a draw from
// softmax(logits / temperature) by inverting the cumulative distribution.
//
// Greedy follows the reference's argmax (src/minillm/cuda/ops.cu:166-201): the largest
// value wins, ties go to the lowest id, and a row that holds a NaN or an infinity yields
// -1 and sets a status bit.  The reference samples greedily only
// (src/http_server.cpp:140-142); the temperature draw is this engine's own: with
// z_i = logit_i / T, e_i = exp(z_i - max z) in float32 and sums in float64, the token is
// the first id whose cumulative sum exceeds u * sum(e), u in [0,1) given per row by the
// host.  One block of 32 warps per row.  Each warp owns one contiguous range of ids and
// walks it 128 ids at a time (a float4 per lane, so a warp's load is 512 consecutive bytes);
// the sums are taken in a fixed order: per lane along the range, a fixed tree over the
// lanes, the warps in order.
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

// The four values at ids i .. i+3 of a row (those at or beyond `end` read as `fill`).
__device__ __forceinline__ void load4(const float* x, int i, int end, bool vector, float fill, float (&v)[4]) {
    if (vector && i + 3 < end) {
        const float4 q = *reinterpret_cast<const float4*>(x + i);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] = i + k < end ? x[i + k] : fill;
    }
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const float* __restrict__ logits, int ld, int vocab,
                                                          const float* __restrict__ temperature,
                                                          const double* __restrict__ uniform,
                                                          int* __restrict__ out, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    __shared__ Best best_of_warp[32];
    __shared__ double sum_of_warp[33];
    __shared__ int nonfinite;
    __shared__ Best winner;
    const int row = blockIdx.x;
    const float* x = logits + static_cast<size_t>(row) * ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int range = (((vocab + 31) >> 5) + 127) & ~127;          // ids per warp, a multiple of 128
    const int begin = min(vocab, warp * range), end = min(vocab, begin + range);
    const bool vector = (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    if (threadIdx.x == 0) nonfinite = 0;
    __syncthreads();

    Best best{-INFINITY, 0x7fffffff};
    bool bad = false;
    int i = begin + 4 * lane;
    if (vector) {
        // Eight loads in flight per lane while whole chunks of 128 ids remain.
        for (; i + 7 * 128 + 3 < end; i += 8 * 128) {
            float4 q[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) q[c] = *reinterpret_cast<const float4*>(x + i + c * 128);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float v[4] = {q[c].x, q[c].y, q[c].z, q[c].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    bad |= !isfinite(v[k]);
                    if (v[k] > best.value) best = Best{v[k], i + c * 128 + k};
                }
            }
        }
    }
    for (; i < end; i += 128) {
        float v[4];
        load4(x, i, end, vector, 0.0f, v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            bad |= !isfinite(v[k]);
            if (i + k < end && v[k] > best.value) best = Best{v[k], i + k};
        }
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
    auto weights = [&](int i, double (&e)[4]) {        // exp(z - max z) of ids i .. i+3 (0 beyond the range)
        float v[4];
        load4(x, i, end, vector, -INFINITY, v);
#pragma unroll
        for (int k = 0; k < 4; ++k) e[k] = i + k < end ? static_cast<double>(expf(v[k] / t - zmax)) : 0.0;
    };
    double mine = 0.0;
    for (int i = begin + 4 * lane; i < end; i += 128) {
        double e[4];
        weights(i, e);
        mine += ((e[0] + e[1]) + e[2]) + e[3];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) sum_of_warp[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        double running = 0.0;
        for (int w = 0; w < 32; ++w) {
            const double s = sum_of_warp[w];
            sum_of_warp[w] = running;       // the sum of all warps before w
            running += s;
        }
        sum_of_warp[32] = running;
        out[row] = vocab - 1;               // if rounding leaves the target beyond the last sum
    }
    __syncthreads();
    const double target = uniform[row] * sum_of_warp[32];
    if (begin >= end || target < sum_of_warp[warp] || (warp < 31 && target >= sum_of_warp[warp + 1])) return;
    // This warp's range holds the target: walk it again, 128 ids at a time, with a running
    // sum over the lanes, until the sum passes the target.
    double running = sum_of_warp[warp];
    int chosen = end - 1;                   // if this pass's rounding differs from the first one's
    for (int base = begin; base < end; base += 128) {
        double e[4];
        weights(base + 4 * lane, e);
        const double own = ((e[0] + e[1]) + e[2]) + e[3];
        double upto = own;                  // inclusive sum over lanes 0 .. lane
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double other = __shfl_up_sync(0xffffffffu, upto, o);
            if (lane >= o) upto += other;
        }
        const unsigned passed = __ballot_sync(0xffffffffu, running + upto > target);
        if (passed) {
            const int first = __ffs(passed) - 1;
            if (lane == first) {
                double sum = running + upto - own;
                chosen = min(base + 4 * lane + 3, end - 1);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    sum += e[k];
                    if (sum > target) {
                        chosen = base + 4 * lane + k;
                        break;
                    }
                }
                out[row] = min(chosen, end - 1);
            }
            return;
        }
        running += __shfl_sync(0xffffffffu, upto, 31);
    }
    if (lane == 0) out[row] = chosen;
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
