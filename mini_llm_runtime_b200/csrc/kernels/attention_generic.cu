// Causal attention over the paged cache, one thread block per (query row, query head),
// for any head size up to 256 and any mix of rows: portions of prompts and single
// decoded tokens take the same path.  Arithmetic is float32 throughout (softmax, the
// running maximum and sum, the weighted sum of values); the cache and the queries are
// float32 or bfloat16.  This is the kernel of the true 32-bit path, and the fallback of
// the bfloat16 path for head sizes the tensor-core kernels refuse.
//
// Per row at position p, head h, kv head h / (Hq/Hkv), keys t in [lo, p]:
//   score_t = (q . k_t) * scale;  P = softmax(score);  out = sum_t P_t v_t
// as src/minillm/runtime.cpp:283-310 and src/minillm/cuda/attention.cu:97-218 compute it
// (there with three kernels and a materialised score matrix).  lo = 0, or
// max(0, p - window + 1) for a layer that reads a window.  Here the keys are walked in
// tiles of 64 positions aligned to multiples of 64 with a running maximum (online
// softmax), so no score matrix exists.  A row's result depends only on its position and
// on the cache contents, never on the other rows of the launch.
//
// Keys outside [lo, p] are never loaded: a cache page that is unused or stale (the pool
// is filled with NaN at start) cannot leak into a result.
#include "common.cuh"

namespace {

constexpr int kTile = 64;
constexpr int kThreads = 128;
constexpr int kMaxDimsPerThread = 2;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(kThreads) attention_generic_kernel(
    const T* __restrict__ q, int ldq, T* __restrict__ out, int ldo, const T* __restrict__ cache,
    int num_pages, const int* __restrict__ positions, const int* __restrict__ segment_of_row,
    const int* __restrict__ block_table, int table_stride, int page_size, int q_heads, int kv_heads,
    int head_dim, int window, float scale, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    long long* offsets = reinterpret_cast<long long*>(smem);  // [kTile] element offset of the token's K row
    float* scores = reinterpret_cast<float*>(offsets + kTile);  // [kTile]
    float* qs = scores + kTile;                                  // [head_dim]
    __shared__ int bad;

    const int row = blockIdx.x, head = blockIdx.y;
    const int kv_head = head / (q_heads / kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int position = positions[row];
    const int segment = segment_of_row[row];
    const int lo = window > 0 ? max(0, position - window + 1) : 0;
    const int* table = block_table + static_cast<size_t>(segment) * table_stride;
    const size_t page_elems = static_cast<size_t>(2) * kv_heads * page_size * head_dim;
    const size_t head_elems = static_cast<size_t>(page_size) * head_dim;
    const size_t value_shift = static_cast<size_t>(kv_heads) * head_elems;  // from a K row to its V row
    const bool swizzled = mlr_cache_swizzled(sizeof(T) == 2, head_dim);

    const T* qrow = q + static_cast<size_t>(row) * ldq + static_cast<size_t>(head) * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += kThreads) qs[i] = mlr_load(qrow, i);
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();

    float running_max = -INFINITY, running_sum = 0.0f;
    float acc[kMaxDimsPerThread] = {0.0f, 0.0f};

    for (int tile = (lo / kTile) * kTile; tile <= position; tile += kTile) {
        // Scores of this tile: one warp per key, lanes split the head dimension.
        for (int i = warp; i < kTile; i += kThreads / 32) {
            const int t = tile + i;
            float score = -INFINITY;
            long long offset = -1;
            if (t >= lo && t <= position) {
                const int page = table[t / page_size];
                if (page < 0 || page >= num_pages) {
                    if (lane == 0) bad = 1;
                } else {
                    offset = static_cast<long long>(page * page_elems + kv_head * head_elems +
                                                    static_cast<size_t>(t % page_size) * head_dim);
                    const T* k = cache + offset;
                    float partial = 0.0f;
                    for (int j = lane; j < head_dim; j += 32) partial = fmaf(qs[j], mlr_load(k, mlr_cache_col(j, t, swizzled)), partial);
                    score = mlr_warp_sum(partial) * scale;
                }
            }
            if (lane == 0) {
                scores[i] = score;
                offsets[i] = offset;
            }
        }
        __syncthreads();
        float tile_max = -INFINITY;
        for (int i = 0; i < kTile; ++i) tile_max = fmaxf(tile_max, scores[i]);
        const float new_max = fmaxf(running_max, tile_max);
        __syncthreads();
        if (threadIdx.x < kTile) {
            const float s = scores[threadIdx.x];
            scores[threadIdx.x] = (s == -INFINITY) ? 0.0f : expf(s - new_max);
        }
        __syncthreads();
        if (new_max > -INFINITY) {
            const float alpha = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
            running_sum *= alpha;
#pragma unroll
            for (int d = 0; d < kMaxDimsPerThread; ++d) acc[d] *= alpha;
            for (int i = 0; i < kTile; ++i) {
                const long long offset = offsets[i];
                if (offset < 0) continue;
                const int t = tile + i;
                const float p = scores[i];
                running_sum += p;
                const T* v = cache + offset + value_shift;
#pragma unroll
                for (int d = 0; d < kMaxDimsPerThread; ++d) {
                    const int c = threadIdx.x + d * kThreads;
                    if (c < head_dim) acc[d] = fmaf(p, mlr_load(v, mlr_cache_col(c, t, swizzled)), acc[d]);
                }
            }
            running_max = new_max;
        }
        __syncthreads();
    }
    if (bad && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
    T* orow = out + static_cast<size_t>(row) * ldo + static_cast<size_t>(head) * head_dim;
#pragma unroll
    for (int d = 0; d < kMaxDimsPerThread; ++d) {
        const int c = threadIdx.x + d * kThreads;
        if (c < head_dim) mlr_store(orow, c, running_sum > 0.0f ? acc[d] / running_sum : 0.0f);
    }
}

}  // namespace

MLR_API int mlr_attention_generic(const void* q, int ldq, void* out, int ldo, int act_bf16, const void* cache,
                                  int num_pages, const int* positions, const int* segment_of_row,
                                  const int* block_table, int table_stride, int page_size, int rows,
                                  int q_heads, int kv_heads, int head_dim, int window, float scale,
                                  int* status, cudaStream_t stream) {
    MLR_REQUIRE(rows >= 0 && q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0,
                "attention_generic: %d query heads cannot share %d kv heads", q_heads, kv_heads);
    MLR_REQUIRE(head_dim >= 1 && head_dim <= kThreads * kMaxDimsPerThread,
                "attention_generic: head size %d is outside [1, %d]", head_dim, kThreads * kMaxDimsPerThread);
    MLR_REQUIRE(q_heads <= 65535, "attention_generic: more than 65535 query heads");
    MLR_REQUIRE(page_size > 0 && num_pages > 0 && window >= 0, "attention_generic: bad page size, page count or window");
    MLR_REQUIRE(ldq >= q_heads * head_dim && ldo >= q_heads * head_dim, "attention_generic: a row stride is smaller than the row");
    if (rows == 0) return 0;
    const size_t shared = sizeof(float) * (head_dim + kTile) + sizeof(long long) * kTile + 16;
    const dim3 grid(rows, q_heads);
    if (act_bf16)
        mlr_launch((attention_generic_kernel<__nv_bfloat16>), dim3(grid), dim3(kThreads), shared, stream, 
            static_cast<const __nv_bfloat16*>(q), ldq, static_cast<__nv_bfloat16*>(out), ldo,
            static_cast<const __nv_bfloat16*>(cache), num_pages, positions, segment_of_row, block_table,
            table_stride, page_size, q_heads, kv_heads, head_dim, window, scale, status);
    else
        mlr_launch((attention_generic_kernel<float>), dim3(grid), dim3(kThreads), shared, stream, 
            static_cast<const float*>(q), ldq, static_cast<float*>(out), ldo, static_cast<const float*>(cache),
            num_pages, positions, segment_of_row, block_table, table_stride, page_size, q_heads, kv_heads,
            head_dim, window, scale, status);
    return mlr_launched("attention_generic");
}
