// Row-wise kernels of the decoder: embedding gather, RMS norm fused with the
// residual add, per-head q/k norm + rotation + cache write, and the SiLU gate.
//
// The residual stream is always float32.  `act` tensors (what matrix products read
// and write) are float32 or bfloat16, chosen per call by `act_bf16`; weights of
// norms and the embedding table by `w_bf16`.  All arithmetic is float32.
//
// Formulas restated from the reference (paths within lilong555/mini-llm-runtime):
//   gather        src/minillm/cuda/ops.cu:60-81     out[r,:] = table[id[r],:]
//   rms norm      src/minillm/kernels.cpp:209-216   (x * 1/sqrt(mean(x^2)+eps)) * w
//   rotation      src/minillm/cuda/ops.cu:128-151   half-split, products rounded separately
//   cache write   src/minillm/cuda/attention.cu:74-95
//   gate          src/minillm/cuda/ops.cu:161       g / (1 + exp(-g)) * u
#include "common.cuh"

namespace {

// ------------------------------------------------------------------ embedding
template <typename W>
__global__ void embed_gather_kernel(float* __restrict__ out, const W* __restrict__ table,
                                    const int* __restrict__ ids, int width, int vocab, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    const int row = blockIdx.x;
    const int id = ids[row];
    float* dst = out + static_cast<size_t>(row) * width;
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_INDEX);
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = 0.0f;
        return;
    }
    const W* src = table + static_cast<size_t>(id) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = mlr_load(src, i);
}

// Eight values per thread: one 16-byte load of bf16 (or two of float), two 16-byte stores.
template <typename W>
__global__ void embed_gather_vec8_kernel(float* __restrict__ out, const W* __restrict__ table,
                                         const int* __restrict__ ids, int width, int vocab, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    const int row = blockIdx.x;
    const int id = ids[row];
    float4* dst = reinterpret_cast<float4*>(out + static_cast<size_t>(row) * width);
    const bool bad = id < 0 || id >= vocab;
    if (bad && threadIdx.x == 0 && status) atomicOr(status, MLR_STATUS_BAD_INDEX);
    const W* src = table + static_cast<size_t>(bad ? 0 : id) * width;
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) {
        float v[8];
        mlr_load8(src + i * 8, v);
        if (bad) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = 0.0f;
        }
        dst[2 * i] = make_float4(v[0], v[1], v[2], v[3]);
        dst[2 * i + 1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// ------------------------------------------------------------------ rms norm
// out[r,:] = rmsnorm(h[row,:] + delta[row,:]) * w, row = rows ? rows[r] : r.
// With write_back the sum replaces h[row,:] (the residual stream moves on).
// `delta` may come in `slices` parts, `slice_stride` elements apart (a product whose K was cut
// into ranges leaves one partial sum per range); they are added in order, then to h.
__device__ __forceinline__ float sliced(const float* p, int slices, size_t slice_stride) {
    float d = p[0];
    for (int s = 1; s < slices; ++s) d += p[s * slice_stride];
    return d;
}

template <typename T, typename W>
__global__ void rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta, int slices, size_t slice_stride,
                               const W* __restrict__ weight, T* __restrict__ out,
                               const int* __restrict__ rows, int width, float eps, int write_back) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t row = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    float* hr = h + row * width;
    const float* dr = delta ? delta + row * width : nullptr;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = dr ? hr[i] + sliced(dr + i, slices, slice_stride) : hr[i];
        sum = fmaf(x, x, sum);
    }
    sum = mlr_block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / static_cast<float>(width) + eps);
    T* dst = out + static_cast<size_t>(r) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = dr ? hr[i] + sliced(dr + i, slices, slice_stride) : hr[i];
        if (write_back && dr) hr[i] = x;
        mlr_store(dst, i, (x * scale) * mlr_load(weight, i));
    }
}

// The same for widths that are multiples of 4 and fit 16 values per thread: each thread
// keeps its values in registers between the two passes, so the row is read once and every
// load of the row is in flight at the same time.  One block per row.
template <typename T, typename W>
__global__ void __launch_bounds__(1024) rmsnorm_cached_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                             int slices, size_t slice_stride,
                                                             const W* __restrict__ weight, T* __restrict__ out,
                                                             const int* __restrict__ rows, int width, float eps,
                                                             int write_back) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const size_t row = rows ? static_cast<size_t>(rows[r]) : static_cast<size_t>(r);
    float4* hr = reinterpret_cast<float4*>(h + row * width);
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + row * width) : nullptr;
    const int quads = width >> 2;
    float4 x[4];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        x[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < quads) {
            x[k] = hr[i];
            if (dr) {
                float4 d = dr[i];
                for (int s = 1; s < slices; ++s) {
                    const float4 e = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(dr) + s * slice_stride)[i];
                    d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
                }
                x[k].x += d.x; x[k].y += d.y; x[k].z += d.z; x[k].w += d.w;
            }
        }
    }
    // A fixed order of summation per thread, then a fixed tree over the block: the result
    // depends on the width alone, not on how many rows the launch has.
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        sum = fmaf(x[k].x, x[k].x, sum);
        sum = fmaf(x[k].y, x[k].y, sum);
        sum = fmaf(x[k].z, x[k].z, sum);
        sum = fmaf(x[k].w, x[k].w, sum);
    }
    sum = mlr_block_sum(sum, scratch);
    const float scale = 1.0f / sqrtf(sum / static_cast<float>(width) + eps);
    T* dst = out + static_cast<size_t>(r) * width;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < quads) {
            if (write_back && dr) hr[i] = x[k];
            float w[4];
            mlr_load4(weight + i * 4, w);
            mlr_store4(dst + i * 4, (x[k].x * scale) * w[0], (x[k].y * scale) * w[1], (x[k].z * scale) * w[2],
                       (x[k].w * scale) * w[3]);
        }
    }
}

// ------------------------------------------------------------------ q/k norm, rotation, cache write
// One warp per (row, head).  Heads [0,Hq) are queries (normed and rotated in place),
// [Hq,Hq+Hkv) keys (normed, rotated, written to the cache; also in place), the last Hkv
// are values (copied to the cache).  The cache of one layer is
// [page][K|V][kv_head][token_in_page][D]; the page of a token is
// block_table[segment][position / page_size].
constexpr int kMaxPairsPerLane = 4;  // D/2 <= 128

// With `partials`, the input is not qkv itself but `slices` float32 partial sums of it
// ([slices][rows][ld_partial]); they are added in order as they are read, and qkv only
// receives the results.
template <typename T, typename W, bool VEC2>
__global__ void qk_norm_rope_cache_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ partials, int slices,
                                          size_t slice_stride, int ld_partial, int rows, int q_heads, int kv_heads,
                                          int head_dim, const W* __restrict__ q_weight,
                                          const W* __restrict__ k_weight, float eps,
                                          const float* __restrict__ cos_sin, int table_positions,
                                          const int* __restrict__ positions,
                                          const int* __restrict__ segment_of_row,
                                          const int* __restrict__ block_table, int table_stride,
                                          int page_size, T* __restrict__ cache, int num_pages,
                                          int write_cache, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    const int warps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    const int head = blockIdx.y * warps + (threadIdx.x >> 5);
    const int heads = q_heads + 2 * kv_heads;
    if (row >= rows || head >= heads) return;
    const int half = head_dim >> 1;
    const int position = positions[row];
    T* x = qkv + static_cast<size_t>(row) * ld + static_cast<size_t>(head) * head_dim;
    const float* xp = partials ? partials + static_cast<size_t>(row) * ld_partial + static_cast<size_t>(head) * head_dim : nullptr;
    auto input = [&](int i) { return xp ? sliced(xp + i, slices, slice_stride) : mlr_load(x, i); };
    const bool is_query = head < q_heads;
    const bool is_key = !is_query && head < q_heads + kv_heads;
    const bool is_value = !is_query && !is_key;
    if (!is_query && !write_cache) return;

    // Destination in the cache for keys and values.
    T* dst = nullptr;
    if (!is_query) {
        const int kv_head = is_key ? head - q_heads : head - q_heads - kv_heads;
        const int segment = segment_of_row[row];
        const int page = block_table[static_cast<size_t>(segment) * table_stride + position / page_size];
        if (page < 0 || page >= num_pages) {
            if (lane == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
            return;
        }
        const size_t page_elems = static_cast<size_t>(2) * kv_heads * page_size * head_dim;
        dst = cache + page * page_elems +
              (static_cast<size_t>(is_key ? 0 : 1) * kv_heads + kv_head) * page_size * head_dim +
              static_cast<size_t>(position % page_size) * head_dim;
    }
    const bool swizzled = mlr_cache_swizzled(sizeof(T) == 2, head_dim);
    // Two adjacent elements per access where the head size allows it (a multiple of 4, so that
    // both halves of a head start on a pair): wider loads and stores, same arithmetic.
    auto input2 = [&](int i, float& a, float& b) {
        if (xp) {
            float2 v = *reinterpret_cast<const float2*>(xp + i);
            for (int s = 1; s < slices; ++s) {
                const float2 e = *reinterpret_cast<const float2*>(xp + s * slice_stride + i);
                v.x += e.x;
                v.y += e.y;
            }
            a = v.x;
            b = v.y;
        } else {
            mlr_load2(x + i, a, b);
        }
    };
    if (is_value) {
        if (VEC2) {
            for (int i = 2 * lane; i < head_dim; i += 64) {
                float a, b;
                input2(i, a, b);
                mlr_store2(dst + mlr_cache_col(i, position, swizzled), a, b);
            }
        } else {
            for (int i = lane; i < head_dim; i += 32) mlr_store(dst, mlr_cache_col(i, position, swizzled), input(i));
        }
        return;
    }
    constexpr int kSlots = VEC2 ? 2 : kMaxPairsPerLane;     // VEC2: 2 x (2 + 2) elements per lane cover a head of 256
    constexpr int kWidth = VEC2 ? 2 : 1;
    float lo[kSlots][kWidth], hi[kSlots][kWidth];
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < kSlots; ++k) {
        const int j = kWidth * (lane + 32 * k);
#pragma unroll
        for (int e = 0; e < kWidth; ++e) lo[k][e] = hi[k][e] = 0.0f;
        if (j < half) {
            if (VEC2) {
                input2(j, lo[k][0], lo[k][kWidth - 1]);
                input2(j + half, hi[k][0], hi[k][kWidth - 1]);
            } else {
                lo[k][0] = input(j);
                hi[k][0] = input(j + half);
            }
#pragma unroll
            for (int e = 0; e < kWidth; ++e) {
                sum = fmaf(lo[k][e], lo[k][e], sum);
                sum = fmaf(hi[k][e], hi[k][e], sum);
            }
        }
    }
    const W* weight = is_query ? q_weight : k_weight;
    float scale = 1.0f;
    if (weight) {
        sum = mlr_warp_sum(sum);
        scale = 1.0f / sqrtf(sum / static_cast<float>(head_dim) + eps);
    }
    const bool rotate = cos_sin != nullptr;
    if (rotate && (position < 0 || position >= table_positions)) {
        if (lane == 0 && status) atomicOr(status, MLR_STATUS_BAD_INDEX);
        return;
    }
    const float* cs = rotate ? cos_sin + static_cast<size_t>(position) * head_dim : nullptr;
#pragma unroll
    for (int k = 0; k < kSlots; ++k) {
        const int j = kWidth * (lane + 32 * k);
        if (j < half) {
            float a[kWidth], b[kWidth];
#pragma unroll
            for (int e = 0; e < kWidth; ++e) {
                a[e] = lo[k][e];
                b[e] = hi[k][e];
                if (weight) {
                    a[e] = (a[e] * scale) * mlr_load(weight, j + e);
                    b[e] = (b[e] * scale) * mlr_load(weight, j + e + half);
                }
                if (rotate) {
                    const float c = cs[j + e], sn = cs[j + e + half];
                    const float ra = __fsub_rn(__fmul_rn(a[e], c), __fmul_rn(b[e], sn));
                    const float rb = __fadd_rn(__fmul_rn(a[e], sn), __fmul_rn(b[e], c));
                    a[e] = ra;
                    b[e] = rb;
                }
            }
            if (VEC2) {
                mlr_store2(x + j, a[0], a[kWidth - 1]);
                mlr_store2(x + j + half, b[0], b[kWidth - 1]);
                if (dst) {
                    mlr_store2(dst + mlr_cache_col(j, position, swizzled), a[0], a[kWidth - 1]);
                    mlr_store2(dst + mlr_cache_col(j + half, position, swizzled), b[0], b[kWidth - 1]);
                }
            } else {
                mlr_store(x, j, a[0]);
                mlr_store(x, j + half, b[0]);
                if (dst) {
                    mlr_store(dst, mlr_cache_col(j, position, swizzled), a[0]);
                    mlr_store(dst, mlr_cache_col(j + half, position, swizzled), b[0]);
                }
            }
        }
    }
}

// The same for prompt portions in bfloat16 with head sizes 64, 128 and 256 and no partial
// sums: a lane holds 8 elements of each half of a head (two 16-byte loads), D/16 lanes a
// head, so a warp covers 32 / (D/16) heads of one row and enough bytes are in flight to
// keep the memory busy.  Same arithmetic, element for element.
template <typename W, int D>
__global__ void __launch_bounds__(128) qk_norm_rope_cache_wide_kernel(
    __nv_bfloat16* __restrict__ qkv, int ld, int rows, int q_heads, int kv_heads, const W* __restrict__ q_weight,
    const W* __restrict__ k_weight, float eps, const float* __restrict__ cos_sin, int table_positions,
    const int* __restrict__ positions, const int* __restrict__ segment_of_row, const int* __restrict__ block_table,
    int table_stride, int page_size, __nv_bfloat16* __restrict__ cache, int num_pages, int write_cache, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    constexpr int kLanes = D / 16, kHeadsPerWarp = 32 / kLanes, kHalf = D / 2;
    const int lane = threadIdx.x & 31, sub = lane % kLanes;
    const int row = blockIdx.x;
    const int head = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kHeadsPerWarp + lane / kLanes;
    const int heads = q_heads + 2 * kv_heads;
    const bool is_query = head < q_heads;
    const bool is_key = !is_query && head < q_heads + kv_heads;
    const bool is_value = !is_query && !is_key && head < heads;
    bool active = head < heads && (is_query || write_cache);
    const int position = positions[row];
    __nv_bfloat16* x = qkv + static_cast<size_t>(row) * ld + static_cast<size_t>(head) * D;
    float lo[8] = {}, hi[8] = {};
    if (active) {
        mlr_load8(x + 8 * sub, lo);
        mlr_load8(x + kHalf + 8 * sub, hi);
    }
    __nv_bfloat16* dst = nullptr;
    if (active && !is_query) {
        const int kv_head = is_key ? head - q_heads : head - q_heads - kv_heads;
        const int page = block_table[static_cast<size_t>(segment_of_row[row]) * table_stride + position / page_size];
        if (page < 0 || page >= num_pages) {
            if (sub == 0 && status) atomicOr(status, MLR_STATUS_BAD_PAGE);
            active = false;
        } else {
            dst = cache + (static_cast<size_t>(page) * 2 * kv_heads + (is_key ? 0 : kv_heads) + kv_head) * page_size * D +
                  static_cast<size_t>(position % page_size) * D;
        }
    }
    // Chunks of 8 elements: the lane's low chunk is `sub`, its high chunk sub + D/16; in the
    // cache chunk c of the token at position p sits at c ^ (p & 7).
    const int chunk_lo = (sub ^ (position & 7)) * 8, chunk_hi = ((sub + kLanes) ^ (position & 7)) * 8;
    if (is_value) {
        if (active) {
            mlr_store8(dst + chunk_lo, lo);
            mlr_store8(dst + chunk_hi, hi);
        }
        return;     // a head's lanes leave together; the shuffles below stay within a head
    }
    const W* weight = is_query ? q_weight : k_weight;
    float scale = 1.0f;
    if (weight) {
        float sum = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            sum = fmaf(lo[e], lo[e], sum);
            sum = fmaf(hi[e], hi[e], sum);
        }
#pragma unroll
        for (int o = kLanes / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(__activemask(), sum, o);
        scale = 1.0f / sqrtf(sum / static_cast<float>(D) + eps);
    }
    if (!active) return;
    const bool rotate = cos_sin != nullptr;
    if (rotate && (position < 0 || position >= table_positions)) {
        if (sub == 0 && status) atomicOr(status, MLR_STATUS_BAD_INDEX);
        return;
    }
    if (weight) {
        float wl[8], wh[8];
        mlr_load8(weight + 8 * sub, wl);
        mlr_load8(weight + kHalf + 8 * sub, wh);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            lo[e] = (lo[e] * scale) * wl[e];
            hi[e] = (hi[e] * scale) * wh[e];
        }
    }
    if (rotate) {
        const float* cs = cos_sin + static_cast<size_t>(position) * D + 8 * sub;
        float c[8], sn[8];
        mlr_load8(cs, c);
        mlr_load8(cs + kHalf, sn);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float ra = __fsub_rn(__fmul_rn(lo[e], c[e]), __fmul_rn(hi[e], sn[e]));
            const float rb = __fadd_rn(__fmul_rn(lo[e], sn[e]), __fmul_rn(hi[e], c[e]));
            lo[e] = ra;
            hi[e] = rb;
        }
    }
    mlr_store8(x + 8 * sub, lo);
    mlr_store8(x + kHalf + 8 * sub, hi);
    if (dst) {
        mlr_store8(dst + chunk_lo, lo);
        mlr_store8(dst + chunk_hi, hi);
    }
}

// ------------------------------------------------------------------ SiLU gate
// gate_up is [rows, 2*inter], in blocks of `block` gate columns followed by the `block` "up"
// columns of the same outputs: output column c reads the gate at (c / block) * 2 * block +
// c % block and "up" `block` columns further.  block == inter is the plain stacking (all gates,
// then all ups); inter is a multiple of block.
__device__ __forceinline__ size_t gate_column(size_t c, int block) { return (c / block) * 2 * block + c % block; }

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int inter, int block) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    const size_t total = static_cast<size_t>(rows) * inter;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / inter, c = i - r * inter;
        const size_t at = r * 2 * inter + gate_column(c, block);
        const float g = mlr_load(gate_up, at);
        const float u = mlr_load(gate_up, at + block);
        mlr_store(out, i, (g / (1.0f + expf(-g))) * u);
    }
}

template <typename T>
__global__ void swiglu_vec8_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int inter, int block) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    // grid = (column blocks, rows): 8 consecutive columns of one row per thread (block % 8 == 0).
    const int per_row = inter >> 3;
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= per_row) return;
    const size_t r = blockIdx.y, c = static_cast<size_t>(q) * 8;
    const size_t at = r * 2 * inter + gate_column(c, block);
    float g[8], u[8];
    mlr_load8(gate_up + at, g);
    mlr_load8(gate_up + at + block, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        // A bfloat16 result keeps 8 bits: the fast exponential and division (2 ulp of float32) do.
        if (sizeof(T) == 2) g[k] = __fdividef(g[k], 1.0f + __expf(-g[k])) * u[k];
        else g[k] = (g[k] / (1.0f + expf(-g[k]))) * u[k];
    }
    mlr_store8(out + r * inter + c, g);
}
template <typename T>
__global__ void swiglu_sliced_kernel(const float* __restrict__ partials, int slices, size_t slice_stride,
                                     T* __restrict__ out, int rows, int inter, int block) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    const size_t total = static_cast<size_t>(rows) * inter;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / inter, c = i - r * inter;
        const size_t at = r * 2 * inter + gate_column(c, block);
        const float g = sliced(partials + at, slices, slice_stride);
        const float u = sliced(partials + at + block, slices, slice_stride);
        mlr_store(out, i, (g / (1.0f + expf(-g))) * u);
    }
}

int row_threads(int width) {
    int t = 32;
    while (t < 256 && t * 4 < width) t <<= 1;
    return t;
}

}  // namespace

MLR_API int mlr_embed_gather(float* out, const void* table, int w_bf16, const int* ids, int rows, int width,
                             int vocab, int* status, cudaStream_t stream) {
    MLR_REQUIRE(rows >= 0 && width > 0 && vocab > 0, "embed_gather: bad sizes rows=%d width=%d vocab=%d", rows, width, vocab);
    if (rows == 0) return 0;
    const int threads = row_threads(width);
    const bool vec = width % 8 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    if (vec && w_bf16)
        mlr_launch((embed_gather_vec8_kernel<__nv_bfloat16>), dim3(rows), dim3(row_threads(width / 2)), 0, stream, out, static_cast<const __nv_bfloat16*>(table), ids, width, vocab, status);
    else if (vec)
        mlr_launch((embed_gather_vec8_kernel<float>), dim3(rows), dim3(row_threads(width / 2)), 0, stream, out, static_cast<const float*>(table), ids, width, vocab, status);
    else if (w_bf16)
        mlr_launch((embed_gather_kernel<__nv_bfloat16>), dim3(rows), dim3(threads), 0, stream, out, static_cast<const __nv_bfloat16*>(table), ids, width, vocab, status);
    else
        mlr_launch((embed_gather_kernel<float>), dim3(rows), dim3(threads), 0, stream, out, static_cast<const float*>(table), ids, width, vocab, status);
    return mlr_launched("embed_gather");
}

MLR_API int mlr_rmsnorm(float* h, const float* delta, int slices, long long slice_stride, const void* weight, int w_bf16,
                        void* out, int act_bf16, const int* rows, int count, int width, float eps, int write_back,
                        cudaStream_t stream) {
    MLR_REQUIRE(count >= 0 && width > 0, "rmsnorm: bad sizes count=%d width=%d", count, width);
    MLR_REQUIRE(!delta || (slices >= 1 && (slices == 1 || slice_stride >= 1)), "rmsnorm: bad delta slices %d", slices);
    MLR_REQUIRE(eps > 0.0f, "rmsnorm: eps must be positive, got %g", static_cast<double>(eps));
    if (count == 0) return 0;
    const int threads = row_threads(width);
    // Register-cached path: width a multiple of 4, at most 16 values per thread of a block
    // of up to 1024 threads, 16-byte aligned rows.
    int cached_threads = 32;
    while (cached_threads < 1024 && cached_threads * 4 < width) cached_threads <<= 1;
    const bool cached = width % 4 == 0 && width <= cached_threads * 16 && reinterpret_cast<uintptr_t>(h) % 16 == 0 &&
                        (!delta || (reinterpret_cast<uintptr_t>(delta) % 16 == 0 && slice_stride % 4 == 0)) &&
                        reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(weight) % 16 == 0;
#define MLR_LAUNCH(T, W)                                                                                   \
    do {                                                                                                   \
        if (cached)                                                                                        \
            mlr_launch((rmsnorm_cached_kernel<T, W>), dim3(count), dim3(cached_threads), 0, stream,                              \
                h, delta, slices, static_cast<size_t>(slice_stride), static_cast<const W*>(weight),       \
                static_cast<T*>(out), rows, width, eps, write_back);                                       \
        else                                                                                               \
            mlr_launch((rmsnorm_kernel<T, W>), dim3(count), dim3(threads), 0, stream, h, delta, slices, static_cast<size_t>(slice_stride), \
                                                                 static_cast<const W*>(weight),            \
                                                                 static_cast<T*>(out), rows, width, eps, write_back); \
    } while (0)
    if (act_bf16 && w_bf16) MLR_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (act_bf16) MLR_LAUNCH(__nv_bfloat16, float);
    else if (w_bf16) MLR_LAUNCH(float, __nv_bfloat16);
    else MLR_LAUNCH(float, float);
#undef MLR_LAUNCH
    return mlr_launched("rmsnorm");
}

MLR_API int mlr_qk_norm_rope_cache(void* qkv, int act_bf16, int ld, const float* partials, int slices,
                                   long long slice_stride, int ld_partial, int rows, int q_heads, int kv_heads,
                                   int head_dim, const void* q_weight, const void* k_weight, int w_bf16,
                                   float eps, const float* cos_sin, int rotary_dim, int table_positions,
                                   const int* positions, const int* segment_of_row, const int* block_table,
                                   int table_stride, int page_size, void* cache, int num_pages,
                                   int write_cache, int* status, cudaStream_t stream) {
    MLR_REQUIRE(rows >= 0 && q_heads > 0 && kv_heads > 0, "qk_norm_rope_cache: bad head counts %d/%d", q_heads, kv_heads);
    MLR_REQUIRE(head_dim >= 2 && head_dim % 2 == 0 && head_dim <= 64 * kMaxPairsPerLane,
                "qk_norm_rope_cache: head size %d is not an even number in [2, %d]", head_dim, 64 * kMaxPairsPerLane);
    MLR_REQUIRE(cos_sin == nullptr || rotary_dim == head_dim,
                "qk_norm_rope_cache: rotary size %d differs from head size %d (partial rotation is not built)", rotary_dim, head_dim);
    MLR_REQUIRE(ld >= (q_heads + 2 * kv_heads) * head_dim, "qk_norm_rope_cache: row stride %d is smaller than the qkv width", ld);
    MLR_REQUIRE(!partials || (slices >= 1 && ld_partial >= (q_heads + 2 * kv_heads) * head_dim),
                "qk_norm_rope_cache: bad partial sums (%d slices, row stride %d)", slices, ld_partial);
    MLR_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "qk_norm_rope_cache: q and k norm weights must both be given or both be absent");
    MLR_REQUIRE(!write_cache || (cache && block_table && page_size > 0 && num_pages > 0), "qk_norm_rope_cache: cache write without a cache");
    if (rows == 0) return 0;
    const int warps = 4;
    // Prompt portions in bfloat16 with a head size of 64, 128 or 256: the wide kernel.
    if (act_bf16 && !partials && rows > 16 && (head_dim == 64 || head_dim == 128 || head_dim == 256) && ld % 8 == 0 &&
        reinterpret_cast<uintptr_t>(qkv) % 16 == 0 && (!cache || reinterpret_cast<uintptr_t>(cache) % 16 == 0) &&
        (!q_weight || (reinterpret_cast<uintptr_t>(q_weight) % 16 == 0 && reinterpret_cast<uintptr_t>(k_weight) % 16 == 0)) &&
        (!cos_sin || reinterpret_cast<uintptr_t>(cos_sin) % 16 == 0)) {
        const int heads_per_block = warps * 32 / (head_dim / 16);
        const dim3 wide_grid(rows, (q_heads + 2 * kv_heads + heads_per_block - 1) / heads_per_block);
#define MLR_WIDE(W, D)                                                                                         \
        mlr_launch((qk_norm_rope_cache_wide_kernel<W, D>), dim3(wide_grid), dim3(warps * 32), 0, stream,        \
                   static_cast<__nv_bfloat16*>(qkv), ld, rows, q_heads, kv_heads, static_cast<const W*>(q_weight), \
                   static_cast<const W*>(k_weight), eps, cos_sin, table_positions, positions, segment_of_row,   \
                   block_table, table_stride, page_size, static_cast<__nv_bfloat16*>(cache), num_pages, write_cache, status)
        if (w_bf16) {
            if (head_dim == 64) MLR_WIDE(__nv_bfloat16, 64);
            else if (head_dim == 128) MLR_WIDE(__nv_bfloat16, 128);
            else MLR_WIDE(__nv_bfloat16, 256);
        } else {
            if (head_dim == 64) MLR_WIDE(float, 64);
            else if (head_dim == 128) MLR_WIDE(float, 128);
            else MLR_WIDE(float, 256);
        }
#undef MLR_WIDE
        return mlr_launched("qk_norm_rope_cache (wide)");
    }
    const dim3 grid(rows, (q_heads + 2 * kv_heads + warps - 1) / warps);
    const bool vec2 = head_dim % 4 == 0 && ld % 2 == 0 && reinterpret_cast<uintptr_t>(qkv) % 8 == 0 &&
                      (!cache || reinterpret_cast<uintptr_t>(cache) % 8 == 0) &&
                      (!partials || (reinterpret_cast<uintptr_t>(partials) % 8 == 0 && ld_partial % 2 == 0 && slice_stride % 2 == 0));
#define MLR_LAUNCH(T, W)                                                                                       \
    do {                                                                                                       \
    if (vec2)                                                                                                  \
    mlr_launch((qk_norm_rope_cache_kernel<T, W, true>), dim3(grid), dim3(warps * 32), 0, stream,             \
        static_cast<T*>(qkv), ld, partials, slices, static_cast<size_t>(slice_stride), ld_partial, rows, q_heads,  \
        kv_heads, head_dim, static_cast<const W*>(q_weight),                                                   \
        static_cast<const W*>(k_weight), eps, cos_sin, table_positions, positions, segment_of_row, block_table, \
        table_stride, page_size, static_cast<T*>(cache), num_pages, write_cache, status);                      \
    else                                                                                                       \
    mlr_launch((qk_norm_rope_cache_kernel<T, W, false>), dim3(grid), dim3(warps * 32), 0, stream,                                           \
        static_cast<T*>(qkv), ld, partials, slices, static_cast<size_t>(slice_stride), ld_partial, rows, q_heads,  \
        kv_heads, head_dim, static_cast<const W*>(q_weight),                                                   \
        static_cast<const W*>(k_weight), eps, cos_sin, table_positions, positions, segment_of_row, block_table, \
        table_stride, page_size, static_cast<T*>(cache), num_pages, write_cache, status);                      \
    } while (0)
    if (act_bf16 && w_bf16) MLR_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (act_bf16) MLR_LAUNCH(__nv_bfloat16, float);
    else if (w_bf16) MLR_LAUNCH(float, __nv_bfloat16);
    else MLR_LAUNCH(float, float);
#undef MLR_LAUNCH
    return mlr_launched("qk_norm_rope_cache");
}

// out[rows, inter] = silu(gate) * up for gate_up [rows, 2 * inter] laid out in blocks of
// `block` gate columns and their `block` "up" columns (block == inter: all gates, then all ups).
MLR_API int mlr_swiglu(const void* gate_up, void* out, int act_bf16, int rows, int inter, int block, cudaStream_t stream) {
    MLR_REQUIRE(rows >= 0 && inter > 0, "swiglu: bad sizes rows=%d inter=%d", rows, inter);
    MLR_REQUIRE(block >= 1 && inter % block == 0, "swiglu: the width %d is no multiple of the gate block %d", inter, block);
    if (rows == 0) return 0;
    const size_t total = static_cast<size_t>(rows) * inter;
    const bool vec = inter % 8 == 0 && block % 8 == 0 && reinterpret_cast<uintptr_t>(gate_up) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(out) % 16 == 0;
    if (vec && rows <= 65535) {
        const dim3 vgrid((inter / 8 + 255) / 256, rows);
        if (act_bf16)
            mlr_launch((swiglu_vec8_kernel<__nv_bfloat16>), dim3(vgrid), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), rows, inter, block);
        else
            mlr_launch((swiglu_vec8_kernel<float>), dim3(vgrid), dim3(256), 0, stream, static_cast<const float*>(gate_up), static_cast<float*>(out), rows, inter, block);
        return mlr_launched("swiglu");
    }
    const int blocks = mlr_grid_stride_blocks(total / 1024 + 1, 16);
    if (act_bf16)
        mlr_launch((swiglu_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), rows, inter, block);
    else
        mlr_launch((swiglu_kernel<float>), dim3(blocks), dim3(256), 0, stream, static_cast<const float*>(gate_up), static_cast<float*>(out), rows, inter, block);
    return mlr_launched("swiglu");
}

// The same from `slices` float32 partial sums of the stacked product [slices][rows][2 * inter].
MLR_API int mlr_swiglu_sliced(const float* partials, int slices, long long slice_stride, void* out, int act_bf16, int rows,
                              int inter, int block, cudaStream_t stream) {
    MLR_REQUIRE(rows >= 0 && inter > 0 && slices >= 1, "swiglu_sliced: bad sizes rows=%d inter=%d slices=%d", rows, inter, slices);
    MLR_REQUIRE(block >= 1 && inter % block == 0, "swiglu_sliced: the width %d is no multiple of the gate block %d", inter, block);
    if (rows == 0) return 0;
    const size_t total = static_cast<size_t>(rows) * inter;
    const int blocks = mlr_grid_stride_blocks(total / 256 + 1, 16);
    if (act_bf16)
        mlr_launch((swiglu_sliced_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, partials, slices, static_cast<size_t>(slice_stride),
                                                         static_cast<__nv_bfloat16*>(out), rows, inter, block);
    else
        mlr_launch((swiglu_sliced_kernel<float>), dim3(blocks), dim3(256), 0, stream, partials, slices, static_cast<size_t>(slice_stride),
                                                         static_cast<float*>(out), rows, inter, block);
    return mlr_launched("swiglu_sliced");
}
