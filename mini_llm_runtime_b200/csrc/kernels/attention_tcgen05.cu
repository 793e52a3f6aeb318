// bfloat16 attention for prompt portions on the fifth-generation tensor cores of sm_100a,
// over the paged cache, for head sizes 64 and 128.
//
// One block per (128 query rows of one request, query head); two blocks share an SM.  The
// block walks the keys in tiles of 64 up to the diagonal (flash attention: a running maximum
// and sum per row, no score matrix in memory).  Six warps:
//   warp 4      one TMA load of the 128 query rows (128-byte swizzle), then per key tile the
//               loads of K and of V through a tensor map over the paged cache: one box per
//               page block and 64-element half of the head.  The cache stores rows already
//               swizzled (16-byte chunk c of the token at position p sits at chunk c ^ (p & 7)),
//               so each half lands in shared memory as rows of 128 bytes in exactly the layout
//               the tensor cores read, both as K (K-major) and as V (MN-major).
//   warp 5      one lane issues tcgen05.mma: S = Q K^T (M 128, N 64) into one of two score
//               buffers in tensor memory, and O += P V (M 128, N head size) with P read from
//               tensor memory.  S of the next tile is issued before P V of this one, so the
//               tensor cores work while the softmax of this tile runs.
//   warps 0-3   thread t owns query row t: reads its 64 scores from tensor memory, masks them,
//               keeps the running maximum (in log2 units; the accumulator is rescaled only when
//               the maximum grows by more than 2^8, which keeps probabilities below 256) and
//               sum in float32, writes the probabilities as bfloat16 over the scores, and at
//               the end divides its row of O by the sum and stores it.
// Rows of V outside the keys that this block may read (other requests' freed pages, slots
// not yet written) are zeroed in shared memory before P V: their probabilities are 0, and
// 0 * garbage must stay 0.  Every wait gives up after about two seconds and sets
// MLR_STATUS_TIMEOUT; the block then leaves through the common exit, which frees the tensor
// memory.
//
// Semantics are those of src/minillm/runtime.cpp:283-310 (scores scaled by `scale`, causal
// mask, softmax over t in [lo, position] in float32, weighted sum of V), with lo = 0 or
// position - window + 1.  The reference computes them with three SIMT kernels and a
// materialised score matrix (src/minillm/cuda/attention.cu:97-218).
#include "tcgen05.cuh"

namespace {

using namespace mlr_tc;

constexpr int kThreads = 192;
constexpr int kRows = 128;          // query rows per block
constexpr int kKeys = 64;           // keys per tile
constexpr int kHalfBytesPerRow = 128;
constexpr int kTmemColumns = 256;   // O: 128, two score buffers of 64
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleStep = 8.0f;    // log2 units by which the maximum may lag

// Barriers of a block.
enum Barrier { kQFull = 0, kKFull = 1, kVFull = 3, kKEmpty = 5, kVEmpty = 7, kSFull = 9, kPFull = 11, kODone = 13, kBarriers = 14 };

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// 2^x by the special-function unit alone (exp2f adds range handling around it that the
// probabilities do not need: the argument is at most kRescaleStep and -inf gives 0).
__device__ __forceinline__ float exp2_raw(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Two float32 operations in one instruction (sm_100a), and the maximum of three.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;\n"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

template <int D>
__global__ void __launch_bounds__(kThreads, 2) prefill_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
    __nv_bfloat16* __restrict__ out, int ldo, int num_pages, const int* __restrict__ tiles,
    const int* __restrict__ segment_info, const int* __restrict__ block_table, int table_stride, int page_size,
    int q_heads, int kv_heads, int window, float scale, int* status) {
    mlr_grid_dependents_may_start();
    mlr_grid_wait();
    constexpr int kHalves = D / 64;
    constexpr int kQHalfBytes = kRows * kHalfBytesPerRow;        // one 64-element half of the query tile
    constexpr int kKvHalfBytes = kKeys * kHalfBytesPerRow;       // one half of a K or V tile
    constexpr int kQBytes = kHalves * kQHalfBytes, kKvBytes = kHalves * kKvHalfBytes;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long barriers[kBarriers];
    __shared__ uint32_t tmem_slot;
    __shared__ int bad_page;   // a block-table entry outside the pool was met
    __shared__ int gave_up;    // a wait ran out
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* smem_ptr = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_tile = smem_base;
    auto k_tile = [&](int s) { return smem_base + kQBytes + s * kKvBytes; };
    auto v_offset = [&](int s) { return kQBytes + 2 * kKvBytes + s * kKvBytes; };
    auto v_tile = [&](int s) { return smem_base + v_offset(s); };
    const uint32_t bar_base = smem_u32(barriers);
    auto bar = [&](int which, int s = 0) { return bar_base + (which + s) * 8; };

    // Blocks start in the order of their index, x fastest: all heads of the first tile (the one
    // with the longest walk over the keys, as the caller sorts them), then all heads of the next.
    // The long walks so begin first and the short ones fill the gaps at the end; the heads of a
    // kv head run side by side and share its keys in L2.
    const int head = blockIdx.x;
    const int segment = tiles[blockIdx.y * 2], tile_token = tiles[blockIdx.y * 2 + 1];
    const int first_row = segment_info[segment * 4 + 0], count = segment_info[segment * 4 + 1];
    const int start = segment_info[segment * 4 + 2];
    const int kv_head = head / (q_heads / kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int tile_rows = min(kRows, count - tile_token);
    const int first_pos = start + tile_token, last_pos = first_pos + tile_rows - 1;
    const int first_key = window > 0 ? max(0, first_pos - window + 1) : 0;     // lowest key any row reads
    const int key_begin = (first_key / kKeys) * kKeys, key_end = last_pos + 1;
    const int n_tiles = (key_end - key_begin + kKeys - 1) / kKeys;

    if (threadIdx.x == 0) {
        bad_page = 0;
        gave_up = 0;
        for (int i = 0; i < kBarriers; ++i) mbar_init(bar(i), i == kPFull || i == kPFull + 1 ? 4 : 1);
        mbar_init_done();
    }
    if (warp == 5) tmem_alloc(&tmem_slot, kTmemColumns);
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const uint32_t tmem_o = tmem_base;                                       // columns 0 .. D-1
    auto tmem_s = [&](int b) { return tmem_base + 128 + b * kKeys; };        // scores; P over their first 32 columns
    // Whoever sees a wait run out says so, and every other wait of the block ends at once.
    auto wait = [&](uint32_t b, uint32_t parity) {
        if (mbar_wait(b, parity, &gave_up)) return true;
        gave_up = 1;
        return false;
    };

    if (warp == 4) {
        // ---------------- loads
        if (lane == 0) {
            mbar_expect_tx(bar(kQFull), kQBytes);
#pragma unroll
            for (int h = 0; h < kHalves; ++h)
                tma_load_2d(q_tile + h * kQHalfBytes, &map_q, head * D + h * 64, first_row + tile_token, bar(kQFull));
        }
        // Page sizes are powers of two here (the host checks it).  Lane c copies rows
        // [sub * rows_per_copy, ..) of half c % kHalves of a tile, if any key of those rows is
        // one this block may read.
        const int page_shift = 31 - __clz(page_size);
        const int rows_per_copy = min(page_size, kKeys);
        const int copies = (kKeys / rows_per_copy) * kHalves;
        const int sub = lane / kHalves, half = lane % kHalves;
        const int* table = block_table + static_cast<size_t>(segment) * table_stride;
        constexpr int kNotMine = -2;
        // The page this lane copies from in tile j.  Looked up two tiles ahead, so that the
        // table read is off the path between a stage becoming free and its next copy.
        auto lookup = [&](int j) {
            const int tile_start = key_begin + j * kKeys;
            const int from = max(tile_start, first_key), to = min(tile_start + kKeys, key_end);
            const int row0 = tile_start + sub * rows_per_copy;
            if (j >= n_tiles || lane >= copies || row0 >= to || row0 + rows_per_copy <= from) return kNotMine;
            return __ldg(table + (row0 >> page_shift));
        };
        // The K (value = 0) or V (value = 1) tile j.
        auto issue = [&](int j, int value, int page) {
            const int stage = j & 1;
            const bool mine = page != kNotMine;
            const unsigned mask = __ballot_sync(0xffffffffu, mine);
            const uint32_t full = bar(value ? kVFull : kKFull, stage);
            if (lane == 0) mbar_expect_tx(full, __popc(mask) * rows_per_copy * kHalfBytesPerRow);
            __syncwarp();
            if (mine) {
                if (page < 0 || page >= num_pages) {
                    bad_page = 1;
                    page = 0;      // still copy something so that the tile's byte count is met
                }
                const int in_page = (key_begin + j * kKeys + sub * rows_per_copy) & (page_size - 1);
                const uint32_t dst = (value ? v_tile(stage) : k_tile(stage)) + half * kKvHalfBytes +
                                     sub * rows_per_copy * kHalfBytesPerRow;
                tma_load_3d(dst, &map_kv, half * 64, in_page, (page * 2 + value) * kv_heads + kv_head, full);
            }
        };
        int page_now = lookup(0), page_next = lookup(1);
        bool ok = true;
        issue(0, 0, page_now);
        for (int j = 0; j < n_tiles && ok; ++j) {
            if (j + 1 < n_tiles) {
                if (j + 1 >= 2) ok = wait(bar(kKEmpty, (j + 1) & 1), (((j + 1) >> 1) - 1) & 1);
                if (!ok) break;
                issue(j + 1, 0, page_next);
            }
            const int page_after = lookup(j + 2);
            if (j >= 2) ok = wait(bar(kVEmpty, j & 1), ((j >> 1) - 1) & 1);
            if (!ok) break;
            issue(j, 1, page_now);
            page_now = page_next;
            page_next = page_after;
        }
    } else if (warp == 5) {
        // ---------------- tensor-core instructions
        if (lane == 0) {
            constexpr uint32_t idesc_s = instruction_descriptor(kKeys);
            constexpr uint32_t idesc_o = instruction_descriptor(D, true);
            bool ok = wait(bar(kQFull), 0);
            // Descriptors of the tiles, made once: an instruction adds a constant to them.
            const uint64_t desc_q = smem_descriptor(q_tile);
            const uint64_t desc_k[2] = {smem_descriptor(k_tile(0)), smem_descriptor(k_tile(1))};
            const uint64_t desc_v[2] = {smem_descriptor(v_tile(0), kKvHalfBytes, 1024), smem_descriptor(v_tile(1), kKvHalfBytes, 1024)};
            // S_j = Q K_j^T: per half of the head four steps of 16 along it (32 bytes = 2 units).
            auto issue_s = [&](int j) {
                const int stage = j & 1;
                if (!wait(bar(kKFull, stage), (j >> 1) & 1)) return false;
                tmem_fence_after();
                const uint32_t tmem_d = tmem_s(stage);
                const uint64_t dk = desc_k[stage];
#pragma unroll
                for (int h = 0; h < kHalves; ++h)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t da = desc_q + (h * (kQHalfBytes >> 4) + 2 * k), db = dk + (h * (kKvHalfBytes >> 4) + 2 * k);
                        if (h == 0 && k == 0) umma_bf16(tmem_d, da, db, idesc_s, 0u);
                        else umma_bf16(tmem_d, da, db, idesc_s, 1u);
                    }
                umma_commit(bar(kKEmpty, stage));
                umma_commit(bar(kSFull, stage));
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int stage = j & 1;
                if (j + 1 < n_tiles) ok = issue_s(j + 1);
                if (!ok) break;
                ok = wait(bar(kPFull, stage), (j >> 1) & 1) && wait(bar(kVFull, stage), (j >> 1) & 1);
                if (!ok) break;
                tmem_fence_after();
                // O += P_j V_j: four steps of 16 keys (16 rows of 128 bytes further into V); P holds
                // two probabilities per column, so a step is 8 columns.
                const uint32_t tmem_p = tmem_s(stage);
                const uint64_t dv = desc_v[stage];
                umma_bf16_tmem_a(tmem_o, tmem_p, dv, idesc_o, j > 0);
#pragma unroll
                for (int k = 1; k < 4; ++k)
                    umma_bf16_tmem_a(tmem_o, tmem_p + 8 * k, dv + k * ((16 * kHalfBytesPerRow) >> 4), idesc_o, 1u);
                umma_commit(bar(kVEmpty, stage));
                umma_commit(bar(kODone));
            }
        }
    } else {
        // ---------------- softmax: thread = query row
        const int row = warp * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const bool valid = row < tile_rows;
        const int hi = valid ? first_pos + row : -1;
        const int lo = window > 0 ? max(0, first_pos + row - window + 1) : 0;
        const int lo_max = window > 0 ? max(0, last_pos - window + 1) : 0;
        const float scale_log2 = scale * kLog2e;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            const uint32_t parity = (j >> 1) & 1;
            const int key0 = key_begin + j * kKeys;
            ok = __all_sync(0xffffffffu, wait(bar(kSFull, b), parity));
            if (!ok) break;
            tmem_fence_after();
            uint32_t raw[64];
            tmem_load32_nowait(tmem_s(b) + lane_base, raw);
            tmem_load32_nowait(tmem_s(b) + lane_base + 32, raw + 32);
            tmem_load_wait();
            // A tile wholly at or before the first row's position and wholly inside every
            // row's window needs no mask (rows past the request's end are not stored).
            const bool need_mask = key0 + kKeys - 1 > first_pos || key0 < lo_max;
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int key = key0 + c;
                    if (key < lo || key > hi) raw[c] = 0xff800000u;      // -inf
                }
            }
            float part_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four short chains, not one long
#pragma unroll
            for (int c = 0; c < 64; c += 2)
                part_max[(c >> 1) & 3] = max3(part_max[(c >> 1) & 3], __uint_as_float(raw[c]), __uint_as_float(raw[c + 1]));
            const float tile_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3]));
            const float m_tile = tile_max * scale_log2;      // scale_log2 > 0
            const bool grow = m_tile > m_ref + kRescaleStep || (m_ref == -INFINITY && m_tile > -INFINITY);
            // P V of tile j-1 is waited for once per tile, in order: a wait by parity can tell a
            // phase only from the one before it.  Here if O must be rescaled, else before the
            // probabilities are handed over, when it has long been done.
            bool o_seen = j == 0;
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = grow ? m_tile : m_ref;
                const float alpha = grow ? exp2_raw(m_ref - m_new) : 1.0f;       // 0 for a row's first keys
                m_ref = m_new;
                l *= alpha;
                if (j > 0) {
                    // O holds the sums up to tile j-1 once that tile's P V is done.
                    ok = __all_sync(0xffffffffu, wait(bar(kODone), (j - 1) & 1));
                    if (!ok) break;
                    o_seen = true;
                    tmem_fence_after();
#pragma unroll
                    for (int c = 0; c < D; c += 32) {
                        uint32_t o[32];
                        tmem_load32_nowait(tmem_o + lane_base + c, o);
                        tmem_load_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_store32(tmem_o + lane_base + c, o);
                    }
                }
            }
            const float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
            uint32_t p[32];
            float2 sum[4] = {{0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}};
            const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-m_use, -m_use);
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                const float2 x = fma2(make_float2(__uint_as_float(raw[c]), __uint_as_float(raw[c + 1])), scale2, shift2);
                const float2 e = make_float2(exp2_raw(x.x), exp2_raw(x.y));
                sum[(c >> 1) & 3] = add2(sum[(c >> 1) & 3], e);
                p[c >> 1] = pack_bf16(e.x, e.y);
            }
            const float2 total = add2(add2(sum[0], sum[1]), add2(sum[2], sum[3]));
            l += total.x + total.y;
            tmem_store32(tmem_s(b) + lane_base, p);
            // Rows of V that hold no key this block may read become zero.
            const int tile_end = key0 + kKeys;
            if (key0 < first_key || tile_end > key_end) {
                ok = __all_sync(0xffffffffu, wait(bar(kVFull, b), parity));
                if (!ok) break;
                constexpr int kChunks = kHalves * 8;       // 16-byte chunks per key
                for (int i = threadIdx.x; i < kKeys * kChunks; i += 128) {
                    const int key_row = i / kChunks, rest = i - key_row * kChunks;
                    const int key = key0 + key_row;
                    if (key < first_key || key >= key_end)
                        *reinterpret_cast<uint4*>(smem_ptr + v_offset(b) + (rest >> 3) * kKvHalfBytes + key_row * kHalfBytesPerRow +
                                                  (rest & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_async_proxy();
            }
            if (!o_seen) {
                ok = __all_sync(0xffffffffu, wait(bar(kODone), (j - 1) & 1));
                if (!ok) break;
            }
            tmem_store_wait();
            tmem_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kPFull, b));
        }
        if (ok) ok = __all_sync(0xffffffffu, wait(bar(kODone), (n_tiles - 1) & 1));
        if (ok) {
            tmem_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* dst = out + static_cast<size_t>(first_row + tile_token + row) * ldo + static_cast<size_t>(head) * D;
#pragma unroll
            for (int c = 0; c < D; c += 32) {
                uint32_t o[32];
                tmem_load32_nowait(tmem_o + lane_base + c, o);
                tmem_load_wait();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + i) = w;
                    }
                }
            }
        }
    }
    tmem_fence_before();
    __syncthreads();
    if (warp == 5) {
        if (gave_up) {
            // Give work that may still be in flight time to finish before the memory goes back.
            for (int i = 0; i < 100; ++i) __nanosleep(1000);
        }
        tmem_free(tmem_base, kTmemColumns);
    }
    if (threadIdx.x == 0 && status && (gave_up || bad_page))
        atomicOr(status, (gave_up ? MLR_STATUS_TIMEOUT : 0) | (bad_page ? MLR_STATUS_BAD_PAGE : 0));
}

template <int D>
int launch(const CUtensorMap& map_q, const CUtensorMap& map_kv, void* out, int ldo, int num_pages, const int* tiles, int n_tiles,
           const int* segment_info, const int* block_table, int table_stride, int page_size, int q_heads, int kv_heads,
           int window, float scale, int* status, cudaStream_t stream) {
    const size_t bytes = static_cast<size_t>(kRows) * D * 2 + 4 * static_cast<size_t>(kKeys) * D * 2 + 1024;
    static thread_local int allowed_device = -1;
    int device = 0;
    cudaGetDevice(&device);
    if (allowed_device != device) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(bytes));
        if (e != cudaSuccess)
            return mlr_fail("attention_prefill_tcgen05: cannot use %zu bytes of shared memory: %s", bytes, cudaGetErrorString(e));
        allowed_device = device;
    }
    mlr_launch((prefill_tcgen05_kernel<D>), dim3(q_heads, n_tiles), dim3(kThreads), bytes, stream, map_q, map_kv,
               static_cast<__nv_bfloat16*>(out), ldo, num_pages, tiles, segment_info, block_table, table_stride, page_size,
               q_heads, kv_heads, window, scale, status);
    return mlr_launched("attention_prefill_tcgen05");
}

}  // namespace

// Whether mlr_attention_prefill_tcgen05 takes this head size and page size.
MLR_API int mlr_attention_prefill_tcgen05_supports(int head_dim, int page_size) {
    return (head_dim == 64 || head_dim == 128) && page_size >= 8 && page_size <= 256 && (page_size & (page_size - 1)) == 0;
}

// q: [q_rows, ldq] bfloat16 with the query heads in the first q_heads * head_dim columns;
// out: [.., ldo]; cache: [num_pages][2][kv_heads][page_size][head_dim] bfloat16 with swizzled
// rows; tiles: n_tiles pairs {segment, first token of a 128-row tile of that segment};
// segment_info: per segment {first row, count, start position, _}.
MLR_API int mlr_attention_prefill_tcgen05(const void* q, int ldq, int q_rows, void* out, int ldo, const void* cache, int num_pages,
                                          const int* tiles, int n_tiles, const int* segment_info, const int* block_table,
                                          int table_stride, int page_size, int q_heads, int kv_heads, int head_dim, int window,
                                          float scale, int* status, cudaStream_t stream) {
    MLR_REQUIRE(mlr_attention_prefill_tcgen05_supports(head_dim, page_size),
                "attention_prefill_tcgen05: head size %d with pages of %d tokens is not supported (head size 64 or 128; "
                "a page size that is a power of two from 8 to 256)", head_dim, page_size);
    MLR_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0, "attention_prefill_tcgen05: %d query heads over %d kv heads",
                q_heads, kv_heads);
    MLR_REQUIRE(num_pages > 0 && window >= 0 && scale > 0.0f && q_rows > 0, "attention_prefill_tcgen05: bad sizes");
    MLR_REQUIRE(ldq % 8 == 0 && ldq >= q_heads * head_dim && ldo % 8 == 0 && ldo >= q_heads * head_dim,
                "attention_prefill_tcgen05: row strides must be multiples of 8 elements and hold all query heads");
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(q) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(cache) % 16 == 0,
                "attention_prefill_tcgen05: q, out and the cache must be 16-byte aligned");
    MLR_REQUIRE(n_tiles >= 0 && n_tiles <= 65535, "attention_prefill_tcgen05: %d tiles in one launch, the most is 65535", n_tiles);
    if (n_tiles == 0) return 0;
    EncodeTiled encode = encode_tiled();
    MLR_REQUIRE(encode != nullptr, "attention_prefill_tcgen05: the driver does not offer cuTensorMapEncodeTiled");
    CUtensorMap map_q, map_kv;
    {
        // Queries: boxes of 128 rows x 64 columns, written with the 128-byte swizzle; rows past
        // the end read as zero.
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(q_heads) * head_dim, static_cast<cuuint64_t>(q_rows)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldq) * 2};
        const cuuint32_t box[2] = {64, kRows};
        const cuuint32_t elem[2] = {1, 1};
        const CUresult r = encode(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(q), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        MLR_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tcgen05: cuTensorMapEncodeTiled (queries) failed with code %d", static_cast<int>(r));
    }
    {
        // The cache as [page block][token in page][head_dim]: boxes of one half (64 elements)
        // of up to 64 tokens of one block, copied as stored (the rows are swizzled already).
        const int box_rows = page_size < kKeys ? page_size : kKeys;
        const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(page_size),
                                    static_cast<cuuint64_t>(num_pages) * 2 * kv_heads};
        const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2, static_cast<cuuint64_t>(page_size) * head_dim * 2};
        const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
        const cuuint32_t elem[3] = {1, 1, 1};
        const CUresult r = encode(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        MLR_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tcgen05: cuTensorMapEncodeTiled (cache) failed with code %d", static_cast<int>(r));
    }
    if (head_dim == 64)
        return launch<64>(map_q, map_kv, out, ldo, num_pages, tiles, n_tiles, segment_info, block_table, table_stride, page_size,
                          q_heads, kv_heads, window, scale, status, stream);
    return launch<128>(map_q, map_kv, out, ldo, num_pages, tiles, n_tiles, segment_info, block_table, table_stride, page_size,
                       q_heads, kv_heads, window, scale, status, stream);
}
