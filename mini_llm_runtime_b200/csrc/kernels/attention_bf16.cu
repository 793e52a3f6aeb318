// bfloat16 attention over the paged cache on the tensor cores, for head sizes that are
// multiples of 16 up to 256.  Two kernels share one set of building blocks:
//
//   decode_splitkv   for requests that bring few rows (tokens x query heads per kv head
//                    <= 16: a decoded token, or a portion of two or three tokens).  One
//                    block per (request, kv head, split of the keys); its four compute warps
//                    walk disjoint keys of each 64-key tile with their own running softmax
//                    and are merged at the end; the block that finishes last merges the splits.  The bytes
//                    of the cache are what it is bound by.
//   prefill          for prompt portions.  One block per (64 query rows, query head); its
//                    four compute warps own 16 rows each and walk the keys up to the
//                    diagonal (flash attention: running maximum and sum, no score matrix).
//
// In both, a fifth warp streams K and V tiles of 64 keys through the block table into a ring
// of three shared-memory stages with bulk copies (cp.async.bulk) whose completion an
// mbarrier counts; the compute warps take fragments with ldmatrix and multiply with
// mma.sync m16n8k16 (bf16 in, float32 accumulate).  For head sizes 64, 128 and 256 the cache
// stores rows pre-swizzled (common.cuh), so a whole page block is one copy and lands
// bank-conflict-free; other head sizes copy row by row into padded tiles.  Scores, maxima,
// sums and the output accumulators are float32.  Keys outside a row's [lo, position] are
// masked in the scores and their V rows are zero or finite, so unused or stale cache memory
// cannot reach a result.  Every wait on a barrier is bounded.
//
// Semantics are those of src/minillm/runtime.cpp:283-310 (scores scaled by `scale`,
// softmax over t in [lo, position], weighted sum of V), with lo = 0 or
// position - window + 1.  The reference computes them with three SIMT kernels and a
// materialised score matrix (src/minillm/cuda/attention.cu:97-218).
#include "common.cuh"

#include <mutex>
#include "attention_no_alloc.h"

#include <type_traits>

namespace {

constexpr int kTileKeys = 64;
constexpr int kThreads = 128;
constexpr int kDecodeStages = 3;   // stages of a block's tile ring; 3 x 32 KB at head size 128: two blocks per SM
constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------- shared-memory tiles
// A tile is [64 keys][DMAX] bf16 with a row pitch of DMAX*2 bytes; the 16-byte chunk c of
// row r lives at chunk position c ^ (r & 7), which spreads the 8 rows of an ldmatrix over
// all banks.
template <int DMAX>
struct Tile {
    static constexpr int kPitch = DMAX * 2;
    static constexpr int kBytes = kTileKeys * kPitch;
    __device__ static __forceinline__ uint32_t offset(int row, int chunk) {
        return row * kPitch + ((chunk ^ (row & 7)) << 4);
    }
};

// The decode kernel's tiles are filled by bulk copies of whole key rows, which cannot
// permute chunks; there each row is padded by 16 bytes instead.  With a pitch of
// DMAX*2 + 16 bytes the 8 rows of an ldmatrix start 4 banks apart: no conflicts.
template <int DMAX>
struct PaddedTile {
    static constexpr int kPitch = DMAX * 2 + 16;
    static constexpr int kBytes = kTileKeys * kPitch;
    __device__ static __forceinline__ uint32_t offset(int row, int chunk) { return row * kPitch + (chunk << 4); }
};

// ---------------------------------------------------------------- mbarrier and bulk copies
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
// Waits for a phase of a barrier, but not for ever: after about two seconds it gives up and
// returns false (the caller then flags the fault and leaves).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > 4000000000LL) return false;
    }
    return true;
}
// One row of a tile: `bytes` (a multiple of 16) from global to shared memory, completion
// counted on `bar`.
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__host__ __device__ inline int log2_or_minus1(int v) {
    int s = 0;
    while ((1 << s) < v) ++s;
    return (1 << s) == v ? s : -1;
}

// One warp: S[16 rows x 16*NB keys] += Q[16 x D] K^T for keys [key0, key0 + 16*NB) of a tile.
// The 2*NB accumulators are independent chains; walking the head dimension in the outer
// loop keeps them all in flight.
template <int DMAX, int NB, typename Layout = Tile<DMAX>>
__device__ __forceinline__ void qk_keys(float (&s)[2 * NB][4], const uint32_t (&q)[DMAX / 16][4], uint32_t k_smem,
                                        int key0, int dim_steps) {
    const int lane = threadIdx.x & 31;
    const int row = key0 + ((lane >> 4) << 3) + (lane & 7);
    const int chunk_in_step = (lane >> 3) & 1;
#pragma unroll
    for (int kd = 0; kd < DMAX / 16; ++kd) {
        if (kd < dim_steps) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                uint32_t b[4];
                ldmatrix_x4(b, k_smem + Layout::offset(row + nb * 16, kd * 2 + chunk_in_step));
                mma_bf16(s[2 * nb], q[kd], b[0], b[1]);
                mma_bf16(s[2 * nb + 1], q[kd], b[2], b[3]);
            }
        }
    }
}

// One warp: O[16 rows x D] += P[16 x 16 keys] V for keys [key0, key0+16) of a tile.
template <int DMAX, typename Layout = Tile<DMAX>>
__device__ __forceinline__ void pv_16keys(float (&o)[DMAX / 8][4], const uint32_t (&p)[4], uint32_t v_smem,
                                          int key0, int dim_steps) {
    const int lane = threadIdx.x & 31;
    const int row = key0 + (((lane >> 3) & 1) << 3) + (lane & 7);
    const int chunk_in_pair = lane >> 4;
#pragma unroll
    for (int dn = 0; dn < DMAX / 16; ++dn) {
        if (dn < dim_steps) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_smem + Layout::offset(row, dn * 2 + chunk_in_pair));
            mma_bf16(o[dn * 2], p, b[0], b[1]);
            mma_bf16(o[dn * 2 + 1], p, b[2], b[3]);
        }
    }
}

// Q fragments of 16 rows from global memory.  row_ptr0 / row_ptr1 point at the head's D
// values of the thread's two rows (lane/4 and lane/4 + 8), or are null for absent rows.
template <int DMAX>
__device__ __forceinline__ void load_q(uint32_t (&q)[DMAX / 16][4], const __nv_bfloat16* row_ptr0,
                                       const __nv_bfloat16* row_ptr1, int dim_steps) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int kd = 0; kd < DMAX / 16; ++kd) {
        q[kd][0] = q[kd][1] = q[kd][2] = q[kd][3] = 0u;
        if (kd < dim_steps) {
            const int col = kd * 16 + 2 * t;
            if (row_ptr0) {
                q[kd][0] = *reinterpret_cast<const uint32_t*>(row_ptr0 + col);
                q[kd][2] = *reinterpret_cast<const uint32_t*>(row_ptr0 + col + 8);
            }
            if (row_ptr1) {
                q[kd][1] = *reinterpret_cast<const uint32_t*>(row_ptr1 + col);
                q[kd][3] = *reinterpret_cast<const uint32_t*>(row_ptr1 + col + 8);
            }
        }
    }
}

// Running softmax state of the two rows a thread owns.
struct RowState {
    float m[2] = {-INFINITY, -INFINITY};
    float l[2] = {0.0f, 0.0f};
};

// One step of the running softmax over `NT` n8-tiles of raw scores (keys key_base + 8*nt +
// 2*t + {0,1}): masks, updates the running maxima (kept in log2 units, i.e. multiplied by
// scale * log2 e), turns scores into probabilities exp2(s * scale_log2 - m), and packs them
// into A fragments (one per 16 keys).  The accumulators are rescaled only when some row of
// the warp saw a new maximum, which after the first tiles is rare.
template <int DMAX, int NT>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], RowState& st, float (&o)[DMAX / 8][4],
                                             uint32_t (&p)[NT / 2][4], int key_base, const int (&lo)[2],
                                             const int (&hi)[2], float scale_log2, bool need_mask) {
    const int t = threadIdx.x & 3;
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = j >> 1;
            if (need_mask) {
                const int key = key_base + nt * 8 + 2 * t + (j & 1);
                if (key < lo[r] || key > hi[r]) s[nt][j] = -INFINITY;
            }
            tile_max[r] = fmaxf(tile_max[r], s[nt][j]);
        }
    }
    float m_use[2], m_new[2];
    bool changed = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        m_new[r] = fmaxf(st.m[r], tile_max[r] * scale_log2);      // scale_log2 > 0
        changed |= m_new[r] > st.m[r];
        m_use[r] = m_new[r] == -INFINITY ? 0.0f : m_new[r];
    }
    if (__any_sync(0xffffffffu, changed)) {
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            alpha[r] = exp2f(st.m[r] - m_use[r]);      // 1 for a row whose maximum stayed, 0 for a row's first keys
            st.m[r] = m_new[r];
            st.l[r] *= alpha[r];
        }
#pragma unroll
        for (int dn = 0; dn < DMAX / 8; ++dn) {
            o[dn][0] *= alpha[0];
            o[dn][1] *= alpha[0];
            o[dn][2] *= alpha[1];
            o[dn][3] *= alpha[1];
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r = j >> 1;
            const float e = exp2f(fmaf(s[nt][j], scale_log2, -m_use[r]));
            s[nt][j] = e;
            st.l[r] += e;
        }
    }
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        p[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        p[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        p[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        p[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    }
}

// How the keys of a decode item are cut: splits of `chunk` keys from `base` (a multiple of 64).
struct SplitPlan {
    int base, first_key, last_key, splits;
};
__device__ __forceinline__ SplitPlan plan_splits(int start, int count, int window, int chunk) {
    SplitPlan p;
    p.last_key = start + count - 1;
    p.first_key = window > 0 ? max(0, start - window + 1) : 0;
    p.base = (p.first_key / kTileKeys) * kTileKeys;
    p.splits = (p.last_key + 1 - p.base + chunk - 1) / chunk;
    return p;
}

// ---------------------------------------------------------------- the copy warp
// Fills the stages of a block with the 64-key tiles of keys [key_begin, key_end) of one
// request and kv head, tile after tile, for the compute warps of the same block.  Per tile:
// wait until the stage is free, announce the tile's bytes on the stage's "full" barrier,
// issue the bulk copies.  BLOCKS (swizzled cache, head size == DMAX): one copy of K and one
// of V per page block the tile touches, byte for byte into an unpadded tile; rows of V
// outside [first_valid, key_end) are zeroed (their scores are masked, but 0 * garbage must
// stay 0).  Otherwise: one copy per key row into a padded tile; a key outside the range
// copies the nearest key inside it.  The block table and the keys below `fresh_from` must
// not be written by any kernel in flight: they are read before the wait for the preceding
// kernel (programmatic dependent launch).  Returns false if a wait ran out.
struct StageRing {
    uint32_t smem_base, bar_base;
    unsigned char* smem;
    int tile_bytes;
    __device__ __forceinline__ uint32_t k_stage(int s) const { return smem_base + s * 2 * tile_bytes; }
    __device__ __forceinline__ uint32_t v_stage(int s) const { return smem_base + s * 2 * tile_bytes + tile_bytes; }
    __device__ __forceinline__ uint32_t full_bar(int s) const { return bar_base + s * 8; }
    __device__ __forceinline__ uint32_t empty_bar(int s) const { return bar_base + (kDecodeStages + s) * 8; }
};

template <int DMAX, bool BLOCKS>
__device__ __forceinline__ bool copy_warp(const StageRing& ring, const __nv_bfloat16* __restrict__ cache, const int* __restrict__ table,
                                          int num_pages, int page_size, int kv_heads, int head_dim, int kv_head, int key_begin,
                                          int key_end, int first_valid, int tiles, int fresh_from, int* fault) {
    using L = typename std::conditional<BLOCKS, Tile<DMAX>, PaddedTile<DMAX>>::type;
    const int lane = threadIdx.x & 31;
    const int page_shift = log2_or_minus1(page_size);
    const size_t head_elems = static_cast<size_t>(page_size) * head_dim;
    const size_t value_shift = head_elems * kv_heads;
    const uint32_t row_bytes = head_dim * 2;
    bool ok = true;
    // Page of the block this lane copies in a tile (looked up one tile ahead, so that the
    // table read is off the critical path): block = first block of the tile + lane.
    auto tile_page = [&](int it_) {
        const int from_ = max(key_begin + it_ * kTileKeys, first_valid);
        const int block_ = (page_shift >= 0 ? from_ >> page_shift : from_ / page_size) + lane;
        const int last_ = min(key_begin + (it_ + 1) * kTileKeys, key_end) - 1;
        const int last_block_ = page_shift >= 0 ? last_ >> page_shift : last_ / page_size;
        return (it_ < tiles && block_ <= last_block_) ? __ldg(table + block_) : -1;
    };
    int ahead = BLOCKS ? tile_page(0) : -1;
    // Keys below `fresh_from` were written by earlier steps; the kernel before this one may
    // still be writing the others.  So the tiles of old keys are fetched at once, and the
    // wait for that kernel comes before the first tile that reaches a fresh key.
    bool waited = false;
    for (int it = 0; it < tiles && ok; ++it) {
        const int stage = it % kDecodeStages;
        if (it >= kDecodeStages) ok = mbar_wait(ring.empty_bar(stage), ((it / kDecodeStages) - 1) & 1);
        if (!ok) break;
        const int tile_start = key_begin + it * kTileKeys;
        if (!waited && min(tile_start + kTileKeys, key_end) > fresh_from) {
            mlr_grid_wait();
            waited = true;
        }
        const int my_page = ahead;
        if (BLOCKS) ahead = tile_page(it + 1);
        if (BLOCKS) {
            const int from = max(tile_start, first_valid), to = min(tile_start + kTileKeys, key_end);
            if (to - from < kTileKeys) {
                const int quads = (head_dim * 2) >> 4;
                for (int i = lane; i < kTileKeys * quads; i += 32) {
                    const int row = i / quads;
                    if (tile_start + row < from || tile_start + row >= to)
                        *reinterpret_cast<uint4*>(ring.smem + (ring.v_stage(stage) - ring.smem_base) + row * L::kPitch +
                                                  (i - row * quads) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                // These plain stores and the bulk copies of later tiles touch the same bytes.
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            __syncwarp();
            if (lane == 0) mbar_expect_tx(ring.full_bar(stage), row_bytes * 2 * (to - from));
            __syncwarp();
            const int first_block = page_shift >= 0 ? from >> page_shift : from / page_size;
            const int last_block = page_shift >= 0 ? (to - 1) >> page_shift : (to - 1) / page_size;
            for (int block = first_block + lane; block <= last_block; block += 32) {
                const int block_start = block * page_size;
                const int lo_key = max(block_start, from), hi_key = min(block_start + page_size, to);
                int page = block == first_block + lane ? my_page : __ldg(table + block);
                if (page < 0 || page >= num_pages) {
                    *fault = 1;
                    page = 0;
                }
                const __nv_bfloat16* src = cache + (static_cast<size_t>(page) * 2 * kv_heads + kv_head) * head_elems +
                                           static_cast<size_t>(lo_key - block_start) * head_dim;
                const uint32_t bytes = row_bytes * (hi_key - lo_key);
                const uint32_t dst = (lo_key - tile_start) * L::kPitch;
                bulk_copy(ring.k_stage(stage) + dst, src, bytes, ring.full_bar(stage));
                bulk_copy(ring.v_stage(stage) + dst, src + value_shift, bytes, ring.full_bar(stage));
            }
        } else {
            if (lane == 0) mbar_expect_tx(ring.full_bar(stage), row_bytes * 2 * kTileKeys);
            __syncwarp();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = lane + 32 * half;
                const int key = min(max(tile_start + row, first_valid), key_end - 1);
                const int block = page_shift >= 0 ? key >> page_shift : key / page_size;
                const int in_page = page_shift >= 0 ? key & (page_size - 1) : key - block * page_size;
                int page = __ldg(table + block);
                if (page < 0 || page >= num_pages) {
                    *fault = 1;
                    page = 0;      // still copy something so that the tile's byte count is met
                }
                const __nv_bfloat16* src = cache + (static_cast<size_t>(page) * 2 * kv_heads + kv_head) * head_elems +
                                           static_cast<size_t>(in_page) * head_dim;
                bulk_copy(ring.k_stage(stage) + row * L::kPitch, src, row_bytes, ring.full_bar(stage));
                bulk_copy(ring.v_stage(stage) + row * L::kPitch, src + value_shift, row_bytes, ring.full_bar(stage));
            }
        }
    }
    return ok;
}

// Barriers of a StageRing; called by one thread before the block's first __syncthreads().
__device__ __forceinline__ void init_ring(const StageRing& ring, int consumers) {
    for (int s = 0; s < kDecodeStages; ++s) {
        mbar_init(ring.full_bar(s), 1);
        mbar_init(ring.empty_bar(s), consumers);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}

// ---------------------------------------------------------------- the step's own tokens, made in place
// What the split-KV kernel needs to make the q, k and v rows of the step's own tokens itself, from the raw
// output of the q/k/v product: per-head RMS norm of q and k (weights may be absent), rotation by the table
// row of the token's position (the table may be absent), and the write of k and v into the cache.  The
// arithmetic is that of the row-wise kernel that otherwise runs before attention
// (elementwise.cu: qk_norm_rope_cache_kernel; src/minillm/runtime.cpp:262-281).
struct FreshRows {
    const void* q_weight;
    const void* k_weight;
    int weight_bf16;
    float eps;
    const float* cos_sin;       // [table_positions][head_dim]: cosines of a position's angles, then sines
    int table_positions;
    __nv_bfloat16* cache;       // the cache again, to write into
};

// A row to make, as one warp sees it: what does not depend on the kernel before this one (norm weight and
// rotation table entries of the lane's elements j = lane + 32 k and j + head_dim / 2) is fetched first, the raw
// values after the wait for that kernel, and several rows' loads are issued before any is used.
struct RowTask {
    bool valid, is_key;
    int index, token, position;
    const __nv_bfloat16* src;
    const void* weight;
    const float* cs;
    float wa[4], wb[4], c[4], sn[4], lo[4], hi[4];
    uint4 value;                    // a key's task also carries 16 bytes of the token's value row
};
__device__ __forceinline__ void task_constants(RowTask& t, int head_dim, int weight_bf16) {
    const int lane = threadIdx.x & 31, half = head_dim >> 1;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int j = lane + 32 * k;
        t.wa[k] = t.wb[k] = 1.0f;
        t.c[k] = 1.0f;
        t.sn[k] = 0.0f;
        if (t.valid && j < half) {
            if (t.weight) {
                t.wa[k] = weight_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(t.weight)[j]) : static_cast<const float*>(t.weight)[j];
                t.wb[k] = weight_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(t.weight)[j + half])
                                      : static_cast<const float*>(t.weight)[j + half];
            }
            if (t.cs) {
                t.c[k] = t.cs[j];
                t.sn[k] = t.cs[j + half];
            }
        }
    }
}
__device__ __forceinline__ void task_raw(RowTask& t, int head_dim, const __nv_bfloat16* value_src) {
    const int lane = threadIdx.x & 31, half = head_dim >> 1;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int j = lane + 32 * k;
        t.lo[k] = t.hi[k] = 0.0f;
        if (t.valid && j < half) {
            t.lo[k] = __bfloat162float(__ldcg(t.src + j));           // not through the read-only path: the kernel before this
            t.hi[k] = __bfloat162float(__ldcg(t.src + j + half));    // one wrote these after this kernel had started
        }
    }
    t.value = make_uint4(0u, 0u, 0u, 0u);
    if (t.valid && value_src && lane < (head_dim >> 3)) t.value = __ldcg(reinterpret_cast<const uint4*>(value_src) + lane);
}
// Norm (if the task has a weight), rotation (if it has table entries), rounding: to `dst` in shared memory in plain
// order and, for a key, into its cache row.  The arithmetic is that of qk_norm_rope_cache_kernel.
__device__ __forceinline__ void task_finish(const RowTask& t, int head_dim, float eps, __nv_bfloat16* dst, __nv_bfloat16* cache_row,
                                            bool swizzled) {
    const int lane = threadIdx.x & 31, half = head_dim >> 1;
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        sum = fmaf(t.lo[k], t.lo[k], sum);
        sum = fmaf(t.hi[k], t.hi[k], sum);
    }
    float scale = 1.0f;
    if (t.weight) {
        sum = mlr_warp_sum(sum);
        scale = 1.0f / sqrtf(sum / static_cast<float>(head_dim) + eps);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int j = lane + 32 * k;
        if (j < half) {
            float a = t.lo[k], b = t.hi[k];
            if (t.weight) {
                a = (a * scale) * t.wa[k];
                b = (b * scale) * t.wb[k];
            }
            if (t.cs) {
                const float ra = __fsub_rn(__fmul_rn(a, t.c[k]), __fmul_rn(b, t.sn[k]));
                const float rb = __fadd_rn(__fmul_rn(a, t.sn[k]), __fmul_rn(b, t.c[k]));
                a = ra;
                b = rb;
            }
            const __nv_bfloat16 va = __float2bfloat16_rn(a), vb = __float2bfloat16_rn(b);
            dst[j] = va;
            dst[j + half] = vb;
            if (cache_row) {
                cache_row[mlr_cache_col(j, t.position, swizzled)] = va;
                cache_row[mlr_cache_col(j + half, t.position, swizzled)] = vb;
            }
        }
    }
}

// ---------------------------------------------------------------- decode: split-KV
// grid = (max_splits, kv_heads, items), 160 threads: warps 0-3 compute, warp 4 copies.
// Row r of the block's 16 rows is token r / group, query head kv_head * group + r % group.
//
// The copy warp walks the split's 64-key tiles: for each it waits until the stage is free,
// announces the tile's bytes on the stage's "full" barrier and issues one bulk copy per key
// row of K and of V (two rows of each per lane; a key outside the split's range copies the
// nearest key inside, whose score is masked).  A compute warp waits for the stage, takes
// keys 16w .. 16w+15 of the tile with its own running softmax, and releases the stage.
// There is no block-wide barrier in the loop.  Every wait has a time limit; a wait that
// runs out sets MLR_STATUS_TIMEOUT and the block leaves without writing a result.
//
// Partial results go to `partial` [item][kv_head][split][16 rows][head_dim + 2] (the last
// two floats: maximum in log2 units and sum); an item whose keys fit one split is written
// to `out` directly.
constexpr int kDecodeThreads = 160;

// FRESH: `q` is the raw output of the q/k/v product (queries, keys, values in a row) and nothing of the
// step's own tokens is in the cache yet.  The block makes its 16 query rows itself (norm, rotation), and the
// block whose keys include a token of the step makes that token's key and value, writes them into the cache
// and puts them into its tile in place of what the copy brought.  The kernel before this one then is the
// product, not a row-wise kernel, and the copies of the keys of earlier steps need not wait for it.
template <int DMAX, bool BLOCKS, bool FRESH>
__global__ void __launch_bounds__(kDecodeThreads) decode_splitkv_kernel(
    const __nv_bfloat16* q, int ldq, __nv_bfloat16* __restrict__ out, int ldo,
    const __nv_bfloat16* cache, int num_pages, const int* __restrict__ items,
    const int* __restrict__ segment_info, const int* __restrict__ block_table, int table_stride,
    int page_size, int q_heads, int kv_heads, int head_dim, int window, float scale, int chunk,
    int max_splits, float* __restrict__ partial, int* __restrict__ counters, int* status, const FreshRows fresh) {
    mlr_grid_dependents_may_start();
    // `q` is NOT declared __restrict__: the kernel before this one writes it while this one may already run, and a
    // load the compiler knows to be of read-only memory may be moved above the wait for that kernel.
    // The segment table and the block table were uploaded before the step's first kernel;
    // what the preceding kernel writes (queries, the new keys and values) is read after
    // mlr_grid_wait() below.
    // BLOCKS: the cache rows are stored swizzled (head size 64, 128 or 256 = DMAX), so whole
    // page blocks are copied byte for byte into unpadded tiles.  Otherwise rows are stored
    // plainly and are copied one by one into padded tiles.
    using L = typename std::conditional<BLOCKS, Tile<DMAX>, PaddedTile<DMAX>>::type;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long barriers[2 * kDecodeStages];
    __shared__ int fault;      // 1: a page outside the pool, 2: a wait ran out
    const int item = blockIdx.z, kv_head = blockIdx.y, split = blockIdx.x;
    const int segment = items ? items[item] : item;
    const int first_row = segment_info[segment * 4 + 0], count = segment_info[segment * 4 + 1];
    const int start = segment_info[segment * 4 + 2];
    const SplitPlan plan = plan_splits(start, count, window, chunk);
    if (split >= plan.splits) return;
    const int group = q_heads / kv_heads;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int dim_steps = BLOCKS ? DMAX / 16 : head_dim >> 4;       // a constant when the head size is the template's

    const int key_begin = plan.base + split * chunk;
    const int key_end = min(key_begin + chunk, plan.last_key + 1);      // exclusive
    const int first_valid = max(key_begin, plan.first_key);
    const int tiles = (key_end - key_begin + kTileKeys - 1) / kTileKeys;

    const StageRing ring{smem_u32(smem), smem_u32(barriers), smem, L::kBytes};
    auto k_stage = [&](int s) { return ring.k_stage(s); };
    auto v_stage = [&](int s) { return ring.v_stage(s); };
    auto full_bar = [&](int s) { return ring.full_bar(s); };
    auto empty_bar = [&](int s) { return ring.empty_bar(s); };
    if (threadIdx.x == 0) {
        fault = 0;
        init_ring(ring, 4);
    }
    __syncthreads();

    float o[DMAX / 8][4];
#pragma unroll
    for (int dn = 0; dn < DMAX / 8; ++dn) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.0f;
    RowState st;

    if (warp == 4) {
        if (!copy_warp<DMAX, BLOCKS>(ring, cache, block_table + static_cast<size_t>(segment) * table_stride, num_pages,
                                     page_size, kv_heads, head_dim, kv_head, key_begin, key_end, first_valid, tiles, FRESH ? 0x7fffffff : start, &fault))
            fault = 2;
    } else {
        // ---------------- compute warps
        if (!FRESH) mlr_grid_wait();
        const int g = lane >> 2;
        int lo[2], hi[2];
        const __nv_bfloat16* qptr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = g + 8 * r;
            const int token = row / group, head = kv_head * group + row % group;
            const bool valid = token < count;
            hi[r] = valid ? start + token : -1;
            lo[r] = valid ? (window > 0 ? max(0, start + token - window + 1) : 0) : 0;
            qptr[r] = valid ? q + static_cast<size_t>(first_row + token) * ldq + static_cast<size_t>(head) * head_dim : nullptr;
        }
        // FRESH: behind the stages, [16][DMAX] made query rows, then the made keys and values of the step's tokens.
        __nv_bfloat16* made_q = reinterpret_cast<__nv_bfloat16*>(smem + static_cast<size_t>(kDecodeStages) * 2 * L::kBytes);
        __nv_bfloat16* made_k = made_q + 16 * DMAX;
        __nv_bfloat16* made_v = made_k + 16 * DMAX;
        if constexpr (FRESH) {
            const bool swizzled = mlr_cache_swizzled(true, head_dim);
            const size_t head_elems = static_cast<size_t>(page_size) * head_dim;
            // The rows to make: this block's query rows, then the tokens of the step among this block's keys (a key's
            // task copies the token's value too).  Warp w takes rows w, w + 4, ...; two at a time.
            const int query_rows = count * group;
            const int token_from = max(0, key_begin - start), token_to = min(count, key_end - start);
            const int total = query_rows + max(0, token_to - token_from);
            bool waited = false;
            for (int base = warp; base < total || !waited; base += 8) {
                RowTask task[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    RowTask& t = task[u];
                    const int id = base + 4 * u;
                    t.valid = id < total;
                    t.is_key = id >= query_rows;
                    t.token = t.is_key ? token_from + id - query_rows : id / group;
                    t.index = t.is_key ? t.token : id;
                    t.position = start + t.token;
                    const int head = t.is_key ? q_heads + kv_head : kv_head * group + id % group;
                    t.src = q + static_cast<size_t>(first_row + t.token) * ldq + static_cast<size_t>(head) * head_dim;
                    t.weight = t.is_key ? fresh.k_weight : fresh.q_weight;
                    t.cs = nullptr;
                    if (t.valid && fresh.cos_sin) {
                        if (t.position < 0 || t.position >= fresh.table_positions) {
                            if (lane == 0 && status) atomicOr(status, MLR_STATUS_BAD_INDEX);
                            t.valid = false;
                        } else {
                            t.cs = fresh.cos_sin + static_cast<size_t>(t.position) * head_dim;
                        }
                    }
                    task_constants(t, head_dim, fresh.weight_bf16);
                }
                if (!waited) {
                    mlr_grid_wait();        // what came so far had no writer in flight; the product's rows have
                    waited = true;
                }
#pragma unroll
                for (int u = 0; u < 2; ++u)
                    task_raw(task[u], head_dim, task[u].is_key ? task[u].src + static_cast<size_t>(kv_heads) * head_dim : nullptr);
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const RowTask& t = task[u];
                    if (!t.valid) continue;
                    __nv_bfloat16 *key_row = nullptr, *value_row = nullptr;
                    if (t.is_key) {
                        const int page = block_table[static_cast<size_t>(segment) * table_stride + t.position / page_size];
                        if (page < 0 || page >= num_pages) {
                            if (lane == 0) fault = 1;
                            continue;
                        }
                        key_row = fresh.cache + static_cast<size_t>(page) * 2 * kv_heads * head_elems + static_cast<size_t>(kv_head) * head_elems +
                                  static_cast<size_t>(t.position % page_size) * head_dim;
                        value_row = key_row + static_cast<size_t>(kv_heads) * head_elems;
                        if (lane < (head_dim >> 3)) {
                            *reinterpret_cast<uint4*>(made_v + t.index * DMAX + lane * 8) = t.value;
                            *reinterpret_cast<uint4*>(value_row + mlr_cache_col(lane * 8, t.position, swizzled)) = t.value;
                        }
                    }
                    task_finish(t, head_dim, fresh.eps, (t.is_key ? made_k : made_q) + t.index * DMAX, key_row, swizzled);
                }
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");        // the four compute warps: every made row is there
#pragma unroll
            for (int r = 0; r < 2; ++r)
                if (qptr[r]) qptr[r] = made_q + (g + 8 * r) * DMAX;
        }
        uint32_t qf[DMAX / 16][4];
        load_q<DMAX>(qf, qptr[0], qptr[1], dim_steps);
        const float scale_log2 = scale * kLog2e;
        const int last_lo = window > 0 ? max(0, start + count - window) : 0;
        bool ok = true;
        for (int it = 0; it < tiles; ++it) {
            const int stage = it % kDecodeStages;
            ok = __all_sync(0xffffffffu, mbar_wait(full_bar(stage), (it / kDecodeStages) & 1));     // the whole warp goes on, or none of it
            if (!ok) break;
            const int key_base = key_begin + it * kTileKeys + warp * 16;
            if constexpr (FRESH) {
                // The keys and values of the step's own tokens among this warp's 16 keys: from the made rows.
                const int from = max(start, key_base), to = min(min(start + count, key_base + 16), key_end);
                const int chunks = head_dim >> 3;
                for (int position = from; position < to; ++position) {
                    const int token = position - start, row = position - (key_begin + it * kTileKeys);
                    for (int c = lane; c < 2 * chunks; c += 32) {
                        const bool value = c >= chunks;
                        const int cc = value ? c - chunks : c;
                        const uint4 v = *reinterpret_cast<const uint4*>((value ? made_v : made_k) + token * DMAX + cc * 8);
                        *reinterpret_cast<uint4*>(ring.smem + ((value ? v_stage(stage) : k_stage(stage)) - ring.smem_base) + L::offset(row, cc)) = v;
                    }
                }
                if (!BLOCKS && (key_base < first_valid || key_base + 16 > key_end)) {
                    // Row by row copies fill a key outside the split's range with the nearest key inside it, which here
                    // may be one the cache does not hold yet: such value rows are zero instead (their scores are masked).
                    for (int c = lane; c < 16 * chunks; c += 32) {
                        const int r = c / chunks, position = key_base + r;
                        if (position < first_valid || position >= key_end)
                            *reinterpret_cast<uint4*>(ring.smem + (v_stage(stage) - ring.smem_base) + L::offset(warp * 16 + r, c - r * chunks)) =
                                make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                __syncwarp();
            }
            if (key_base < key_end) {
                float s[2][4] = {};
                qk_keys<DMAX, 1, L>(s, qf, k_stage(stage), warp * 16, dim_steps);
                uint32_t p[1][4];
                // No key of these 16 needs a mask if all are at or before the first token's
                // position and at or after the last token's window start.
                const bool need_mask = key_base + 15 > start || key_base < last_lo;
                softmax_step<DMAX, 2>(s, st, o, p, key_base, lo, hi, scale_log2, need_mask);
                pv_16keys<DMAX, L>(o, p[0], v_stage(stage), warp * 16, dim_steps);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(stage));
        }
        if (!ok) fault = 2;
    }
    __syncthreads();
    if (fault) {
        if (threadIdx.x == 0 && status) atomicOr(status, fault == 2 ? MLR_STATUS_TIMEOUT : MLR_STATUS_BAD_PAGE);
        if (fault == 2) {
            // Give copies that may still be in flight time to land before the block's shared
            // memory is handed to another block.
            for (int i = 0; i < 100; ++i) __nanosleep(1000);
            // Still count this block, so that the counter goes back to zero.
            if (threadIdx.x == 0 && plan.splits > 1) {
                int* counter = counters + item * kv_heads + kv_head;
                if (atomicAdd(counter, 1) == plan.splits - 1) *counter = 0;
            }
            return;
        }
    }

    // Merge the four compute warps through shared memory (the tile stages are free now).
    const int g = lane >> 2, t = lane & 3;
    float* merge_o = reinterpret_cast<float*>(smem);                       // [4][16][DMAX]
    float* merge_ml = merge_o + 4 * 16 * DMAX;                             // [4][16][2]
    if (warp < 4) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
        }
#pragma unroll
        for (int dn = 0; dn < DMAX / 8; ++dn) {
            if (dn * 8 < head_dim) {
                float* row0 = merge_o + (warp * 16 + g) * DMAX + dn * 8 + 2 * t;
                float* row1 = merge_o + (warp * 16 + g + 8) * DMAX + dn * 8 + 2 * t;
                row0[0] = o[dn][0];
                row0[1] = o[dn][1];
                row1[0] = o[dn][2];
                row1[1] = o[dn][3];
            }
        }
        if (t == 0) {
            merge_ml[(warp * 16 + g) * 2 + 0] = st.m[0];
            merge_ml[(warp * 16 + g) * 2 + 1] = st.l[0];
            merge_ml[(warp * 16 + g + 8) * 2 + 0] = st.m[1];
            merge_ml[(warp * 16 + g + 8) * 2 + 1] = st.l[1];
        }
    }
    __syncthreads();
    const int rows = count * group;
    const bool direct = plan.splits == 1;
    // Scratch: for every (request, kv head, split) 16 rows of head_dim sums, and after all of
    // those 16 (maximum, sum of weights) pairs each.
    const size_t unit = (static_cast<size_t>(item) * kv_heads + kv_head) * max_splits;
    float* part = partial + (unit + split) * 16 * head_dim;
    float* part_ml = partial + static_cast<size_t>(gridDim.z) * kv_heads * max_splits * 16 * head_dim + (unit + split) * 32;
    for (int idx = threadIdx.x; idx < rows * head_dim; idx += kDecodeThreads) {
        const int row = idx / head_dim, d = idx - row * head_dim;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, merge_ml[(w * 16 + row) * 2]);
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = merge_ml[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - m);
            l += merge_ml[(w * 16 + row) * 2 + 1] * f;
            acc += merge_o[(w * 16 + row) * DMAX + d] * f;
        }
        if (direct) {
            const int token = row / group, head = kv_head * group + row % group;
            out[static_cast<size_t>(first_row + token) * ldo + static_cast<size_t>(head) * head_dim + d] =
                __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
        } else {
            part[row * head_dim + d] = acc;
            if (d == 0) {
                part_ml[row * 2] = m;
                part_ml[row * 2 + 1] = l;
            }
        }
    }
    if (direct) return;

    // The block that finishes last among the splits of this (request, kv head) adds them up,
    // in split order, so the sum does not depend on which block that is.  The counter is left
    // at zero for the next launch.
    __shared__ int is_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        // One fence after the block's barrier orders every thread's partial results before
        // the count (fences are cumulative), as a grid-wide barrier does it.
        __threadfence();
        int* counter = counters + item * kv_heads + kv_head;
        is_last = atomicAdd(counter, 1) == plan.splits - 1;
        if (is_last) {
            *counter = 0;
            __threadfence();       // the other blocks' partial results, for every thread after the barrier
        }
    }
    __syncthreads();
    if (!is_last) return;
    // The weights exp2(m_split - m) / l are worked out once per (split, row) in shared memory
    // from maxima and sums that all threads fetch together; the sums over splits then have
    // no dependent loads and are fetched four values and eight splits at a time.  Other SMs
    // wrote the partial results: they are read from L2, past this SM's L1.
    float* factor = merge_ml + 4 * 16 * 2;      // [splits][16]: maxima, then weights
    float* weight_sum = factor + 16 * max_splits;
    const float* base = partial + unit * 16 * head_dim;
    const float* base_ml = part_ml - split * 32;
    for (int i = threadIdx.x; i < plan.splits * 16; i += kDecodeThreads) {
        const float2 ml = (i & 15) < rows ? __ldcg(reinterpret_cast<const float2*>(base_ml) + i) : make_float2(-INFINITY, 0.0f);
        factor[i] = ml.x;
        weight_sum[i] = ml.y;
    }
    __syncthreads();
    if (threadIdx.x < rows) {
        const int row = threadIdx.x;
        float m = -INFINITY;
        for (int s = 0; s < plan.splits; ++s) m = fmaxf(m, factor[s * 16 + row]);
        float l = 0.0f;
        for (int s = 0; s < plan.splits; ++s) {
            const float ms = factor[s * 16 + row];
            const float f = ms == -INFINITY ? 0.0f : exp2f(ms - m);
            l += weight_sum[s * 16 + row] * f;
            factor[s * 16 + row] = f;
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        for (int s = 0; s < plan.splits; ++s) factor[s * 16 + row] *= inv;
    }
    __syncthreads();
    const int quads = head_dim >> 2;        // head_dim is a multiple of 16
    for (int idx = threadIdx.x; idx < rows * quads; idx += kDecodeThreads) {
        const int row = idx / quads, d = (idx - row * quads) * 4;
        const float4* src = reinterpret_cast<const float4*>(base + row * head_dim + d);
        const int split_stride = 4 * head_dim;      // float4 units between splits: 16 rows of head_dim floats
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        int s = 0;
        for (; s + 8 <= plan.splits; s += 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(src + (s + u) * split_stride);
#pragma unroll
            for (int u = 0; u < 8; ++u) {       // in split order, whatever the batch size
                const float f = factor[(s + u) * 16 + row];
                acc.x = fmaf(v[u].x, f, acc.x);
                acc.y = fmaf(v[u].y, f, acc.y);
                acc.z = fmaf(v[u].z, f, acc.z);
                acc.w = fmaf(v[u].w, f, acc.w);
            }
        }
        for (; s < plan.splits; ++s) {
            const float4 v = __ldcg(src + s * split_stride);
            const float f = factor[s * 16 + row];
            acc.x = fmaf(v.x, f, acc.x);
            acc.y = fmaf(v.y, f, acc.y);
            acc.z = fmaf(v.z, f, acc.z);
            acc.w = fmaf(v.w, f, acc.w);
        }
        const int token = row / group, head = kv_head * group + row % group;
        __nv_bfloat16* dst = out + static_cast<size_t>(first_row + token) * ldo + static_cast<size_t>(head) * head_dim + d;
        reinterpret_cast<uint32_t*>(dst)[0] = pack_bf16(acc.x, acc.y);      // row strides are even, not more
        reinterpret_cast<uint32_t*>(dst)[1] = pack_bf16(acc.z, acc.w);
    }
}

// ---------------------------------------------------------------- prefill: flash attention
// grid = (q_heads, tiles), 160 threads.  tiles[i] = {segment, first token of the 64-row tile
// within the segment}.  Warp 4 copies the key tiles (copy_warp); compute warp w owns rows
// 16w .. 16w+15 of the query tile and walks the keys up to the diagonal with a running
// softmax.  No block-wide barrier in the loop; waits are bounded.
// Registers: an SM's register file is split over four schedulers of 16384 registers each, and
// a block's five warps spread over them, so two blocks per SM need three warps to fit one
// scheduler: at most 168 registers per thread (5376 per warp).  Above that only one block
// runs per SM and the kernel loses about a third of its speed.
template <int DMAX, bool BLOCKS>
__global__ void __launch_bounds__(kDecodeThreads) __maxnreg__(DMAX <= 128 ? 168 : 255) prefill_kernel(
    const __nv_bfloat16* q, int ldq, __nv_bfloat16* __restrict__ out, int ldo,
    const __nv_bfloat16* __restrict__ cache, int num_pages, const int* __restrict__ tiles,
    const int* __restrict__ segment_info, const int* __restrict__ block_table, int table_stride,
    int page_size, int q_heads, int kv_heads, int head_dim, int window, float scale, int* status) {
    mlr_grid_dependents_may_start();
    using L = typename std::conditional<BLOCKS, Tile<DMAX>, PaddedTile<DMAX>>::type;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long barriers[2 * kDecodeStages];
    __shared__ int fault;
    // Blocks start in the order of their index, x fastest: all heads of the first tile (the one
    // with the longest walk over the keys, as the caller sorts them), then all heads of the next.
    const int head = blockIdx.x;
    const int segment = tiles[blockIdx.y * 2], tile_token = tiles[blockIdx.y * 2 + 1];
    const int first_row = segment_info[segment * 4 + 0], count = segment_info[segment * 4 + 1];
    const int start = segment_info[segment * 4 + 2];
    const int kv_head = head / (q_heads / kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int dim_steps = BLOCKS ? DMAX / 16 : head_dim >> 4;

    const int tile_rows = min(kTileKeys, count - tile_token);
    const int first_pos = start + tile_token, last_pos = first_pos + tile_rows - 1;
    const int first_key = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int key_begin = (first_key / kTileKeys) * kTileKeys;
    const int n_tiles = (last_pos + 1 - key_begin + kTileKeys - 1) / kTileKeys;

    const StageRing ring{smem_u32(smem), smem_u32(barriers), smem, L::kBytes};
    if (threadIdx.x == 0) {
        fault = 0;
        init_ring(ring, 4);
    }
    __syncthreads();

    if (warp == 4) {
        if (!copy_warp<DMAX, BLOCKS>(ring, cache, block_table + static_cast<size_t>(segment) * table_stride, num_pages,
                                     page_size, kv_heads, head_dim, kv_head, key_begin, last_pos + 1, max(first_key, key_begin),
                                     n_tiles, start, &fault))
            fault = 2;
    } else {
        mlr_grid_wait();
        const int g = lane >> 2, t = lane & 3;
        int lo[2], hi[2];
        const __nv_bfloat16* qptr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = warp * 16 + g + 8 * r;
            const bool valid = row < tile_rows;
            hi[r] = valid ? first_pos + row : -1;
            lo[r] = valid ? (window > 0 ? max(0, first_pos + row - window + 1) : 0) : 0;
            qptr[r] = valid ? q + static_cast<size_t>(first_row + tile_token + row) * ldq + static_cast<size_t>(head) * head_dim
                            : nullptr;
        }
        uint32_t qf[DMAX / 16][4];
        load_q<DMAX>(qf, qptr[0], qptr[1], dim_steps);
        float o[DMAX / 8][4];
#pragma unroll
        for (int dn = 0; dn < DMAX / 8; ++dn) o[dn][0] = o[dn][1] = o[dn][2] = o[dn][3] = 0.0f;
        RowState st;
        const float scale_log2 = scale * kLog2e;
        // Rows of this warp: their lowest lower bound and highest position decide which key
        // tiles the warp can skip and which need no mask at all.
        const int warp_first = first_pos + warp * 16, warp_last = min(last_pos, warp_first + 15);
        const int warp_lo_min = window > 0 ? max(0, warp_first - window + 1) : 0;
        const int warp_lo_max = window > 0 ? max(0, warp_last - window + 1) : 0;
        const bool warp_active = warp * 16 < tile_rows;
        bool ok = true;
        for (int it = 0; it < n_tiles; ++it) {
            const int stage = it % kDecodeStages;
            ok = __all_sync(0xffffffffu, mbar_wait(ring.full_bar(stage), (it / kDecodeStages) & 1));
            if (!ok) break;
            const int key0 = key_begin + it * kTileKeys;
            if (warp_active && key0 <= warp_last && key0 + kTileKeys - 1 >= warp_lo_min) {
                float s[8][4] = {};
                qk_keys<DMAX, 4, L>(s, qf, ring.k_stage(stage), 0, dim_steps);
                // Rows 16w.. are all at or after warp_first; a tile wholly before it and wholly
                // inside every row's window needs no mask (rows past the tile's end are not stored).
                const bool need_mask = key0 + kTileKeys - 1 > warp_first || key0 < warp_lo_max;
                uint32_t p[4][4];
                softmax_step<DMAX, 8>(s, st, o, p, key0, lo, hi, scale_log2, need_mask);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) pv_16keys<DMAX, L>(o, p[kk], ring.v_stage(stage), kk * 16, dim_steps);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(ring.empty_bar(stage));
        }
        if (!ok) fault = 2;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
            st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
        }
        if (ok) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = warp * 16 + g + 8 * r;
                if (row >= tile_rows) continue;
                const float inv = st.l[r] > 0.0f ? 1.0f / st.l[r] : 0.0f;
                __nv_bfloat16* dst = out + static_cast<size_t>(first_row + tile_token + row) * ldo + static_cast<size_t>(head) * head_dim;
#pragma unroll
                for (int dn = 0; dn < DMAX / 8; ++dn) {
                    if (dn * 8 < head_dim)
                        *reinterpret_cast<uint32_t*>(dst + dn * 8 + 2 * t) = pack_bf16(o[dn][2 * r] * inv, o[dn][2 * r + 1] * inv);
                }
            }
        }
    }
    __syncthreads();
    if (fault && threadIdx.x == 0) {
        if (status) atomicOr(status, fault == 2 ? MLR_STATUS_TIMEOUT : MLR_STATUS_BAD_PAGE);
        if (fault == 2)
            for (int i = 0; i < 100; ++i) __nanosleep(1000);   // let copies in flight land before the block ends
    }
}

// Raises a kernel's dynamic shared memory limit; remembered per kernel and device so that
// the attribute call is made once, not at every launch.
template <typename Kernel>
int allow_smem(Kernel kernel, size_t bytes, const char* what) {
    struct Entry {
        const void* kernel;
        int device;
        size_t bytes;
    };
    static thread_local Entry seen[64];
    static thread_local int count = 0;
    int device = 0;
    cudaGetDevice(&device);
    const void* key = reinterpret_cast<const void*>(kernel);
    for (int i = 0; i < count; ++i)
        if (seen[i].kernel == key && seen[i].device == device && seen[i].bytes >= bytes) return 0;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e != cudaSuccess) return mlr_fail("%s: cannot use %zu bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
    if (count < 64) seen[count++] = Entry{key, device, bytes};
    return 0;
}

int check_common(const char* what, int q_heads, int kv_heads, int head_dim, int page_size, int num_pages, int window,
                 int ldq, int ldo, float scale) {
    MLR_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0, "%s: %d query heads cannot share %d kv heads", what, q_heads, kv_heads);
    MLR_REQUIRE(head_dim >= 16 && head_dim <= 256 && head_dim % 16 == 0,
                "%s: head size %d is not a multiple of 16 in [16, 256]", what, head_dim);
    MLR_REQUIRE(page_size > 0 && num_pages > 0 && window >= 0, "%s: bad page size, page count or window", what);
    MLR_REQUIRE(scale > 0.0f, "%s: the score scale must be positive, got %g", what, static_cast<double>(scale));
    MLR_REQUIRE(ldq >= q_heads * head_dim && ldo >= q_heads * head_dim && ldq % 2 == 0 && ldo % 2 == 0,
                "%s: a row stride is smaller than the row or odd", what);
    MLR_REQUIRE(kv_heads <= 65535 && q_heads <= 65535, "%s: more than 65535 heads", what);
    return 0;
}

}  // namespace

// Floats of scratch the decode kernel needs for `items` requests cut into `max_splits`.
MLR_API long long mlr_attention_decode_scratch_floats(int items, int kv_heads, int head_dim, int max_splits) {
    return static_cast<long long>(items) * kv_heads * max_splits * 16 * (head_dim + 2);
}

// items: segment indices (null = segments 0..n_items-1).  Every item must have
// count * (q_heads / kv_heads) <= 16 rows.  chunk: keys per split, a multiple of 64.
// max_splits: the most splits any item needs (the grid's x extent).  partial: scratch of
// mlr_attention_decode_scratch_floats floats, and counters: n_items * kv_heads ints that are
// zero on entry and are left zero (both may be null when max_splits == 1).
namespace {
int launch_decode(const char* what, const void* q, int ldq, void* out, int ldo, const void* cache, int num_pages, const int* items,
                  int n_items, const int* segment_info, const int* block_table, int table_stride, int page_size, int q_heads,
                  int kv_heads, int head_dim, int window, float scale, int chunk, int max_splits, float* partial, int* counters,
                  int* status, const FreshRows* fresh, cudaStream_t stream) {
    if (int e = check_common(what, q_heads, kv_heads, head_dim, page_size, num_pages, window, ldq, ldo, scale)) return e;
    MLR_REQUIRE(q_heads / kv_heads <= 16, "%s: %d query heads per kv head exceed the 16 rows of a block", what, q_heads / kv_heads);
    MLR_REQUIRE(chunk > 0 && chunk % kTileKeys == 0, "%s: chunk %d is not a positive multiple of %d", what, chunk, kTileKeys);
    MLR_REQUIRE(max_splits >= 1 && max_splits <= 512 && (max_splits == 1 || (partial && counters)),
                "%s: the split count must be in [1, 512], with scratch and counters when above 1", what);
    MLR_REQUIRE(reinterpret_cast<uintptr_t>(partial) % 16 == 0, "%s: the scratch must be 16-byte aligned", what);
    MLR_REQUIRE(n_items >= 0 && n_items <= 65535, "%s: more than 65535 requests in one launch", what);
    if (n_items == 0) return 0;
    const dim3 grid(max_splits, kv_heads, n_items);
    const FreshRows none = {};
#define MLR_LAUNCH_AS(DMAX, BLOCKS, FRESH)                                                                              \
    do {                                                                                                                \
        const size_t merge = sizeof(float) * (4 * 16 * DMAX + 4 * 16 * 2 + 32 * max_splits);                            \
        const size_t tile = BLOCKS ? Tile<DMAX>::kBytes : PaddedTile<DMAX>::kBytes;                                     \
        const size_t stages = static_cast<size_t>(kDecodeStages) * 2 * tile + (FRESH ? 3 * 16 * DMAX * 2 : 0);          \
        const size_t bytes = stages > merge ? stages : merge;                                                           \
        if (int e = allow_smem(decode_splitkv_kernel<DMAX, BLOCKS, FRESH>, bytes, what)) return e;                      \
        mlr_launch((decode_splitkv_kernel<DMAX, BLOCKS, FRESH>), dim3(grid), dim3(kDecodeThreads), bytes, stream,       \
            static_cast<const __nv_bfloat16*>(q), ldq, static_cast<__nv_bfloat16*>(out), ldo,                           \
            static_cast<const __nv_bfloat16*>(cache), num_pages, items, segment_info, block_table, table_stride,        \
            page_size, q_heads, kv_heads, head_dim, window, scale, chunk, max_splits, partial, counters, status,        \
            FRESH ? *fresh : none);                                                                                     \
    } while (0)
#define MLR_LAUNCH(DMAX, BLOCKS)                    \
    do {                                            \
        if (fresh) MLR_LAUNCH_AS(DMAX, BLOCKS, true); \
        else MLR_LAUNCH_AS(DMAX, BLOCKS, false);    \
    } while (0)
    if (head_dim == 64) MLR_LAUNCH(64, true);
    else if (head_dim == 128) MLR_LAUNCH(128, true);
    else if (head_dim == 256) MLR_LAUNCH(256, true);
    else if (head_dim < 64) MLR_LAUNCH(64, false);
    else if (head_dim < 128) MLR_LAUNCH(128, false);
    else MLR_LAUNCH(256, false);
#undef MLR_LAUNCH
#undef MLR_LAUNCH_AS
    return mlr_launched(what);
}
}  // namespace

MLR_API int mlr_attention_decode_bf16(const void* q, int ldq, void* out, int ldo, const void* cache, int num_pages,
                                      const int* items, int n_items, const int* segment_info,
                                      const int* block_table, int table_stride, int page_size, int q_heads,
                                      int kv_heads, int head_dim, int window, float scale, int chunk,
                                      int max_splits, float* partial, int* counters, int* status, cudaStream_t stream) {
    return launch_decode("attention_decode_bf16", q, ldq, out, ldo, cache, num_pages, items, n_items, segment_info, block_table,
                         table_stride, page_size, q_heads, kv_heads, head_dim, window, scale, chunk, max_splits, partial, counters,
                         status, nullptr, stream);
}

// The same over the RAW output of the q/k/v product: `qkv` rows hold q_heads query heads, then kv_heads key
// heads, then kv_heads value heads, none of them normed or rotated, and the cache does not hold the step's own
// tokens yet.  The kernel norms q and k per head (`q_weight`, `k_weight`: bfloat16 or float32 as `weight_bf16`
// says, both null for no norm; `eps`), rotates them by row `position` of `cos_sin` [table_positions][head_dim]
// (null: no rotation), writes k and v into `cache` and attends.  It replaces the row-wise kernel that otherwise
// runs before attention when every segment of the step is one of `items`.
MLR_API int mlr_attention_decode_fresh_bf16(const void* qkv, int ld, void* out, int ldo, void* cache, int num_pages, const int* items,
                                            int n_items, const int* segment_info, const int* block_table, int table_stride,
                                            int page_size, int q_heads, int kv_heads, int head_dim, int window, float scale,
                                            int chunk, int max_splits, float* partial, int* counters, const void* q_weight,
                                            const void* k_weight, int weight_bf16, float eps, const float* cos_sin,
                                            int table_positions, int* status, cudaStream_t stream) {
    MLR_REQUIRE((q_weight == nullptr) == (k_weight == nullptr), "attention_decode_fresh_bf16: q and k norm weights must both be given or both be absent");
    MLR_REQUIRE(ld >= (q_heads + 2 * kv_heads) * head_dim, "attention_decode_fresh_bf16: row stride %d is smaller than the q/k/v width", ld);
    MLR_REQUIRE(cos_sin == nullptr || table_positions > 0, "attention_decode_fresh_bf16: a rotation table without rows");
    const FreshRows fresh = {q_weight, k_weight, weight_bf16, eps, cos_sin, table_positions, static_cast<__nv_bfloat16*>(cache)};
    return launch_decode("attention_decode_fresh_bf16", qkv, ld, out, ldo, cache, num_pages, items, n_items, segment_info, block_table,
                         table_stride, page_size, q_heads, kv_heads, head_dim, window, scale, chunk, max_splits, partial, counters,
                         status, &fresh, stream);
}

// ---------------------------------------------------------------- the entry point that allocates nothing
// Scratch for mlr_attention_decode_bf16_no_alloc (see attention_no_alloc.h).  In host code
// this name is only a handle for the runtime: the device address comes from
// cudaGetSymbolAddress.
static __device__ __align__(256) float mlr_static_scratch[MLR_ATTENTION_STATIC_SCRATCH_FLOATS];
// One counter per (request, kv head) of a call: zero when the library is loaded, and every
// call leaves them zero again.
static __device__ __align__(256) int mlr_static_counters[MLR_ATTENTION_STATIC_COUNTERS];

MLR_API int mlr_attention_decode_bf16_no_alloc(const void* q, int ldq, void* out, int ldo, const void* cache,
                                               int num_pages, const int* items, int n_items,
                                               const int* segment_info, const int* block_table, int table_stride,
                                               int page_size, int q_heads, int kv_heads, int head_dim, int window,
                                               float scale, int chunk, int max_splits, int* status,
                                               cudaStream_t stream) {
    MLR_REQUIRE(n_items >= 0 && kv_heads > 0 && head_dim > 0 && max_splits >= 1,
                "attention_decode_bf16_no_alloc: bad sizes items=%d kv_heads=%d head_dim=%d splits=%d", n_items, kv_heads,
                head_dim, max_splits);
    const long long need = mlr_attention_decode_scratch_floats(n_items, kv_heads, head_dim, max_splits);
    MLR_REQUIRE(need <= MLR_ATTENTION_STATIC_SCRATCH_FLOATS,
                "attention_decode_bf16_no_alloc: the call needs %lld floats of scratch, the built-in array holds %d; "
                "use fewer requests per call, fewer splits, or mlr_attention_decode_bf16 with a buffer of your own",
                need, MLR_ATTENTION_STATIC_SCRATCH_FLOATS);
    MLR_REQUIRE(static_cast<long long>(n_items) * kv_heads <= MLR_ATTENTION_STATIC_COUNTERS,
                "attention_decode_bf16_no_alloc: %d requests x %d kv heads exceed the %d built-in counters", n_items, kv_heads,
                MLR_ATTENTION_STATIC_COUNTERS);
    // Device addresses of the arrays, looked up once per device with that device current.  Both
    // addresses of a device are published together under a lock, so a second host thread never
    // sees one without the other.
    constexpr int kMaxDevices = 64;
    struct Addresses {
        float* scratch;
        int* counters;
    };
    static Addresses table[kMaxDevices] = {};
    static std::mutex table_lock;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return mlr_fail("attention_decode_bf16_no_alloc: cudaGetDevice: %s", cudaGetErrorString(e));
    MLR_REQUIRE(device >= 0 && device < kMaxDevices, "attention_decode_bf16_no_alloc: device index %d is not below %d", device, kMaxDevices);
    Addresses found;
    {
        std::lock_guard<std::mutex> guard(table_lock);
        if (table[device].scratch == nullptr) {
            void* scratch = nullptr;
            e = cudaGetSymbolAddress(&scratch, mlr_static_scratch);
            if (e != cudaSuccess || scratch == nullptr)
                return mlr_fail("attention_decode_bf16_no_alloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            void* counters = nullptr;
            e = cudaGetSymbolAddress(&counters, mlr_static_counters);
            if (e != cudaSuccess || counters == nullptr)
                return mlr_fail("attention_decode_bf16_no_alloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            table[device] = Addresses{static_cast<float*>(scratch), static_cast<int*>(counters)};
        }
        found = table[device];
    }
    return mlr_attention_decode_bf16(q, ldq, out, ldo, cache, num_pages, items, n_items, segment_info, block_table,
                                     table_stride, page_size, q_heads, kv_heads, head_dim, window, scale, chunk,
                                     max_splits, found.scratch, found.counters, status, stream);
}

// tiles: n_tiles pairs {segment, first token of a 64-row tile of that segment}.
MLR_API int mlr_attention_prefill_bf16(const void* q, int ldq, void* out, int ldo, const void* cache, int num_pages,
                                       const int* tiles, int n_tiles, const int* segment_info,
                                       const int* block_table, int table_stride, int page_size, int q_heads,
                                       int kv_heads, int head_dim, int window, float scale, int* status,
                                       cudaStream_t stream) {
    if (int e = check_common("attention_prefill_bf16", q_heads, kv_heads, head_dim, page_size, num_pages, window, ldq, ldo, scale)) return e;
    MLR_REQUIRE(n_tiles >= 0, "attention_prefill_bf16: negative tile count");
    if (n_tiles == 0) return 0;
    MLR_REQUIRE(n_tiles <= 65535, "attention_prefill_bf16: %d tiles in one launch, the most is 65535", n_tiles);
    const dim3 grid(q_heads, n_tiles);
#define MLR_LAUNCH(DMAX, BLOCKS)                                                                                   \
    do {                                                                                                           \
        const size_t tile = BLOCKS ? Tile<DMAX>::kBytes : PaddedTile<DMAX>::kBytes;                                \
        const size_t bytes = static_cast<size_t>(kDecodeStages) * 2 * tile;                                        \
        if (int e = allow_smem(prefill_kernel<DMAX, BLOCKS>, bytes, "attention_prefill_bf16")) return e;          \
        mlr_launch((prefill_kernel<DMAX, BLOCKS>), dim3(grid), dim3(kDecodeThreads), bytes, stream,               \
                   static_cast<const __nv_bfloat16*>(q), ldq, static_cast<__nv_bfloat16*>(out), ldo,               \
                   static_cast<const __nv_bfloat16*>(cache), num_pages, tiles, segment_info, block_table,          \
                   table_stride, page_size, q_heads, kv_heads, head_dim, window, scale, status);                   \
    } while (0)
    if (head_dim == 64) MLR_LAUNCH(64, true);
    else if (head_dim == 128) MLR_LAUNCH(128, true);
    else if (head_dim == 256) MLR_LAUNCH(256, true);
    else if (head_dim < 64) MLR_LAUNCH(64, false);
    else if (head_dim < 128) MLR_LAUNCH(128, false);
    else MLR_LAUNCH(256, false);
#undef MLR_LAUNCH
    return mlr_launched("attention_prefill_bf16");
}
