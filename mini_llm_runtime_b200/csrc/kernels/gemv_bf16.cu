// Products of a decode step's few rows (one to eight): out[M, N] = f(x[M, K] W[N, K]^T), alone or
// several in a CHAIN that one persistent grid runs without a launch boundary in between.
//
// With so few rows a product is a pass over the weight matrix and nothing else, so the kernel is
// built around the memory system.  A group of four warps takes 16 rows of W at a time and cuts K among
// its warps; every lane reads 16 contiguous bytes of two weight rows per load, straight from global
// memory into the registers that are the A operand of `mma.sync.m16n8k16` (the order of the k
// values inside an instruction is permuted the same way for W and for x, which a sum does not
// notice), several loads in flight per lane, no staging of weights in shared memory.  The B operand
// is the step's activations, which the block keeps in shared memory as bfloat16 (at most 8 rows;
// rows beyond M are zero registers).  The tensor cores do the multiply-adds of all rows at once, so
// eight rows cost what one costs; the sums over the warps' K ranges are added in shared memory
// in a fixed order, so a result depends neither on the grid nor on timing.  (`mma.sync` is the
// older tensor-core instruction; `tcgen05.mma` wants both operands in shared memory, which is
// exactly the copy this kernel avoids.  The products of prompt portions use tcgen05.)
//
// Folded in, so that they are no launches of their own:
//  * prologue: the RMS norm of the rows of the float32 residual stream that feed the product
//    (`(h * 1/sqrt(mean(h^2) + eps)) * w`, rounded to bfloat16 as the norm kernel rounds it), on
//    all rows or on the rows an index names (the final norm before the output head);
//  * epilogue: store as bfloat16 or float32, ADD into the float32 residual stream (each element
//    has one owner, so the add is a plain read-modify-write), or the SiLU gate of a stacked
//    gate/up matrix (blocks of 128 gate rows followed by their 128 "up" rows): a block's 16 rows
//    are then 8 gate rows and their 8 up rows, and it stores silu(gate) * up.
//
// A chain (o_proj -> gate/up -> down -> the next layer's q/k/v, say) is run link by link by the same
// blocks; between two links all blocks meet at a barrier in global memory (a counter; the wait is
// bounded and a block that gives up sets MLR_STATUS_TIMEOUT and leaves), and before a warp goes
// to the barrier it has issued the loads of its first weights of the next link, so that memory
// keeps streaming while the blocks meet.  Measured on a B200 with the 8B layer sizes: four
// products as four launches 72 us, as one pass 58 us (6.6 TB/s).  Inside a chain everything that
// another block may have written (activations, the stream) is read past L1.
//
// The reference sends these products to cuBLAS gemv kernels (src/minillm/cuda/matrix.cpp:30-36) and
// runs norm, gate and residual add as kernels of their own (src/minillm/cuda/layer.cpp:42-70).
#include "common.cuh"

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kUnitRows = 16;
constexpr int kGroupWarps = 4;           // warps that share a unit of 16 rows (they cut K among them)
constexpr int kGroups = kWarps / kGroupWarps;
constexpr int kGateBlock = 128;
constexpr int kMaxLinks = 8;
constexpr int kMaxRows = 8;
constexpr long long kWaitLimitCycles = 4000000000LL;      // about two seconds

enum Mode : int { kStoreBf16 = 0, kStoreF32 = 1, kAddF32 = 2, kSiluGateBf16 = 3 };

struct Link {
    const __nv_bfloat16* W;
    long long ldw;
    int N, K;
    const void* x;              // bfloat16 activations [M, K], or the float32 stream when `norm`
    long long ldx;
    int norm;
    int norm_weight_bf16;
    const void* norm_weight;
    const int* row_index;       // with `norm`: row r of the product is row row_index[r] of the stream (null: r)
    float eps;
    int mode;
    void* out;
    long long ldo;
};

struct Chain {
    Link links[kMaxLinks];
    int n_links;
    int M;
    unsigned* barrier;          // zero at launch, zero again when the grid has finished
    int* status;
};

__device__ __forceinline__ uint4 load_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mma_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The two weight rows a lane reads in unit `u`: rows `first` + g and `first` + g + 8 of a plain matrix; in
// a stacked gate/up matrix gate row j and its up row, for the 8 outputs j = 8 u .. 8 u + 7.
__device__ __forceinline__ void rows_of_lane(const Link& l, int unit, int g, int& row_a, int& row_b) {
    if (l.mode == kSiluGateBf16) {
        const int j = unit * 8 + g;
        row_a = (j / kGateBlock) * 2 * kGateBlock + j % kGateBlock;
        row_b = row_a + kGateBlock;
    } else {
        row_a = unit * kUnitRows + g;
        row_b = row_a + 8;
    }
}
__host__ __device__ inline int units_of(const Link& l) {
    return l.mode == kSiluGateBf16 ? l.N / kUnitRows : (l.N + kUnitRows - 1) / kUnitRows;
}
// Bytes between rows of the activations in shared memory: K values and a pad that makes it 64 modulo 128,
// so that the 16-byte reads of the eight rows a quarter-warp touches fall into different banks.
__host__ __device__ inline int x_stride_bytes(int K) { return K * 2 + ((64 - (K * 2) % 128) + 128) % 128; }

// One batch of a lane's weights: two windows of 64 values of its two rows in `unit`, as four 16-byte loads per
// row (the halves of a window are 32 values apart); nothing beyond K or beyond the warp's last window.
__device__ __forceinline__ void load_batch(const Link& l, int unit, int win, int win_end, int g, int t, uint4 (&a)[4], uint4 (&b)[4]) {
    int row_a, row_b;
    rows_of_lane(l, unit, g, row_a, row_b);
    const __nv_bfloat16* wa = l.W + static_cast<size_t>(min(row_a, l.N - 1)) * l.ldw;
    const __nv_bfloat16* wb = l.W + static_cast<size_t>(min(row_b, l.N - 1)) * l.ldw;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k = (win + (i >> 1)) * 64 + (i & 1) * 32 + t * 8;
        const bool in = win + (i >> 1) < win_end && k < l.K;
        a[i] = in ? load_stream(wa + k) : make_uint4(0, 0, 0, 0);
        b[i] = in ? load_stream(wb + k) : make_uint4(0, 0, 0, 0);
    }
}

// All blocks of the grid meet; `target` arrivals in total.  False if the wait ran out.
__device__ bool grid_meeting(unsigned* counter, unsigned target, int* status, int* shared_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        int ok = 1;
        if (load_acquire(counter) < target) {
            const long long start = clock64();
            while (load_acquire(counter) < target) {
                if (clock64() - start > kWaitLimitCycles) {
                    ok = 0;
                    break;
                }
            }
        }
        __threadfence();
        if (!ok && status) atomicOr(status, MLR_STATUS_TIMEOUT);
        *shared_flag = ok;
    }
    __syncthreads();
    return *shared_flag != 0;
}

__global__ void __launch_bounds__(kThreads, 1) chain_kernel(const __grid_constant__ Chain chain) {
    extern __shared__ __align__(16) unsigned char shared[];
    __shared__ float reduce_scratch[32];
    __shared__ int meeting_flag;
    // [2][kWarps][16 rows][8 tokens] partial sums of the warps' K ranges, then the activations.
    float* partial = reinterpret_cast<float*>(shared);
    unsigned char* xs = shared + 2 * kWarps * kUnitRows * kMaxRows * sizeof(float);
    mlr_grid_dependents_may_start();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int group = warp / kGroupWarps, in_group = warp % kGroupWarps;
    const int M = chain.M;
    const bool chained = chain.n_links > 1;

    // A warp's first batch of weights of a link is loaded BEFORE the link starts: before the kernels before
    // this one are done (weights have no writer), and before the blocks meet between two links.
    uint4 a[4], b[4];
    int unit = 0, win = 0, win_begin = 0, win_end = 0;
    bool have = false;
    auto start_link = [&](const Link& l) {
        const int windows = (l.K + 63) / 64;
        win_begin = in_group * windows / kGroupWarps;
        win_end = (in_group + 1) * windows / kGroupWarps;
        unit = blockIdx.x * kGroups + group;
        win = win_begin;
        have = unit < units_of(l) && win_begin < win_end;
        if (have) load_batch(l, unit, win, win_end, g, t, a, b);
    };
    start_link(chain.links[0]);
    mlr_grid_wait();

    int parity = 0;
    for (int link = 0; link < chain.n_links; ++link) {
        const Link& l = chain.links[link];
        const int K = l.K, stride = x_stride_bytes(K);
        if (link > 0 && !grid_meeting(chain.barrier, static_cast<unsigned>(link) * gridDim.x, chain.status, &meeting_flag)) return;

        // ---- this link's activations into shared memory (what another block wrote is read past L1)
        // Rows are dealt to the warps (16 warps: all of them on one row, or 8, 4, 2 warps per row), and every
        // thread issues its loads in batches of eight before it touches any of them, so that a row costs a
        // round trip or two to L2 however many rows there are.
        const int rows_pow2 = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
        const int row_warps = kWarps / rows_pow2, m = warp / row_warps;
        const int in_row = (warp % row_warps) * 32 + lane, row_threads = row_warps * 32;
        if (l.norm) {
            const float* h = static_cast<const float*>(l.x);
            const float* row = h + static_cast<size_t>(m < M ? (l.row_index ? l.row_index[m] : m) : 0) * l.ldx;
            const int quads = K >> 2;
            float sum = 0.0f;
            if (m < M)
                for (int base = in_row; base < quads; base += row_threads * 8) {
                    float4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int q = base + j * row_threads;
                        v[j] = q < quads ? __ldcg(reinterpret_cast<const float4*>(row) + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) sum += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
                }
            sum = mlr_warp_sum(sum);
            if (lane == 0) reduce_scratch[warp] = sum;
            __syncthreads();
            if (m < M) {
                float total = 0.0f;
                for (int w = 0; w < row_warps; ++w) total += reduce_scratch[m * row_warps + w];
                const float scale = 1.0f / sqrtf(total / static_cast<float>(K) + l.eps);
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(xs + static_cast<size_t>(m) * stride);
                for (int base = in_row; base < quads; base += row_threads * 8) {
                    float4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int q = base + j * row_threads;
                        v[j] = q < quads ? __ldcg(reinterpret_cast<const float4*>(row) + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int q = base + j * row_threads;
                        if (q < quads) {
                            float w[4];
                            if (l.norm_weight_bf16) mlr_load4(static_cast<const __nv_bfloat16*>(l.norm_weight) + 4 * q, w);
                            else mlr_load4(static_cast<const float*>(l.norm_weight) + 4 * q, w);
                            mlr_store4(dst + 4 * q, (v[j].x * scale) * w[0], (v[j].y * scale) * w[1], (v[j].z * scale) * w[2],
                                       (v[j].w * scale) * w[3]);
                        }
                    }
                }
            }
        } else if (m < M) {
            const uint4* x = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(l.x) + static_cast<size_t>(m) * l.ldx);
            uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * stride);
            const int octs = K >> 3;
            for (int base = in_row; base < octs; base += row_threads * 8) {
                uint4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int q = base + j * row_threads;
                    v[j] = q < octs ? __ldcg(x + q) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int q = base + j * row_threads;
                    if (q < octs) dst[q] = v[j];
                }
            }
        }
        __syncthreads();

        // ---- the rows: a group of four warps takes 16 at a time and cuts K among its warps in windows of 64
        // values.  A warp's loads run one batch (two windows) ahead of its multiply-adds, across the end of a
        // unit too, so that its requests to memory never pause.
        const int units = units_of(l);
        const unsigned char* xrow = xs + static_cast<size_t>(g) * stride;
        const int unit_stride = gridDim.x * kGroups;
        const bool idle_warp = win_begin >= win_end;       // more warps than windows: this one only meets the others
        float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        while (unit < units) {
            int next_unit = unit, next_win = win + 2;
            if (next_win >= win_end) {
                next_unit = unit + unit_stride;
                next_win = win_begin;
            }
            uint4 na[4], nb[4];
            const bool next_have = next_unit < units && !idle_warp;
            if (next_have) load_batch(l, next_unit, next_win, win_end, g, t, na, nb);
            if (have) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int k = (win + (i >> 1)) * 64 + (i & 1) * 32 + t * 8;
                    const bool in = win + (i >> 1) < win_end && k < K && g < M;
                    const uint4 x = in ? *reinterpret_cast<const uint4*>(xrow + k * 2) : make_uint4(0, 0, 0, 0);
                    mma_16x8x16(c, a[i].x, b[i].x, a[i].y, b[i].y, x.x, x.y);
                    mma_16x8x16(c, a[i].z, b[i].z, a[i].w, b[i].w, x.z, x.w);
                }
            }
            if (next_unit != unit) {
                // The group's four sums meet in shared memory; its 128 threads add them in warp order and finish the rows.
                float* mine = partial + (((parity * kGroups + group) * kGroupWarps + in_group) * kUnitRows) * kMaxRows;
                mine[g * kMaxRows + 2 * t] = c[0];
                mine[g * kMaxRows + 2 * t + 1] = c[1];
                mine[(g + 8) * kMaxRows + 2 * t] = c[2];
                mine[(g + 8) * kMaxRows + 2 * t + 1] = c[3];
                c[0] = c[1] = c[2] = c[3] = 0.0f;
                asm volatile("bar.sync %0, %1;\n" ::"r"(1 + group), "r"(kGroupWarps * 32) : "memory");
                {
                    const int i = in_group * 32 + lane, r = i >> 3, m = i & 7;
                    const float* sums = partial + ((parity * kGroups + group) * kGroupWarps * kUnitRows) * kMaxRows + r * kMaxRows + m;
                    float y = 0.0f;
#pragma unroll
                    for (int w = 0; w < kGroupWarps; ++w) y += sums[w * kUnitRows * kMaxRows];
                    if (m < M) {
                        const size_t at = static_cast<size_t>(m) * l.ldo;
                        if (l.mode == kSiluGateBf16) {
                            if (r < 8) {
                                float up = 0.0f;
#pragma unroll
                                for (int w = 0; w < kGroupWarps; ++w) up += sums[w * kUnitRows * kMaxRows + 8 * kMaxRows];
                                static_cast<__nv_bfloat16*>(l.out)[at + unit * 8 + r] = __float2bfloat16_rn((y / (1.0f + expf(-y))) * up);
                            }
                        } else {
                            const int row = unit * kUnitRows + r;
                            if (row < l.N) {
                                if (l.mode == kStoreBf16) static_cast<__nv_bfloat16*>(l.out)[at + row] = __float2bfloat16_rn(y);
                                else if (l.mode == kStoreF32) static_cast<float*>(l.out)[at + row] = y;
                                else {
                                    float* cell = static_cast<float*>(l.out) + at + row;
                                    *cell = __ldcg(cell) + y;
                                }
                            }
                        }
                    }
                }
                parity ^= 1;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = na[i];
                b[i] = nb[i];
            }
            unit = next_unit;
            win = next_win;
            have = next_have;
        }

        // ---- before the blocks meet: the first weights of the next link
        if (link + 1 < chain.n_links) start_link(chain.links[link + 1]);
    }
    if (chained) {
        // The last block to leave sets the counter back to zero for the next launch.
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            const unsigned total = static_cast<unsigned>(chain.n_links) * gridDim.x;
            if (atomicAdd(chain.barrier, 1u) + 1u == total) *chain.barrier = 0u;
        }
    }
}

size_t shared_bytes_for(const Chain& chain) {
    size_t most = 0;
    for (int i = 0; i < chain.n_links; ++i) {
        const size_t rows = static_cast<size_t>(chain.M) * x_stride_bytes(chain.links[i].K);
        most = rows > most ? rows : most;
    }
    return 2 * kWarps * kUnitRows * kMaxRows * sizeof(float) + most;
}

int sm_limit_bytes() {
    int device = 0, bytes = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&bytes, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    return bytes;
}

int check_link(const Link& l, int index) {
    MLR_REQUIRE(l.N >= 1 && l.K >= 8 && l.K % 8 == 0, "gemv_bf16: link %d: bad sizes N=%d K=%d (K must be a multiple of 8)", index, l.N, l.K);
    MLR_REQUIRE(l.mode >= kStoreBf16 && l.mode <= kSiluGateBf16, "gemv_bf16: link %d: unknown mode %d", index, l.mode);
    MLR_REQUIRE(l.mode != kSiluGateBf16 || l.N % (2 * kGateBlock) == 0,
                "gemv_bf16: link %d: a stacked gate/up matrix has a multiple of 256 rows, got %d", index, l.N);
    MLR_REQUIRE(l.ldw % 8 == 0 && reinterpret_cast<uintptr_t>(l.W) % 16 == 0, "gemv_bf16: link %d: the weight rows must be 16-byte aligned", index);
    MLR_REQUIRE(l.norm ? (l.ldx % 4 == 0 && reinterpret_cast<uintptr_t>(l.x) % 16 == 0 && l.norm_weight != nullptr &&
                          reinterpret_cast<uintptr_t>(l.norm_weight) % 16 == 0)
                       : (l.ldx % 8 == 0 && reinterpret_cast<uintptr_t>(l.x) % 16 == 0),
                "gemv_bf16: link %d: the activation rows must be 16-byte aligned (and a norm needs its weight)", index);
    return 0;
}

int launch_chain(const Chain& chain, cudaStream_t stream) {
    MLR_REQUIRE(chain.M >= 1 && chain.M <= kMaxRows, "gemv_bf16: takes 1 to %d rows, got %d", kMaxRows, chain.M);
    MLR_REQUIRE(chain.n_links >= 1 && chain.n_links <= kMaxLinks, "gemv_bf16: a chain has 1 to %d links, got %d", kMaxLinks, chain.n_links);
    MLR_REQUIRE(chain.n_links == 1 || chain.barrier != nullptr, "gemv_bf16: a chain of several links needs its meeting counter");
    for (int i = 0; i < chain.n_links; ++i)
        if (int e = check_link(chain.links[i], i)) return e;
    const size_t bytes = shared_bytes_for(chain);
    MLR_REQUIRE(bytes + 1024 <= static_cast<size_t>(sm_limit_bytes()), "gemv_bf16: rows of %d values do not fit shared memory",
                chain.links[0].K);
    static size_t allowed = 0;
    if (bytes > allowed) {
        if (cudaFuncSetAttribute(chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess) {
            cudaGetLastError();
            return mlr_fail("gemv_bf16: %zu bytes of shared memory were refused", bytes);
        }
        allowed = bytes;
    }
    // As many blocks as are resident at once (a chain's blocks wait for one another), at most one per unit of the largest link.
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, chain_kernel, kThreads, bytes) != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        return mlr_fail("gemv_bf16: the kernel does not fit an SM with %zu bytes of shared memory", bytes);
    }
    int most_units = 0;
    for (int i = 0; i < chain.n_links; ++i) most_units = units_of(chain.links[i]) > most_units ? units_of(chain.links[i]) : most_units;
    const int resident = mlr_sm_count() * per_sm;
    const int wanted = (most_units + kGroups - 1) / kGroups;          // a block's four groups take a unit each
    const int grid = wanted < resident ? wanted : resident;
    mlr_launch((chain_kernel), dim3(grid), dim3(kThreads), bytes, stream, chain);
    return mlr_launched("gemv_bf16");
}

}  // namespace

// One link as the host describes it (mirrored by the Python binding).
struct MlrGemvLink {
    const void* W;
    long long ldw;
    int N, K;
    const void* x;
    long long ldx;
    int norm;
    int norm_weight_bf16;
    const void* norm_weight;
    const int* row_index;
    float eps;
    int mode;
    void* out;
    long long ldo;
};

// Whether mlr_gemv_bf16 takes a product of `M` rows over K values (its activations must fit shared memory).
MLR_API int mlr_gemv_bf16_fits(int M, int K) {
    return M >= 1 && M <= kMaxRows && K >= 8 && K % 8 == 0 &&
           2 * kWarps * kUnitRows * kMaxRows * sizeof(float) + static_cast<size_t>(M) * x_stride_bytes(K) + 1024 <=
               static_cast<size_t>(sm_limit_bytes());
}

// out = f(x W^T) for 1 <= M <= 8 rows.  W: [N, K] bfloat16, rows `ldw` elements apart (a multiple of 8),
// 16-byte aligned.  `norm` = 0: x is bfloat16 [M, K], rows `ldx` apart; `norm` = 1: x is the float32
// residual stream, rows `ldx` apart, and the product's row r is the RMS norm (weight `norm_weight`,
// bfloat16 or float32, `eps`) of its row row_index[r] (r when row_index is null), rounded to bfloat16.
// mode 0: out bfloat16 [M, N]; 1: out float32 [M, N]; 2: out float32 [M, N] += the product; 3: W is a
// stacked gate/up matrix (blocks of 128 gate rows, each followed by its 128 "up" rows; N a multiple of
// 256) and out is bfloat16 [M, N / 2] = silu(gate) * up.  `ldo`: elements between rows of out.
MLR_API int mlr_gemv_bf16(const void* W, long long ldw, int N, int K, const void* x, long long ldx, int norm,
                          const void* norm_weight, int norm_weight_bf16, float eps, const int* row_index, int M, void* out,
                          long long ldo, int mode, cudaStream_t stream) {
    Chain chain = {};
    chain.links[0] = Link{static_cast<const __nv_bfloat16*>(W), ldw, N, K, x, ldx, norm, norm_weight_bf16, norm_weight, row_index, eps, mode, out, ldo};
    chain.n_links = 1;
    chain.M = M;
    return launch_chain(chain, stream);
}

// Several such products, each reading what earlier ones wrote, run link by link by one persistent grid
// (see the head of this file).  `links`: host memory.  `barrier`: one unsigned on the device, zero before the
// first launch; the kernel leaves it zero.  Launches that share a counter must not overlap on the GPU.
MLR_API int mlr_gemv_chain(const MlrGemvLink* links, int n_links, int M, unsigned* barrier, int* status, cudaStream_t stream) {
    MLR_REQUIRE(n_links >= 1 && n_links <= kMaxLinks, "gemv_bf16: a chain has 1 to %d links, got %d", kMaxLinks, n_links);
    Chain chain = {};
    for (int i = 0; i < n_links; ++i) {
        const MlrGemvLink& s = links[i];
        chain.links[i] = Link{static_cast<const __nv_bfloat16*>(s.W), s.ldw, s.N, s.K, s.x, s.ldx, s.norm, s.norm_weight_bf16, s.norm_weight,
                              s.row_index, s.eps, s.mode, s.out, s.ldo};
    }
    chain.n_links = n_links;
    chain.M = M;
    chain.barrier = barrier;
    chain.status = status;
    return launch_chain(chain, stream);
}
