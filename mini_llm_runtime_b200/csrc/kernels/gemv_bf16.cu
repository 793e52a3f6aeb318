// Products of a decode step's few rows (one to eight): out[M, N] = f(x[M, K] W[N, K]^T).
//
// With so few rows a product is a pass over the weight matrix and nothing else, so the kernel is built
// around the memory system.  One warp of each block does nothing but fetch: it keeps a ring of two slots
// (three where one row of activations leaves room: more bytes on their way, 3 us a layer at the 8B sizes)
// of shared memory filled with the weights of 16 rows of W (a "unit") over a chunk of K, a bulk copy
// (`cp.async.bulk`, completion counted by an mbarrier) of up to 4 KB per row.  A bulk copy costs the copy
// engine about 50 ns whatever its size, so the rows are copied in pieces as long as shared memory allows;
// and because the copies land in shared memory, what is in flight does not depend on how much L1 the
// activations leave (loads into registers did: with eight rows of activations in shared memory they fell
// to half the bandwidth).  Weights have no writer, so the fetching warp starts before the kernel before
// this one has finished (programmatic dependent launch) and memory streams while the others still wait.
// The 16 other warps multiply: warp w takes values 32 w .. 32 w + 31 of every 512 of a chunk, a lane reads
// 16 bytes of two weight rows and of its token's activations from shared memory, and these are the
// operands of two `mma.sync.m16n8k16` (the order of the k values inside an instruction is permuted the
// same way for W and for x, which a sum does not notice).  The tensor cores do the multiply-adds of all
// rows at once, so eight rows cost what one costs; the 16 warps' sums are added in shared memory in a fixed
// order, so a result depends neither on the grid nor on timing.  (`mma.sync` is the older tensor-core
// instruction; `tcgen05.mma` pays off when both operands are tiles of 64 rows and more, as in the products
// of prompt portions, which use it.)
//
// Folded in, so that they are no launches of their own:
//  * prologue: the RMS norm of the rows of the float32 residual stream that feed the product: the rows
//    times the norm's weight go to shared memory as bfloat16 while their squares are summed, and the row's
//    1/rms multiplies the finished sums (it is one factor for a whole row of x); on all rows or on the
//    rows an index names (the final norm before the output head);
//  * epilogue: store as bfloat16 or float32, ADD into the float32 residual stream (each element has one
//    owner, so the add is a plain read-modify-write), or the SiLU gate of a stacked gate/up matrix (blocks
//    of 128 gate rows followed by their 128 "up" rows): a unit's 16 rows are then 8 gate rows and their 8
//    up rows, and it stores silu(gate) * up.
//
// Two more things keep eight rows as fast as one:
//  * Where K is at most 4096 and no norm has to be worked out from the stream, the activations never go to shared
//    memory: a lane needs 16 bytes of its token's row per 512 values of K, eight registers' worth of loads, and
//    shared memory is all ring (three slots at any row count).  A product that ADDS into the stream is cut along K
//    into parts of at most 4096 values for that: each part adds its partial product into the stream (a cell has the
//    same owner in every part).  Other products (a norm prologue, a wider K) stage their activations in shared
//    memory beside a ring of two slots (three at one row), with shorter copies or one buffer of partial sums
//    where room is short.
//  * Every block needs all of a product's activations, so 148 blocks reading eight float32 rows of the
//    stream for a norm is 19 MB through L2 (8 us).  The product that added into that stream last has the
//    final values in hand: `mlr_gemv_bf16_add_prepare` stores them a second time as bfloat16, already times
//    the norm's weight, and the sum of squares of its 16 rows per token; `mlr_gemv_bf16_prepared` then
//    reads half the bytes and adds up the partial sums in a fixed order for the row's 1/rms.
//
// Measured on a B200 with the 8B layer sizes in a CUDA graph (o_proj, gate/up, down, q/k/v as launches of
// their own): 6.9 / 30.4 / 18.1 / 8.8 us at one row, 8.2 / 31.9 / 21.7 / 9.7 us at eight, 6.3 to 6.6 TB/s on
// the largest.  Run by one persistent grid with meetings of all blocks between the products instead of launch
// boundaries they took 3.5 us longer per layer, so that form was dropped.
//
// The reference sends these products to cuBLAS gemv kernels (src/minillm/cuda/matrix.cpp:30-36) and
// runs norm, gate and residual add as kernels of their own (src/minillm/cuda/layer.cpp:42-70).
#include "common.cuh"

namespace {

constexpr int kConsumerWarps = 16;          // the warps that multiply; they cut each 512 values of K among them
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;   // and the warp that fetches weights
constexpr int kUnitRows = 16;
constexpr int kMostSlots = 3;
constexpr int kRegisterBlocks = 8;          // blocks of 512 values of K whose activations a lane can keep in registers
constexpr int kMostChunk = 2048;            // values of K of a unit's 16 rows in one slot of the ring, at most (4 KB copies)
constexpr int kStageLoads = 8;              // loads a thread has in flight while a part's activations are staged
constexpr int kGateBlock = 128;
constexpr int kMaxParts = 16;
constexpr int kMaxRows = 8;
constexpr int kPartialBytes = kConsumerWarps * kUnitRows * kMaxRows * 4;        // one buffer of the warps' partial sums
constexpr long long kWaitLimitCycles = 4000000000LL;      // about two seconds

enum Mode : int { kStoreBf16 = 0, kStoreF32 = 1, kAddF32 = 2, kSiluGateBf16 = 3 };

struct Link {
    const __nv_bfloat16* W;
    long long ldw;
    int N, K;
    const void* x;              // bfloat16 activations [M, K]; the float32 stream when `norm` is 1
    long long ldx;
    int norm;                   // 0: x as it is; 1: the RMS norm of the stream in the prologue; 2: x was prepared by the product before
    int norm_weight_bf16;
    const void* norm_weight;
    const int* row_index;       // with `norm` 1: row r of the product is row row_index[r] of the stream (null: r)
    float eps;
    int mode;
    void* out;
    long long ldo;
    // An adding product that prepares the norm of the product after it:
    __nv_bfloat16* side;        // [M, N] bfloat16: the new stream times `side_weight`
    const void* side_weight;
    int side_weight_bf16;
    float* squares;             // producer: [units][8] sums of squares of a unit's rows per token; consumer (norm 2): the same, to add up
    int n_squares;              // consumer: how many lines `squares` has
};

// One product as the kernel runs it: whole, or cut along K into parts that each add into the stream.
struct Job {
    Link parts[kMaxParts];
    int n_parts;
    int M;
    int chunk;                  // values of K per ring slot: a multiple of 512
    int x_bytes;                // shared memory for the activations
    int slots;                  // of the ring: 2, or 3 where the activations leave room
    int partial_buffers;        // 2: a unit's partial sums do not wait for the unit before to be finished; 1 where shared memory is short
    int* status;
};

__device__ __forceinline__ void mma_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 load_shared16(uint32_t address) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(address));
    return v;
}

// ---- mbarriers and bulk copies (the ring of weights)
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
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// Waits for a phase of a barrier, but not for ever.  A wait that runs out (about two seconds) sets the block's
// `failed` flag and MLR_STATUS_TIMEOUT; from then on no wait of the block waits, so that every thread still walks
// through the same barriers to the kernel's end (its results are then worthless, and the status says so).
__device__ __forceinline__ void wait_phase(uint32_t bar, uint32_t parity, volatile int* failed, int* status) {
    if (mbar_try_wait(bar, parity)) return;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*failed) return;
        if (clock64() - start > kWaitLimitCycles) {
            *failed = 1;
            if (status) atomicOr(status, MLR_STATUS_TIMEOUT);
            return;
        }
    }
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 2, %0;\n" ::"n"(kConsumers) : "memory"); }

// Row `r` (0..15) of unit `unit` in W: rows 16 u .. 16 u + 15 of a plain matrix; in a stacked gate/up matrix the gate
// rows of the 8 outputs j = 8 u .. 8 u + 7 (r < 8) and their up rows (r >= 8).
__device__ __forceinline__ int row_of_unit(const Link& l, int unit, int r) {
    if (l.mode == kSiluGateBf16) {
        const int j = unit * 8 + (r & 7);
        return (j / kGateBlock) * 2 * kGateBlock + j % kGateBlock + (r >= 8 ? kGateBlock : 0);
    }
    return unit * kUnitRows + r;
}
__host__ __device__ inline int units_of(const Link& l) {
    return l.mode == kSiluGateBf16 ? l.N / kUnitRows : (l.N + kUnitRows - 1) / kUnitRows;
}
// Bytes between rows of the activations in shared memory, and between a slot's rows of weights: the values and a
// pad that makes it 64 modulo 128, so that the 16-byte reads of the eight rows a quarter-warp touches fall into
// different banks.
__host__ __device__ inline int pitch_bytes(int values) { return values * 2 + ((64 - (values * 2) % 128) + 128) % 128; }
__host__ __device__ inline size_t x_region_bytes(int M, int K) { return (static_cast<size_t>(M) * pitch_bytes(K) + 127) / 128 * 128; }
__host__ __device__ inline size_t ring_bytes(int chunk, int slots) { return static_cast<size_t>(slots) * kUnitRows * pitch_bytes(chunk); }

// XREG: the activations stay in registers (a lane needs 16 bytes of its token's row per 512 values of K, at most
// kRegisterBlocks of them), shared memory holds no copy of them and the ring has a third slot at any row count.  Only
// for parts of at most 512 * kRegisterBlocks values whose norm, if any, was prepared.
template <bool XREG>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const __grid_constant__ Job job) {
    extern __shared__ __align__(128) unsigned char shared[];
    __shared__ float reduce_scratch[32];
    __shared__ float row_scale[kMaxRows];
    __shared__ __align__(16) float square_scratch[kConsumerWarps * kMaxRows];
    __shared__ __align__(8) unsigned long long barriers[2 * kMostSlots];
    __shared__ int failed_flag;
    // [2][16 warps][16 rows][8 tokens] partial sums of the warps' K ranges | the activations | the ring of weights
    float* partial = reinterpret_cast<float*>(shared);
    unsigned char* xs = shared + job.partial_buffers * kPartialBytes;
    const int slot_pitch = pitch_bytes(job.chunk), slot_bytes = kUnitRows * slot_pitch;
    const uint32_t ring = static_cast<uint32_t>(__cvta_generic_to_shared(xs + job.x_bytes));
    const uint32_t bars = static_cast<uint32_t>(__cvta_generic_to_shared(barriers));
    auto full_bar = [&](int slot) { return bars + 8u * slot; };
    auto empty_bar = [&](int slot) { return bars + 8u * (kMostSlots + slot); };
    volatile int* failed = &failed_flag;
    mlr_grid_dependents_may_start();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int M = job.M, slots = job.slots;
    if (threadIdx.x == 0) {
        failed_flag = 0;
        for (int s = 0; s < slots; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---- the warp that fetches: slot after slot, 16 rows x one chunk of W each, a bulk copy per row issued
        // by 16 lanes, as far ahead as the ring has room.  It does not wait for the kernels before this one.
        int i = 0;
        for (int part = 0; part < job.n_parts; ++part) {
            const Link& l = job.parts[part];
            const int units = units_of(l), chunks = (l.K + job.chunk - 1) / job.chunk;
            for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
                const int row = row_of_unit(l, unit, lane & 15);
                const bool valid = lane < kUnitRows && row < l.N;
                const int n_valid = __popc(__ballot_sync(0xffffffffu, valid));
                const __nv_bfloat16* src = l.W + static_cast<size_t>(valid ? row : 0) * l.ldw;
                for (int c = 0; c < chunks; ++c, ++i) {
                    const int slot = i % slots;
                    if (i >= slots) wait_phase(empty_bar(slot), ((i / slots) - 1) & 1, failed, job.status);
                    const int k0 = c * job.chunk;
                    const uint32_t bytes = static_cast<uint32_t>(min(job.chunk, l.K - k0)) * 2u;
                    if (lane == 0) mbar_expect_tx(full_bar(slot), bytes * n_valid);
                    __syncwarp();
                    if (valid && !*failed) bulk_copy(ring + slot * slot_bytes + lane * slot_pitch, src + k0, bytes, full_bar(slot));
                }
            }
        }
        if (*failed) {
            // Leave only when the copies that were issued have landed (or after another bounded wait): the block's
            // shared memory must not be given to another block with copies into it in flight.
            for (int back = 1; back <= slots && back <= i; ++back) {
                const int j = i - back;
                const long long start = clock64();
                while (!mbar_try_wait(full_bar(j % slots), (j / slots) & 1) && clock64() - start < kWaitLimitCycles) {
                }
            }
        }
        return;
    }

    // ---- the 16 warps that multiply
    const int g = lane >> 2, t = lane & 3;
    mlr_grid_wait();
    int parity = 0, i = 0;
    for (int part = 0; part < job.n_parts; ++part) {
        const Link& l = job.parts[part];
        const int K = l.K, stride = pitch_bytes(K);
        consumers_sync();        // the block's warps are done with the activations of the part before

        // ---- this part's activations into shared memory (read past L1: the kernel before this one wrote them)
        // Rows are dealt to the warps (16 warps: all of them on one row, or 8, 4, 2 warps per row), and every
        // thread issues its loads in batches of eight before it touches any of them, so that a row costs a
        // round trip or two to L2 however many rows there are.
        const int rows_pow2 = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
        const int row_warps = kConsumerWarps / rows_pow2, m = warp / row_warps;
        const int in_row = (warp % row_warps) * 32 + lane, row_threads = row_warps * 32;
        if (l.norm == 1) {
            // One pass: x * weight goes to shared memory as bfloat16 while the squares are summed; the row's
            // 1/rms multiplies the finished sums instead (it is one factor for the whole row of x).
            const float* h = static_cast<const float*>(l.x);
            const float* row = h + static_cast<size_t>(m < M ? (l.row_index ? l.row_index[m] : m) : 0) * l.ldx;
            const int quads = K >> 2;
            float sum = 0.0f;
            if (m < M) {
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(xs + static_cast<size_t>(m) * stride);
                for (int base = in_row; base < quads; base += row_threads * kStageLoads) {
                    float4 v[kStageLoads];
#pragma unroll
                    for (int j = 0; j < kStageLoads; ++j) {
                        const int q = base + j * row_threads;
                        v[j] = q < quads ? __ldcg(reinterpret_cast<const float4*>(row) + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
#pragma unroll
                    for (int j = 0; j < kStageLoads; ++j) {
                        const int q = base + j * row_threads;
                        sum += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
                        if (q < quads) {
                            float w[4];
                            if (l.norm_weight_bf16) mlr_load4(static_cast<const __nv_bfloat16*>(l.norm_weight) + 4 * q, w);
                            else mlr_load4(static_cast<const float*>(l.norm_weight) + 4 * q, w);
                            mlr_store4(dst + 4 * q, v[j].x * w[0], v[j].y * w[1], v[j].z * w[2], v[j].w * w[3]);
                        }
                    }
                }
            }
            sum = mlr_warp_sum(sum);
            if (lane == 0) reduce_scratch[warp] = sum;
            consumers_sync();
            if (threadIdx.x < kMaxRows) {
                float total = 0.0f;
                if (threadIdx.x < M)
                    for (int w = 0; w < row_warps; ++w) total += reduce_scratch[threadIdx.x * row_warps + w];
                row_scale[threadIdx.x] = 1.0f / sqrtf(total / static_cast<float>(K) + l.eps);
            }
        } else {
            if (l.norm == 2) {
                // The product before left a line of 8 sums of squares per unit.  Thread j takes the half lines j, j + 512, ...
                // (4 tokens each, one load per round), lanes 2 apart add up, then the warps in order.
                const int halves = 2 * l.n_squares;
                float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int j = threadIdx.x; j < halves; j += kConsumers) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(l.squares) + j);
                    total.x += v.x, total.y += v.y, total.z += v.z, total.w += v.w;
                }
#pragma unroll
                for (int step = 2; step < 32; step <<= 1) {
                    total.x += __shfl_xor_sync(0xffffffffu, total.x, step);
                    total.y += __shfl_xor_sync(0xffffffffu, total.y, step);
                    total.z += __shfl_xor_sync(0xffffffffu, total.z, step);
                    total.w += __shfl_xor_sync(0xffffffffu, total.w, step);
                }
                if (lane < 2) *reinterpret_cast<float4*>(square_scratch + warp * kMaxRows + lane * 4) = total;
                consumers_sync();
                if (threadIdx.x < kMaxRows) {
                    float sum = 0.0f;
                    for (int w = 0; w < kConsumerWarps; ++w) sum += square_scratch[w * kMaxRows + threadIdx.x];
                    row_scale[threadIdx.x] = 1.0f / sqrtf(sum / static_cast<float>(K) + l.eps);
                }
            } else if (threadIdx.x < kMaxRows) {
                row_scale[threadIdx.x] = 1.0f;
            }
            if (!XREG && m < M) {
            const uint4* x = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(l.x) + static_cast<size_t>(m) * l.ldx);
            uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(m) * stride);
            const int octs = K >> 3;
            for (int base = in_row; base < octs; base += row_threads * kStageLoads) {
                uint4 v[kStageLoads];
#pragma unroll
                for (int j = 0; j < kStageLoads; ++j) {
                    const int q = base + j * row_threads;
                    v[j] = q < octs ? __ldcg(x + q) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < kStageLoads; ++j) {
                    const int q = base + j * row_threads;
                    if (q < octs) dst[q] = v[j];
                }
            }
            }
        }
        consumers_sync();

        // ---- the rows: a unit of 16 at a time, chunk by chunk as the ring delivers them
        const int units = units_of(l), chunks = (K + job.chunk - 1) / job.chunk, subs = job.chunk / 512;
        const uint32_t x_at = static_cast<uint32_t>(__cvta_generic_to_shared(xs)) + g * stride;
        const uint32_t in_slot = (warp * 32 + t * 8) * 2;
        uint4 xr[XREG ? kRegisterBlocks : 1];
        if constexpr (XREG) {
            // This lane's 16 bytes of its token's row for every 512 values of K, straight from the kernel before.
            const uint4 zero = make_uint4(0, 0, 0, 0);
            const __nv_bfloat16* row = static_cast<const __nv_bfloat16*>(l.x) + static_cast<size_t>(g < M ? g : 0) * l.ldx;
#pragma unroll
            for (int b = 0; b < kRegisterBlocks; ++b) {
                const int k = b * 512 + warp * 32 + t * 8;
                xr[b] = g < M && k < K ? __ldcg(reinterpret_cast<const uint4*>(row + k)) : zero;
            }
        }
        for (int unit = blockIdx.x; unit < units; unit += gridDim.x) {
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if constexpr (XREG) {
                // chunks of kMostChunk values: at most kRegisterBlocks / 4 of them, so every register's index is a constant
#pragma unroll
                for (int chunk = 0; chunk < kRegisterBlocks / 4; ++chunk) {
                    if (chunk < chunks) {
                        const int slot = i % slots;
                        wait_phase(full_bar(slot), (i / slots) & 1, failed, job.status);
#pragma unroll
                        for (int sub = 0; sub < 4; ++sub) {
                            const int k = chunk * kMostChunk + sub * 512 + warp * 32 + t * 8;
                            const bool in = k < K;
                            const uint32_t at = ring + slot * slot_bytes + sub * 1024 + in_slot;
                            const uint4 zero = make_uint4(0, 0, 0, 0);
                            const uint4 a = in ? load_shared16(at + g * slot_pitch) : zero;
                            const uint4 b = in ? load_shared16(at + (g + 8) * slot_pitch) : zero;
                            const uint4 x = xr[chunk * 4 + sub];
                            mma_16x8x16(c, a.x, b.x, a.y, b.y, x.x, x.y);
                            mma_16x8x16(c, a.z, b.z, a.w, b.w, x.z, x.w);
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(empty_bar(slot));
                        ++i;
                    }
                }
            } else {
            for (int chunk = 0; chunk < chunks; ++chunk, ++i) {
                const int slot = i % slots;
                wait_phase(full_bar(slot), (i / slots) & 1, failed, job.status);
                for (int sub = 0; sub < subs; ++sub) {
                    const int k = chunk * job.chunk + sub * 512 + warp * 32 + t * 8;
                    const bool in = k < K;
                    const uint32_t at = ring + slot * slot_bytes + sub * 1024 + in_slot;
                    const uint4 zero = make_uint4(0, 0, 0, 0);
                    const uint4 a = in ? load_shared16(at + g * slot_pitch) : zero;
                    const uint4 b = in ? load_shared16(at + (g + 8) * slot_pitch) : zero;
                    const uint4 x = in && g < M ? load_shared16(x_at + k * 2) : zero;
                    mma_16x8x16(c, a.x, b.x, a.y, b.y, x.x, x.y);
                    mma_16x8x16(c, a.z, b.z, a.w, b.w, x.z, x.w);
                }
                __syncwarp();          // every lane's reads of the slot have ended in its multiply-adds
                if (lane == 0) mbar_arrive(empty_bar(slot));
            }
            }
            {
                // The 16 warps' sums meet in shared memory; 128 threads add them in warp order and finish the rows.
                if (job.partial_buffers == 1) asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumers) : "memory");      // the unit before has been finished
                float* mine = partial + ((parity * kConsumerWarps + warp) * kUnitRows) * kMaxRows;
                mine[g * kMaxRows + 2 * t] = c[0];
                mine[g * kMaxRows + 2 * t + 1] = c[1];
                mine[(g + 8) * kMaxRows + 2 * t] = c[2];
                mine[(g + 8) * kMaxRows + 2 * t + 1] = c[3];
                asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumers) : "memory");
                if (threadIdx.x < kUnitRows * kMaxRows) {
                    // Thread i finishes row i % 16 of token i / 16: a token's 16 rows are neighbours in memory and in a warp.
                    const int r = threadIdx.x & 15, m = threadIdx.x >> 4;
                    const float* sums = partial + (parity * kConsumerWarps * kUnitRows) * kMaxRows + r * kMaxRows + m;
                    float y = 0.0f, square = 0.0f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) y += sums[w * kUnitRows * kMaxRows];
                    y *= row_scale[m];
                    if (m < M) {
                        const size_t at = static_cast<size_t>(m) * l.ldo;
                        if (l.mode == kSiluGateBf16) {
                            if (r < 8) {
                                float up = 0.0f;
#pragma unroll
                                for (int w = 0; w < kConsumerWarps; ++w) up += sums[w * kUnitRows * kMaxRows + 8 * kMaxRows];
                                up *= row_scale[m];
                                static_cast<__nv_bfloat16*>(l.out)[at + unit * 8 + r] = __float2bfloat16_rn((y / (1.0f + expf(-y))) * up);
                            }
                        } else {
                            const int row = unit * kUnitRows + r;
                            if (row < l.N) {
                                if (l.mode == kStoreBf16) static_cast<__nv_bfloat16*>(l.out)[at + row] = __float2bfloat16_rn(y);
                                else if (l.mode == kStoreF32) static_cast<float*>(l.out)[at + row] = y;
                                else {
                                    float* cell = static_cast<float*>(l.out) + at + row;
                                    float w = 0.0f;
                                    if (l.side)
                                        w = l.side_weight_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(l.side_weight)[row])
                                                               : static_cast<const float*>(l.side_weight)[row];
                                    const float sum = __ldcg(cell) + y;
                                    *cell = sum;
                                    if (l.side) {
                                        l.side[static_cast<size_t>(m) * l.N + row] = __float2bfloat16_rn(sum * w);
                                        square = sum * sum;
                                    }
                                }
                            }
                        }
                    }
                    if (l.side) {
                        // The squares of a token's 16 rows, added up over the 16 lanes that hold them: one line of 8 per unit.
#pragma unroll
                        for (int step = 1; step < 16; step <<= 1) square += __shfl_xor_sync(0xffffffffu, square, step);
                        if (r == 0) l.squares[static_cast<size_t>(unit) * kMaxRows + m] = square;
                    }
                }
                if (job.partial_buffers == 2) parity ^= 1;
            }
        }
    }
}

int sm_limit_bytes() {
    int device = 0, bytes = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&bytes, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    return bytes;
}

// The longest chunk (a multiple of 512 values, at most kMostChunk) whose ring fits beside `x_bytes` of activations; 0: none does.
int chunk_for(size_t x_bytes, int partial_buffers = 2) {
    const size_t room = static_cast<size_t>(sm_limit_bytes()) - 2048;        // the kernel's static shared memory and what the driver keeps
    for (int chunk = kMostChunk; chunk >= 512; chunk -= 512)
        if (partial_buffers * kPartialBytes + x_bytes + ring_bytes(chunk, 2) <= room) return chunk;
    return 0;
}
// Slots of the ring: a third one where the activations leave room for it (one or two rows of a model's width).
int slots_for(size_t x_bytes, int chunk) {
    const size_t room = static_cast<size_t>(sm_limit_bytes()) - 2048;
    return 2 * kPartialBytes + x_bytes + ring_bytes(chunk, kMostSlots) <= room ? kMostSlots : 2;
}

// How many parts a product over K values is cut into for M rows (1: it stays whole), and the width of a part.  Only a
// product that adds into the stream can be cut; it is, when its activations would push the ring below its best size.
// Whether a product keeps its activations in registers: its norm, if any, was prepared, and its K (or, for a product
// that adds into the stream, the K of its parts) is at most 512 * kRegisterBlocks.
bool in_registers(int K, int mode, int norm) { return norm != 1 && (mode == kAddF32 || K <= 512 * kRegisterBlocks); }

int parts_of(int M, int K, int mode, int norm, int& part_width) {
    part_width = K;
    if (in_registers(K, mode, norm)) {
        const int parts = (K + 512 * kRegisterBlocks - 1) / (512 * kRegisterBlocks);
        if (parts > kMaxParts) return 0;        // (the caller falls back to shared memory)
        part_width = ((K + parts - 1) / parts + 63) / 64 * 64;
        return (K + part_width - 1) / part_width;
    }
    if (mode != kAddF32 || norm != 0 || chunk_for(x_region_bytes(M, K)) == kMostChunk) return 1;
    for (int least = kMostChunk; least >= 512; least -= kMostChunk - 512)       // the best ring if some cut allows it, else any ring
        for (int parts = 2; parts <= kMaxParts; ++parts) {
            const int width = ((K + parts - 1) / parts + 63) / 64 * 64;
            if (chunk_for(x_region_bytes(M, width)) >= least) {
                part_width = width;
                return (K + width - 1) / width;
            }
        }
    return 1;
}

int check_link(const Link& l) {
    MLR_REQUIRE(l.N >= 1 && l.K >= 8 && l.K % 8 == 0, "gemv_bf16: bad sizes N=%d K=%d (K must be a multiple of 8)", l.N, l.K);
    MLR_REQUIRE(l.mode >= kStoreBf16 && l.mode <= kSiluGateBf16, "gemv_bf16: unknown mode %d", l.mode);
    MLR_REQUIRE(l.mode != kSiluGateBf16 || l.N % (2 * kGateBlock) == 0,
                "gemv_bf16: a stacked gate/up matrix has a multiple of 256 rows, got %d", l.N);
    MLR_REQUIRE(l.ldw % 8 == 0 && reinterpret_cast<uintptr_t>(l.W) % 16 == 0, "gemv_bf16: the weight rows must be 16-byte aligned");
    MLR_REQUIRE(l.norm == 1 ? (l.ldx % 4 == 0 && reinterpret_cast<uintptr_t>(l.x) % 16 == 0 && l.norm_weight != nullptr &&
                               reinterpret_cast<uintptr_t>(l.norm_weight) % 16 == 0)
                            : (l.ldx % 8 == 0 && reinterpret_cast<uintptr_t>(l.x) % 16 == 0),
                "gemv_bf16: the activation rows must be 16-byte aligned (and a norm needs its weight)");
    return 0;
}

int launch(const Link& l, int M, int* status, cudaStream_t stream) {
    MLR_REQUIRE(M >= 1 && M <= kMaxRows, "gemv_bf16: takes 1 to %d rows, got %d", kMaxRows, M);
    if (int e = check_link(l)) return e;
    Job job = {};
    job.M = M;
    job.status = status;
    int width = 0;
    job.n_parts = parts_of(M, l.K, l.mode, l.norm, width);
    if (job.n_parts == 0) job.n_parts = 1, width = l.K;
    for (int part = 0; part < job.n_parts; ++part) {
        Link& p = job.parts[part];
        p = l;
        if (job.n_parts > 1) {
            const int from = part * width;
            p.W = l.W + from;
            p.x = static_cast<const __nv_bfloat16*>(l.x) + from;
            p.K = l.K - from < width ? l.K - from : width;
            if (part + 1 < job.n_parts) p.side = nullptr, p.squares = nullptr;       // the last part has the stream's final values
        }
    }
    const bool registers = in_registers(l.K, l.mode, l.norm) && job.parts[0].K <= 512 * kRegisterBlocks;
    size_t x_bytes = 0;
    if (registers) {
        job.partial_buffers = 2;
        job.chunk = kMostChunk;
        job.slots = kMostSlots;
    } else {
        x_bytes = x_region_bytes(M, job.parts[0].K);
        // One buffer of partial sums instead of two where that buys longer copies (eight rows of 5120 values are 1.5 KB
        // too many for the best ring beside two); not for a product that adds: its finish waits for the stream's cells.
        job.partial_buffers = 2;
        job.chunk = chunk_for(x_bytes, 2);
        if (l.mode != kAddF32 && chunk_for(x_bytes, 1) > job.chunk) {
            job.partial_buffers = 1;
            job.chunk = chunk_for(x_bytes, 1);
        }
        MLR_REQUIRE(job.chunk > 0, "gemv_bf16: %d rows of %d values do not fit shared memory", M, l.K);
        job.slots = job.partial_buffers == 2 ? slots_for(x_bytes, job.chunk) : 2;
    }
    job.x_bytes = static_cast<int>(x_bytes);
    const size_t bytes = job.partial_buffers * kPartialBytes + x_bytes + ring_bytes(job.chunk, job.slots);
    const int units = units_of(l), sms = mlr_sm_count();
    const dim3 grid(units < sms ? units : sms);
    static size_t allowed[2] = {0, 0};
    if (bytes > allowed[registers]) {
        const cudaError_t e = registers ? cudaFuncSetAttribute(gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes))
                                        : cudaFuncSetAttribute(gemv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
        if (e != cudaSuccess) {
            cudaGetLastError();
            return mlr_fail("gemv_bf16: %zu bytes of shared memory were refused", bytes);
        }
        allowed[registers] = bytes;
    }
    if (registers) mlr_launch((gemv_kernel<true>), grid, dim3(kThreads), bytes, stream, job);
    else mlr_launch((gemv_kernel<false>), grid, dim3(kThreads), bytes, stream, job);
    return mlr_launched("gemv_bf16");
}

}  // namespace

// Whether mlr_gemv_bf16 takes a product of `M` rows over K values that does not add into the stream (its activations
// must fit shared memory beside the ring; a product that adds is cut into parts that do).
MLR_API int mlr_gemv_bf16_fits(int M, int K) {
    return M >= 1 && M <= kMaxRows && K >= 8 && K % 8 == 0 && (K <= 512 * kRegisterBlocks || chunk_for(x_region_bytes(M, K), 1) > 0);
}

// Into how many parts along K an adding product of `M` rows is cut.
MLR_API int mlr_gemv_bf16_parts(int M, int K) {
    int width = 0;
    return parts_of(M < 1 ? 1 : M > kMaxRows ? kMaxRows : M, K, kAddF32, 0, width);
}

// out = f(x W^T) for 1 <= M <= 8 rows.  W: [N, K] bfloat16, rows `ldw` elements apart (a multiple of 8),
// 16-byte aligned.  `norm` = 0: x is bfloat16 [M, K], rows `ldx` apart; `norm` = 1: x is the float32
// residual stream, rows `ldx` apart, and the product's row r is the RMS norm (weight `norm_weight`,
// bfloat16 or float32, `eps`) of its row row_index[r] (r when row_index is null), rounded to bfloat16.
// mode 0: out bfloat16 [M, N]; 1: out float32 [M, N]; 2: out float32 [M, N] += the product; 3: W is a
// stacked gate/up matrix (blocks of 128 gate rows, each followed by its 128 "up" rows; N a multiple of
// 256) and out is bfloat16 [M, N / 2] = silu(gate) * up.  `ldo`: elements between rows of out.  `status`: a
// device word in which a wait that ran out sets MLR_STATUS_TIMEOUT.
MLR_API int mlr_gemv_bf16(const void* W, long long ldw, int N, int K, const void* x, long long ldx, int norm,
                          const void* norm_weight, int norm_weight_bf16, float eps, const int* row_index, int M, void* out,
                          long long ldo, int mode, int* status, cudaStream_t stream) {
    Link l = {static_cast<const __nv_bfloat16*>(W), ldw, N, K, x, ldx, norm, norm_weight_bf16, norm_weight, row_index, eps, mode, out, ldo};
    return launch(l, M, status, stream);
}

// The two halves of a norm that a product prepares for the product after it.
// `mlr_gemv_bf16_add_prepare`: out [M, N] float32 += x W^T, and for the RMS norm (weight `norm_weight`) that
// reads `out` next: `side` [M, N] bfloat16 = the new out times the weight, `squares` [ceil(N / 16)][8] float32 =
// the sums of squares of 16 columns of out per row.  `mlr_gemv_bf16_prepared`: the product whose input is that
// norm: x W^T with x = side * 1/sqrt(sum(squares) / K + eps), modes as mlr_gemv_bf16.
MLR_API int mlr_gemv_bf16_add_prepare(const void* W, long long ldw, int N, int K, const void* x, long long ldx, int M, void* out,
                                      long long ldo, void* side, const void* norm_weight, int norm_weight_bf16, float* squares,
                                      int* status, cudaStream_t stream) {
    MLR_REQUIRE(side != nullptr && norm_weight != nullptr && squares != nullptr && reinterpret_cast<uintptr_t>(side) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(squares) % 16 == 0 && N % 8 == 0,
                "gemv_bf16: preparing a norm takes a side buffer, the norm's weight and room for the squares, 16-byte aligned");
    Link l = {static_cast<const __nv_bfloat16*>(W), ldw, N, K, x, ldx, 0, 0, nullptr, nullptr, 0.0f, kAddF32, out, ldo};
    l.side = static_cast<__nv_bfloat16*>(side);
    l.side_weight = norm_weight;
    l.side_weight_bf16 = norm_weight_bf16;
    l.squares = squares;
    return launch(l, M, status, stream);
}

MLR_API int mlr_gemv_bf16_prepared(const void* W, long long ldw, int N, int K, const void* side, const float* squares, float eps, int M,
                                   void* out, long long ldo, int mode, int* status, cudaStream_t stream) {
    MLR_REQUIRE(side != nullptr && squares != nullptr && reinterpret_cast<uintptr_t>(squares) % 16 == 0,
                "gemv_bf16: a prepared norm is a side buffer and its squares");
    Link l = {static_cast<const __nv_bfloat16*>(W), ldw, N, K, side, K, 2, 0, nullptr, nullptr, eps, mode, out, ldo};
    l.squares = const_cast<float*>(squares);
    l.n_squares = (K + kUnitRows - 1) / kUnitRows;
    return launch(l, M, status, stream);
}
