// The native step executor: a bound model as launch programs, and the one step function.
//
// The reference's step function and layer executor are C++ (src/minillm/cuda/runtime.cpp:146-254
// validates the batch, takes pages, uploads the step's metadata, enqueues the layers and publishes;
// src/minillm/cuda/layer.cpp:21-72 is the list of enqueues of one layer).  Here the list of enqueues
// is DATA: the Python parts of a model each emit their launches once, at bind time, into a program,
//
//     op  = { C entry point of a kernel module, its arguments }
//     arg = a constant (a size, a weight pointer, a workspace address) or a reference to something
//           only the step knows: its row count, the number of wanted rows, a section of the step's
//           metadata on the device, a block table, a field of an attention launch plan, the stream
//
// and `mlr_model_step` runs a step without the interpreter of the host language: it validates the
// entries, takes the cache pages (prepare), packs ids, positions, segment tables, wanted rows and block
// tables into one pinned buffer, plans the attention launches for the step's segments, uploads
// everything with one copy, walks the program (or replays the CUDA graph of a decode shape) and
// publishes lengths and page maps (commit).  Nothing is allocated on the way: workspace, metadata and
// logits buffers are handed in by the owner, and a step that needs more than they hold is refused with
// the sizes it needs.  A program serves a range of row counts within which every routing decision of
// its parts is the same; the owner builds one per range on first use.
//
// Failure rules (src/minillm/cuda/runtime.cpp:216-253): a step refused before device work changes
// nothing; one that fails after its first launch gives its pages back, and the model is poisoned:
// every later step is refused.
//
// Calling convention of an op: all arguments of the pointer/integer class in order, then (at most
// four) float arguments in order.  On x86-64 (System V) and AArch64 Linux the two classes are passed in
// separate register files, integer arguments beyond the registers go to 8-byte stack slots in order,
// and surplus arguments are ignored by the callee, so one function type calls every kernel entry
// point, whose parameters are pointers, `int`, `long long` and `float`.  A part may therefore bring a
// kernel module of its own without a change here.
#include <cuda_runtime.h>
#include <cublas_v2.h>

#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#if !defined(__x86_64__) && !defined(__aarch64__)
#error "the op calling convention of this file is written for x86-64 and AArch64 Linux"
#endif

extern "C" {
int mlr_cache_prepare(void* handle, int n, const int* slots, const int* new_tokens);
int mlr_cache_commit(void* handle);
int mlr_cache_discard(void* handle);
int mlr_cache_length(void* handle, int slot);
int mlr_cache_max_blocks(void* handle);
int mlr_cache_fill_table(void* handle, int group, int n, const int* slots, int columns, int32_t* out, int row_stride);
const char* mlr_cache_error(void* handle);
}

namespace {

// ---------------------------------------------------------------------------- programs
enum ArgKind : int32_t {
    kImm = 0,          // i
    kFloat = 1,        // f
    kRows = 2,         // rows of the step
    kWant = 3,         // rows whose logits are wanted
    kSegments = 4,     // requests in the step
    kMeta = 5,         // aux: section (0 ids, 1 positions, 2 segment_of_row, 3 segment_info, 4 slots, 5 wanted rows)
    kTable = 6,        // aux: cache group -> its block table rows on the device
    kTableStride = 7,  // columns of a table row
    kPlan = 8,         // aux: attention plan, i: field (PlanField)
    kStream = 9,
    kLogits = 10,      // where this step's logits go
};
enum PlanField : int64_t {
    kItems = 0, kItemCount = 1, kChunk = 2, kMaxSplits = 3, kScratch = 4, kCounters = 5,
    kTiles = 6, kTileCount = 7, kWideTiles = 8, kWideTileCount = 9,
    // derived: the split-KV items when the step has no prompt tiles / when it has some; the prompt tiles of both kinds
    kItemsAlone = 10, kItemsBeside = 11, kPromptTiles = 12,
};
enum Need : int32_t { kAlways = 0, kIfWanted = 1, kIfPlanField = 2 };

struct Arg {
    int32_t kind;
    int32_t aux;
    int64_t i;
    double f;
};
constexpr int kMaxArgs = 30;
struct Op {
    void* fn;                   // int fn(integer-class arguments..., float arguments...)
    void* error_text;           // const char* error_text(): the module's message after a non-zero return
    int32_t n_args;
    int32_t need;               // Need
    int32_t need_plan;          // for kIfPlanField
    int32_t need_field;
    Arg args[kMaxArgs];
};

struct PlanSpec {
    int32_t group;      // query heads per kv head
    int32_t kv_heads;
    int32_t window;     // 0: every key
    int32_t wide;       // 128-row tiles of the tcgen05 kernel may be used
    int32_t head_dim;
    int32_t small_ok;   // segments of few rows may take the split-KV kernel (bf16 tensor-core path)
};
struct PlanResult {
    int n_items = 0, items_offset = -1, chunk = 0, max_splits = 1;
    int n_tiles = 0, tiles_offset = -1, n_wide = 0, wide_offset = -1;
    long long scratch_floats = 0;
    int counters = 0;
};

struct Segment {
    int slot, start, count, row;
};

constexpr int kTile = 64, kWideTile = 128, kMinChunk = 128;

// Keys per split (a multiple of 64) and the number of splits for the split-KV kernel: the split
// count with the smallest estimated time.  `blocks_per_split` thread blocks run per split (items x kv
// heads); two blocks fit an SM; every block pays a fixed start and merge cost, and a partly filled last
// wave costs as much as a full one.
void split_plan(int longest, int blocks_per_split, int sm_count, int& chunk_out, int& splits_out) {
    const double slots = 2.0 * sm_count;
    const double per_key_ns = 0.022, per_block_ns = 5.0;
    const int limit = std::max(1, std::min(512, (longest + kMinChunk - 1) / kMinChunk));
    double best = -1.0;
    for (int splits = 1; splits <= limit; ++splits) {
        const int per = (longest + splits - 1) / splits;
        const int chunk = (per + kTile - 1) / kTile * kTile;
        const int real = (longest + chunk - 1) / chunk;
        const long long blocks = static_cast<long long>(real) * blocks_per_split;
        const long long waves = static_cast<long long>((blocks + slots - 1) / slots);
        const double share = std::min(1.0, blocks / slots / waves * 2.0);
        const double estimate = waves * (chunk * per_key_ns * std::max(share, 0.5) + per_block_ns);
        if (best < 0 || estimate < best - 1e-9) {
            best = estimate;
            chunk_out = chunk;
            splits_out = real;
        }
    }
}

// Which attention kernels a step launches for one (head grouping, window) and with what lists.
// Segments that bring at most 16 rows per kv head go to the split-KV kernel (`items`); the others are
// prompt portions: 128-row tiles while more than 64 rows are left (when `wide`), then 64-row tiles.
// `context_bound` > 0: the plan is for a CUDA graph that will be replayed with contexts up to the bound.
void plan_attention(const PlanSpec& spec, const std::vector<Segment>& segments, int context_bound, int sm_count,
                    PlanResult& out, std::vector<int32_t>& extra, int extra_base) {
    out = PlanResult();
    std::vector<int> small, large;
    for (int i = 0; i < static_cast<int>(segments.size()); ++i) {
        if (spec.small_ok && spec.group <= 16 && segments[i].count * spec.group <= 16) small.push_back(i);
        else large.push_back(i);
    }
    if (!small.empty()) {
        out.n_items = static_cast<int>(small.size());
        if (small.size() != segments.size()) {
            out.items_offset = extra_base + static_cast<int>(extra.size());
            for (int i : small) extra.push_back(i);
        }
        int longest = 0;
        for (int i : small) {
            const Segment& s = segments[i];
            int span;
            if (context_bound <= 0) {
                const int first = spec.window ? std::max(0, s.start - spec.window + 1) : 0;
                span = s.start + s.count - (first / kTile) * kTile;
            } else {
                span = spec.window ? std::min(context_bound, spec.window + s.count + kTile) : context_bound;
            }
            longest = std::max(longest, span);
        }
        split_plan(longest, out.n_items * spec.kv_heads, sm_count, out.chunk, out.max_splits);
        out.counters = out.n_items * spec.kv_heads;
        if (out.max_splits > 1)
            out.scratch_floats = static_cast<long long>(out.n_items) * spec.kv_heads * out.max_splits * 16 * (spec.head_dim + 2);
    }
    if (!large.empty()) {
        std::vector<std::pair<int, int>> tiles, wide;
        for (int i : large) {
            const int count = segments[i].count;
            int cut = 0;
            while (spec.wide && count - cut > kTile) {
                wide.push_back({i, cut});
                cut += kWideTile;
            }
            for (int t = cut; t < count; t += kTile) tiles.push_back({i, t});
        }
        auto longest_first = [&](const std::pair<int, int>& a, const std::pair<int, int>& b) {
            return segments[a.first].start + a.second > segments[b.first].start + b.second;
        };
        std::stable_sort(tiles.begin(), tiles.end(), longest_first);
        std::stable_sort(wide.begin(), wide.end(), longest_first);
        if (!tiles.empty()) {
            out.n_tiles = static_cast<int>(tiles.size());
            out.tiles_offset = extra_base + static_cast<int>(extra.size());
            for (auto& t : tiles) { extra.push_back(t.first); extra.push_back(t.second); }
        }
        if (!wide.empty()) {
            out.n_wide = static_cast<int>(wide.size());
            out.wide_offset = extra_base + static_cast<int>(extra.size());
            for (auto& t : wide) { extra.push_back(t.first); extra.push_back(t.second); }
        }
    }
}

// ---------------------------------------------------------------------------- errors, test hooks
thread_local char g_error[1024];
int fail(int code, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_error, sizeof(g_error), format, args);
    va_end(args);
    return code;
}

long long g_fail_after = -1;        // < 0: never; otherwise the launches still allowed before one is refused
long long g_launches = 0;           // ops launched by programs (graph replays count their captured ops)

// ---------------------------------------------------------------------------- the vendor library's product
struct Library {
    cublasHandle_t handle = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
};
std::mutex g_library_lock;
std::map<int, Library> g_libraries;     // by device

Library* library_for_current_device() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> guard(g_library_lock);
    Library& lib = g_libraries[device];
    if (lib.handle == nullptr) {
        if (cublasCreate(&lib.handle) != CUBLAS_STATUS_SUCCESS) {
            lib.handle = nullptr;
            return nullptr;
        }
        cublasSetMathMode(lib.handle, CUBLAS_DEFAULT_MATH);
    }
    return &lib;
}

// ---------------------------------------------------------------------------- the model
constexpr int kStepOk = 0, kStepRefused = 1, kStepNoPages = 2, kStepNeedsRoom = 3, kStepFailed = 4, kStepPoisoned = 5;
constexpr int kPinnedBuffers = 4;
constexpr int kMaxGroups = 16;

struct StepInfo {       // mirrored by the Python binding
    int32_t rows, want, graphed, captured;
    int64_t h2d_bytes, launches;
    // When the step was refused for lack of room (kStepNeedsRoom): what it needs.
    int64_t need_rows, need_want, need_meta_ints, need_scratch_floats, need_counters;
};

struct Program {
    int lo = 0, hi = 0;             // rows of a step it serves
    int want_lo = 0, want_hi = 0;   // wanted rows of a step it serves
    std::vector<Op> ops;
};

struct GraphEntry {
    cudaGraphExec_t exec = nullptr;
    cudaGraph_t graph = nullptr;
    long long launches = 0;
};

typedef void (*TableHook)(int group, int n, int columns, int32_t* rows);

struct Model {
    void* cache = nullptr;
    int n_groups = 0, page_size = 0, max_model_len = 0, vocab = 0, sm_count = 1;
    bool host_mode = false;             // no CUDA calls: the "device" buffers are host memory (tests of the host logic)
    std::vector<PlanSpec> plans;
    std::vector<Program> programs;
    // Room handed in by the owner.
    int32_t* device_meta = nullptr;
    long long device_meta_ints = 0;
    int32_t* pinned[kPinnedBuffers] = {};
    long long pinned_ints = 0;
    cudaEvent_t pinned_done[kPinnedBuffers] = {};
    int pinned_next = 0;
    float* logits = nullptr;
    long long logits_rows = 0;
    long long capacity_rows = 0;        // rows the programs' workspace is laid out for
    float* scratch = nullptr;
    long long scratch_floats = 0;
    int32_t* counters = nullptr;
    long long n_counters = 0;
    // Graphs of decode shapes.
    bool use_graphs = true;
    int graph_after = 2, max_graphs = 48, bucket_blocks = 64;
    std::map<std::pair<int, int>, GraphEntry> graphs;
    std::map<std::pair<int, int>, int> graph_uses;
    std::vector<std::pair<int, int>> graph_order;
    cudaStream_t capture_stream = nullptr;
    TableHook table_hook = nullptr;
    bool poisoned = false;
    std::string poison_reason;
};

struct StepVars {
    int rows = 0, want = 0, segments = 0, table_stride = 0;
    const int32_t* meta[6] = {};
    const int32_t* tables[kMaxGroups] = {};
    const int32_t* extra_base = nullptr;        // device address of element 0 of the metadata buffer
    std::vector<PlanResult> plans;
    float* logits = nullptr;
    float* scratch = nullptr;
    int32_t* counters = nullptr;
    cudaStream_t stream = nullptr;
};

int64_t resolve(const Arg& a, const StepVars& v) {
    switch (a.kind) {
        case kImm: return a.i;
        case kRows: return v.rows;
        case kWant: return v.want;
        case kSegments: return v.segments;
        case kMeta: return reinterpret_cast<int64_t>(v.meta[a.aux]);
        case kTable: return reinterpret_cast<int64_t>(v.tables[a.aux]);
        case kTableStride: return v.table_stride;
        case kStream: return reinterpret_cast<int64_t>(v.stream);
        case kLogits: return reinterpret_cast<int64_t>(v.logits);
        case kPlan: {
            const PlanResult& p = v.plans[a.aux];
            switch (a.i) {
                case kItems: return p.items_offset < 0 ? 0 : reinterpret_cast<int64_t>(v.extra_base + p.items_offset);
                case kItemCount: return p.n_items;
                case kChunk: return p.chunk;
                case kMaxSplits: return p.max_splits;
                case kScratch: return p.max_splits > 1 ? reinterpret_cast<int64_t>(v.scratch) : 0;
                case kCounters: return reinterpret_cast<int64_t>(v.counters);
                case kTiles: return p.tiles_offset < 0 ? 0 : reinterpret_cast<int64_t>(v.extra_base + p.tiles_offset);
                case kTileCount: return p.n_tiles;
                case kWideTiles: return p.wide_offset < 0 ? 0 : reinterpret_cast<int64_t>(v.extra_base + p.wide_offset);
                case kWideTileCount: return p.n_wide;
                case kItemsAlone: return p.n_tiles + p.n_wide == 0 ? p.n_items : 0;
                case kItemsBeside: return p.n_tiles + p.n_wide == 0 ? 0 : p.n_items;
                case kPromptTiles: return p.n_tiles + p.n_wide;
            }
            return 0;
        }
    }
    return 0;
}

using AnyKernel = int (*)(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                          int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                          int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, float, float, float, float);
using ErrorText = const char* (*)();

int run_op(const Op& op, const StepVars& v) {
    if (op.need == kIfWanted && v.want == 0) return 0;
    if (op.need == kIfPlanField) {
        Arg probe{kPlan, op.need_plan, op.need_field, 0.0};
        if (resolve(probe, v) == 0) return 0;
    }
    if (g_fail_after >= 0) {
        if (g_fail_after == 0) {
            g_fail_after = -1;
            return fail(kStepFailed, "injected failure in place of a launch");
        }
        --g_fail_after;
    }
    int64_t ints[kMaxArgs] = {};
    float floats[4] = {};
    int n_int = 0, n_float = 0;
    for (int k = 0; k < op.n_args; ++k) {
        const Arg& a = op.args[k];
        if (a.kind == kFloat) {
            if (n_float == 4) return fail(kStepFailed, "an op has more than four float arguments");
            floats[n_float++] = static_cast<float>(a.f);
        } else {
            ints[n_int++] = resolve(a, v);
        }
    }
    ++g_launches;
    const int rc = reinterpret_cast<AnyKernel>(op.fn)(
        ints[0], ints[1], ints[2], ints[3], ints[4], ints[5], ints[6], ints[7], ints[8], ints[9], ints[10], ints[11], ints[12], ints[13],
        ints[14], ints[15], ints[16], ints[17], ints[18], ints[19], ints[20], ints[21], ints[22], ints[23], ints[24], ints[25], ints[26],
        ints[27], ints[28], ints[29], floats[0], floats[1], floats[2], floats[3]);
    if (rc != 0) {
        const char* text = op.error_text ? reinterpret_cast<ErrorText>(op.error_text)() : "a kernel entry point refused its arguments";
        return fail(kStepFailed, "%s", text);
    }
    return 0;
}

int run_program(const Program& p, const StepVars& v) {
    for (const Op& op : p.ops)
        if (int rc = run_op(op, v)) return rc;
    return 0;
}

const Program* program_for(const Model& m, int rows, int want) {
    for (const Program& p : m.programs)
        if (rows >= p.lo && rows <= p.hi && want >= p.want_lo && want <= p.want_hi) return &p;
    return nullptr;
}

void drop_graphs(Model& m) {
    for (auto& kv : m.graphs) {
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
        if (kv.second.graph) cudaGraphDestroy(kv.second.graph);
    }
    m.graphs.clear();
    m.graph_order.clear();
}

int copy_to_device(Model& m, int buffer, long long ints, cudaStream_t stream) {
    if (m.host_mode) {
        std::memcpy(m.device_meta, m.pinned[buffer], sizeof(int32_t) * ints);
        return 0;
    }
    cudaError_t e = cudaMemcpyAsync(m.device_meta, m.pinned[buffer], sizeof(int32_t) * ints, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(m.pinned_done[buffer], stream);
    if (e != cudaSuccess) return fail(kStepFailed, "uploading the step's metadata failed: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace

extern "C" {

const char* mlr_exec_error() { return g_error; }
const char* mlr_last_error() { return g_error; }      // the name every kernel module gives its message function

// After `launches` more ops the next one is refused INSTEAD of being launched (< 0: never).  For
// failure tests that must not touch the GPU's health.
void mlr_exec_fail_after(long long launches) { g_fail_after = launches; }
long long mlr_exec_launch_count() { return g_launches; }
void mlr_exec_reset_launch_count() { g_launches = 0; }

// out[M, N] (+)= x[M, K] w[N, K]^T through the vendor library (the reference sends every product there:
// src/minillm/cuda/matrix.cpp:30-36).  bfloat16 operands, float32 accumulation; the result is bfloat16,
// or float32 (`out_f32`), in which case `accumulate` adds it to what `out` holds.
int mlr_library_gemm(const void* x, long long ldx, int M, const void* w, long long ldw, int N, int K, void* out, long long ldo,
                     int out_f32, int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return fail(1, "library_gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    if (accumulate && !out_f32) return fail(1, "library_gemm: only a float32 result can be added to");
    Library* lib = library_for_current_device();
    if (lib == nullptr) return fail(1, "library_gemm: the vendor library could not be initialised");
    cublasStatus_t s = cublasSetStream(lib->handle, stream);
    if (s == CUBLAS_STATUS_SUCCESS && lib->workspace != nullptr) s = cublasSetWorkspace(lib->handle, lib->workspace, lib->workspace_bytes);
    const float alpha = 1.0f, beta = accumulate ? 1.0f : 0.0f;
    // Row-major out = x w^T is column-major out^T[N, M] = w^T' x': the weights transposed, x as it is.
    if (s == CUBLAS_STATUS_SUCCESS)
        s = cublasGemmEx(lib->handle, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, static_cast<int>(ldw), x, CUDA_R_16BF,
                         static_cast<int>(ldx), &beta, out, out_f32 ? CUDA_R_32F : CUDA_R_16BF, static_cast<int>(ldo), CUBLAS_COMPUTE_32F,
                         CUBLAS_GEMM_DEFAULT);
    if (s != CUBLAS_STATUS_SUCCESS) return fail(1, "library_gemm: the vendor library returned status %d", static_cast<int>(s));
    return 0;
}

// Workspace of the vendor library on the current device (so that it allocates none of its own, which a
// CUDA graph capture would not allow).
int mlr_library_set_workspace(void* workspace, long long bytes) {
    Library* lib = library_for_current_device();
    if (lib == nullptr) return fail(1, "the vendor library could not be initialised");
    lib->workspace = workspace;
    lib->workspace_bytes = static_cast<size_t>(bytes);
    return 0;
}

// Plans the attention launches of a step outside a model (the Python step path of models with parts
// that are not compiled into programs uses the same planner).  segments: n x {start, count}.
// out: {n_items, items_offset, chunk, max_splits, n_tiles, tiles_offset, n_wide, wide_offset, counters}
// plus scratch floats; lists go to `extra` (capacity `extra_capacity` ints, used count returned in *extra_used),
// offsets are relative to `extra`.
int mlr_plan_attention(const int32_t* spec6, int n, const int32_t* starts, const int32_t* counts, int context_bound, int sm_count,
                       int32_t* out9, long long* scratch_floats, int32_t* extra, int extra_capacity, int* extra_used) {
    PlanSpec spec{spec6[0], spec6[1], spec6[2], spec6[3], spec6[4], spec6[5]};
    std::vector<Segment> segments(static_cast<size_t>(n));
    int row = 0;
    for (int i = 0; i < n; ++i) {
        segments[i] = {i, starts[i], counts[i], row};
        row += counts[i];
    }
    PlanResult r;
    std::vector<int32_t> lists;
    plan_attention(spec, segments, context_bound, sm_count, r, lists, 0);
    if (static_cast<int>(lists.size()) > extra_capacity) return fail(1, "plan_attention: the lists need %zu ints", lists.size());
    std::copy(lists.begin(), lists.end(), extra);
    *extra_used = static_cast<int>(lists.size());
    const int32_t values[9] = {r.n_items, r.items_offset, r.chunk, r.max_splits, r.n_tiles, r.tiles_offset, r.n_wide, r.wide_offset, r.counters};
    std::copy(values, values + 9, out9);
    *scratch_floats = r.scratch_floats;
    return 0;
}

// How many ranges to cut K into when a weight matrix of `rows` rows is streamed in tiles of 128 rows by
// `sms` blocks at a time: the smallest count whose units fill whole rounds to 93 % or better, with at
// least four 64-wide blocks of K per range and at most 16 ranges.
int mlr_k_splits(int rows, int K, int sms) {
    const int tiles = (rows + 127) / 128;
    int best = 1;
    double best_fill = 0.0;
    for (int s = 1; s <= 16; ++s) {
        if (s > 1 && ((K + 63) / 64) / s < 4) break;
        const long long units = static_cast<long long>(tiles) * s;
        const double fill = static_cast<double>(units) / (static_cast<double>(sms) * ((units + sms - 1) / sms));
        if (fill > best_fill + 1e-9) {
            best = s;
            best_fill = fill;
        }
        if (fill >= 0.93) return s;
    }
    return best;
}

// ---------------------------------------------------------------------------- model handle
void* mlr_model_create(void* cache, int n_groups, int page_size, int max_model_len, int vocab, int sm_count, int host_mode) {
    if (cache == nullptr || n_groups < 0 || n_groups > kMaxGroups || page_size <= 0 || max_model_len <= 0 || vocab <= 0) {
        fail(1, "model_create: bad arguments");
        return nullptr;
    }
    Model* m = new Model();
    m->cache = cache;
    m->n_groups = n_groups;
    m->page_size = page_size;
    m->max_model_len = max_model_len;
    m->vocab = vocab;
    m->sm_count = sm_count > 0 ? sm_count : 1;
    m->host_mode = host_mode != 0;
    m->bucket_blocks = std::max(1, 1024 / page_size);
    return m;
}

void mlr_model_destroy(void* handle) {
    Model* m = static_cast<Model*>(handle);
    if (m == nullptr) return;
    if (!m->host_mode) {
        drop_graphs(*m);
        for (auto& e : m->pinned_done)
            if (e) cudaEventDestroy(e);
        if (m->capture_stream) cudaStreamDestroy(m->capture_stream);
    }
    delete m;
}

int mlr_model_add_plan(void* handle, const int32_t* spec6) {
    Model* m = static_cast<Model*>(handle);
    m->plans.push_back(PlanSpec{spec6[0], spec6[1], spec6[2], spec6[3], spec6[4], spec6[5]});
    return static_cast<int>(m->plans.size()) - 1;
}

// The room a step may use; any change invalidates programs (their workspace addresses) and graphs.
int mlr_model_set_room(void* handle, int32_t* device_meta, long long device_meta_ints, int32_t* const* pinned, long long pinned_ints,
                       float* logits, long long logits_rows, long long capacity_rows, float* scratch, long long scratch_floats,
                       int32_t* counters, long long n_counters) {
    Model* m = static_cast<Model*>(handle);
    if (!m->host_mode) drop_graphs(*m);      // they hold the old addresses; how often a shape has come is still true
    m->device_meta = device_meta;
    m->device_meta_ints = device_meta_ints;
    for (int i = 0; i < kPinnedBuffers; ++i) m->pinned[i] = pinned[i];
    m->pinned_ints = pinned_ints;
    m->logits = logits;
    m->logits_rows = logits_rows;
    m->capacity_rows = capacity_rows;
    m->scratch = scratch;
    m->scratch_floats = scratch_floats;
    m->counters = counters;
    m->n_counters = n_counters;
    if (!m->host_mode) {
        for (auto& e : m->pinned_done) {
            if (e == nullptr && cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess)
                return fail(1, "model_set_room: cannot create an event");
        }
    }
    return 0;
}

void mlr_model_clear_programs(void* handle) {
    Model* m = static_cast<Model*>(handle);
    if (!m->host_mode) drop_graphs(*m);
    m->graph_uses.clear();
    m->programs.clear();
}

int mlr_model_add_program(void* handle, int lo, int hi, int want_lo, int want_hi, const Op* ops, int n_ops) {
    Model* m = static_cast<Model*>(handle);
    if (lo < 1 || hi < lo || want_lo < 0 || want_hi < want_lo || n_ops < 0) return fail(1, "model_add_program: bad range or op count");
    // An overlap with an older program is harmless (the first match serves a step), but an identical
    // range would mean the owner builds the same program again and again.
    for (const Program& p : m->programs)
        if (p.lo == lo && p.hi == hi && p.want_lo == want_lo && p.want_hi == want_hi)
            return fail(1, "model_add_program: rows %d..%d with %d..%d wanted rows have a program already", lo, hi, want_lo, want_hi);
    for (int i = 0; i < n_ops; ++i) {
        if (ops[i].fn == nullptr || ops[i].n_args < 0 || ops[i].n_args > kMaxArgs) return fail(1, "model_add_program: op %d is malformed", i);
        for (int k = 0; k < ops[i].n_args; ++k) {
            const Arg& a = ops[i].args[k];
            if ((a.kind == kMeta && (a.aux < 0 || a.aux > 5)) || (a.kind == kTable && (a.aux < 0 || a.aux >= m->n_groups)) ||
                (a.kind == kPlan && (a.aux < 0 || a.aux >= static_cast<int>(m->plans.size()))) || a.kind < kImm || a.kind > kLogits)
                return fail(1, "model_add_program: op %d argument %d refers to something the model does not have", i, k);
        }
    }
    Program p;
    p.lo = lo;
    p.hi = hi;
    p.want_lo = want_lo;
    p.want_hi = want_hi;
    p.ops.assign(ops, ops + n_ops);
    m->programs.push_back(std::move(p));
    return 0;
}

int mlr_model_has_program(void* handle, int rows, int want) {
    return program_for(*static_cast<Model*>(handle), rows, want) != nullptr;
}

void mlr_model_set_graphs(void* handle, int use_graphs, int graph_after, int bucket_blocks, int max_graphs) {
    Model* m = static_cast<Model*>(handle);
    m->use_graphs = use_graphs != 0;
    if (graph_after >= 0) m->graph_after = graph_after;
    if (bucket_blocks > 0) m->bucket_blocks = bucket_blocks;
    if (max_graphs > 0) m->max_graphs = max_graphs;
}
int mlr_model_graph_count(void* handle) { return static_cast<int>(static_cast<Model*>(handle)->graphs.size()); }
void mlr_model_set_table_hook(void* handle, TableHook hook) { static_cast<Model*>(handle)->table_hook = hook; }
int mlr_model_poisoned(void* handle) { return static_cast<Model*>(handle)->poisoned ? 1 : 0; }
const char* mlr_model_poison_reason(void* handle) { return static_cast<Model*>(handle)->poison_reason.c_str(); }
void mlr_model_poison(void* handle, const char* why) {
    Model* m = static_cast<Model*>(handle);
    if (!m->poisoned) {
        m->poisoned = true;
        m->poison_reason = why ? why : "";
    }
}

// The step function.  Entry i is request `slots[i]` with its next `counts[i]` tokens; `tokens` holds all
// rows' ids in entry order (host memory; may be null when `device_tokens`, one int32 per row on the
// device, supplies them); entry i wants logits at `want_places[want_offsets[i] .. want_offsets[i+1])`
// among its tokens.  The logits [wanted, vocab] go to the room's logits buffer.  Returns a kStep* code;
// mlr_exec_error() has the message.
int mlr_model_step(void* handle, int n, const int32_t* slots, const int32_t* counts, const int32_t* tokens, const int32_t* want_offsets,
                   const int32_t* want_places, const int32_t* device_tokens, cudaStream_t stream, StepInfo* info) {
    Model& m = *static_cast<Model*>(handle);
    std::memset(info, 0, sizeof(*info));
    if (m.poisoned) return fail(kStepPoisoned, "the model is poisoned and must not be used further (%s)", m.poison_reason.c_str());
    if (n <= 0) return fail(kStepRefused, "a step needs at least one entry");
    // ---- validate; nothing has changed yet
    std::vector<Segment> segments(static_cast<size_t>(n));
    int rows = 0;
    bool all_single = true;
    for (int i = 0; i < n; ++i) {
        if (counts[i] <= 0) return fail(kStepRefused, "the entry of slot %d has no tokens", slots[i]);
        for (int j = 0; j < i; ++j)
            if (slots[j] == slots[i]) return fail(kStepRefused, "slot %d appears twice in one step", slots[i]);
        const int start = mlr_cache_length(m.cache, slots[i]);
        if (start < 0) return fail(kStepRefused, "slot %d is not open", slots[i]);
        if (start + counts[i] > m.max_model_len)
            return fail(kStepRefused, "slot %d would hold %d tokens, the limit is %d", slots[i], start + counts[i], m.max_model_len);
        for (int w = want_offsets[i]; w < want_offsets[i + 1]; ++w)
            if (want_places[w] < 0 || want_places[w] >= counts[i])
                return fail(kStepRefused, "slot %d wants logits at place %d of %d tokens", slots[i], want_places[w], counts[i]);
        segments[i] = {slots[i], start, counts[i], rows};
        rows += counts[i];
        all_single = all_single && counts[i] == 1;
    }
    const int want = want_offsets[n];
    if (tokens != nullptr && device_tokens == nullptr)
        for (int r = 0; r < rows; ++r)
            if (tokens[r] < 0 || tokens[r] >= m.vocab) return fail(kStepRefused, "a token id is outside the vocabulary of %d", m.vocab);
    if (tokens == nullptr && device_tokens == nullptr) return fail(kStepRefused, "a step needs token ids, on the host or on the device");
    const Program* program = program_for(m, rows, want);
    info->rows = rows;
    info->want = want;
    // ---- what the step will launch, and whether the room holds it
    int max_context = 0;
    for (const Segment& s : segments) max_context = std::max(max_context, s.start + s.count);
    int columns = (max_context + m.page_size - 1) / m.page_size;
    const int max_blocks = mlr_cache_max_blocks(m.cache);
    bool graphed = m.use_graphs && !m.host_mode && all_single && want == rows;
    std::pair<int, int> key{rows, 0};
    if (graphed) {
        const int bucketed = std::min((columns + m.bucket_blocks - 1) / m.bucket_blocks * m.bucket_blocks, max_blocks);
        key.second = bucketed;
        const int seen = m.graph_uses[key]++;
        graphed = m.graphs.count(key) != 0 || seen >= m.graph_after;
        if (graphed) columns = bucketed;
    }
    const int context_bound = graphed ? columns * m.page_size : 0;
    std::vector<int32_t> extra;
    const long long fixed_ints = 3LL * rows + 4LL * n + n + want + static_cast<long long>(m.n_groups) * n * columns;
    StepVars vars;
    vars.plans.resize(m.plans.size());
    long long scratch_need = 0, counters_need = 0;
    for (size_t p = 0; p < m.plans.size(); ++p) {
        plan_attention(m.plans[p], segments, context_bound, m.sm_count, vars.plans[p], extra, static_cast<int>(fixed_ints));
        scratch_need = std::max(scratch_need, vars.plans[p].scratch_floats);
        counters_need = std::max<long long>(counters_need, vars.plans[p].counters);
    }
    const long long total_ints = fixed_ints + static_cast<long long>(extra.size());
    if (program == nullptr || rows > m.capacity_rows || want > m.logits_rows || total_ints > m.device_meta_ints ||
        total_ints > m.pinned_ints || scratch_need > m.scratch_floats || counters_need > m.n_counters) {
        if (graphed && m.graphs.count(key) == 0) --m.graph_uses[key];
        info->need_rows = rows;
        info->need_want = want;
        info->need_meta_ints = total_ints;
        info->need_scratch_floats = scratch_need;
        info->need_counters = counters_need;
        return fail(kStepNeedsRoom, "the step needs a program for %d rows, %d logits rows, %lld metadata ints, %lld scratch floats", rows,
                    want, total_ints, scratch_need);
    }
    // ---- take the pages
    {
        const int rc = mlr_cache_prepare(m.cache, n, slots, counts);
        if (rc == 2) return fail(kStepNoPages, "%s", mlr_cache_error(m.cache));
        if (rc != 0) return fail(kStepRefused, "%s", mlr_cache_error(m.cache));
    }
    // ---- pack the metadata (still nothing on the device)
    const int buffer = m.pinned_next;
    m.pinned_next = (m.pinned_next + 1) % kPinnedBuffers;
    if (!m.host_mode && m.pinned_done[buffer] != nullptr) cudaEventSynchronize(m.pinned_done[buffer]);
    int32_t* host = m.pinned[buffer];
    long long offset[7 + kMaxGroups];
    offset[0] = 0;
    offset[1] = rows;
    offset[2] = 2LL * rows;
    offset[3] = 3LL * rows;
    offset[4] = offset[3] + 4LL * n;
    offset[5] = offset[4] + n;
    offset[6] = offset[5] + want;
    for (int g = 0; g < m.n_groups; ++g) offset[7 + g] = offset[6 + g] + static_cast<long long>(n) * columns;
    if (tokens != nullptr) std::memcpy(host, tokens, sizeof(int32_t) * rows);
    else std::memset(host, 0, sizeof(int32_t) * rows);
    int want_at = 0;
    for (int i = 0; i < n; ++i) {
        const Segment& s = segments[i];
        for (int r = 0; r < s.count; ++r) {
            host[offset[1] + s.row + r] = s.start + r;
            host[offset[2] + s.row + r] = i;
        }
        int32_t* row_info = host + offset[3] + 4LL * i;
        row_info[0] = s.row;
        row_info[1] = s.count;
        row_info[2] = s.start;
        row_info[3] = s.slot;
        host[offset[4] + i] = s.slot;
        for (int w = want_offsets[i]; w < want_offsets[i + 1]; ++w) host[offset[5] + want_at++] = s.row + want_places[w];
    }
    int failure = 0;
    for (int g = 0; g < m.n_groups && !failure; ++g) {
        int32_t* table = host + offset[6 + g];
        if (graphed) std::fill(table, table + static_cast<long long>(n) * columns, -1);
        const int filled = std::min(columns, max_blocks);
        if (mlr_cache_fill_table(m.cache, g, n, slots, filled, table, columns) != 0)
            failure = fail(kStepRefused, "%s", mlr_cache_error(m.cache));
        else if (m.table_hook != nullptr)
            m.table_hook(g, n, columns, table);
    }
    if (failure) {
        mlr_cache_discard(m.cache);
        return failure;
    }
    std::copy(extra.begin(), extra.end(), host + fixed_ints);
    // ---- device work begins
    vars.rows = rows;
    vars.want = want;
    vars.segments = n;
    vars.table_stride = columns;
    for (int k = 0; k < 6; ++k) vars.meta[k] = m.device_meta + offset[k];
    for (int g = 0; g < m.n_groups; ++g) vars.tables[g] = m.device_meta + offset[6 + g];
    vars.extra_base = m.device_meta;
    vars.logits = m.logits;
    vars.scratch = m.scratch;
    vars.counters = m.counters;
    vars.stream = stream;
    info->h2d_bytes = 4 * total_ints;
    info->graphed = graphed ? 1 : 0;
    const long long launches_before = g_launches;
    int rc = copy_to_device(m, buffer, total_ints, stream);
    if (rc == 0 && device_tokens != nullptr && !m.host_mode) {
        const cudaError_t e = cudaMemcpyAsync(m.device_meta, device_tokens, sizeof(int32_t) * rows, cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) rc = fail(kStepFailed, "copying the token ids on the device failed: %s", cudaGetErrorString(e));
    }
    if (rc == 0 && graphed) {
        auto found = m.graphs.find(key);
        if (found == m.graphs.end()) {
            // Warm-up outside the capture (the step is idempotent: it rewrites the same cache rows), then the capture.
            rc = run_program(*program, vars);
            if (rc == 0 && m.capture_stream == nullptr && cudaStreamCreateWithFlags(&m.capture_stream, cudaStreamNonBlocking) != cudaSuccess)
                rc = fail(kStepFailed, "cannot create the capture stream");
            GraphEntry entry;
            if (rc == 0) {
                StepVars captured = vars;
                captured.stream = m.capture_stream;
                const long long before = g_launches;
                cudaError_t e = cudaStreamBeginCapture(m.capture_stream, cudaStreamCaptureModeThreadLocal);
                if (e != cudaSuccess) rc = fail(kStepFailed, "cannot begin a graph capture: %s", cudaGetErrorString(e));
                if (rc == 0) {
                    const int run = run_program(*program, captured);
                    e = cudaStreamEndCapture(m.capture_stream, &entry.graph);
                    if (run != 0) rc = run;
                    else if (e != cudaSuccess) rc = fail(kStepFailed, "the graph capture failed: %s", cudaGetErrorString(e));
                }
                if (rc == 0) {
                    e = cudaGraphInstantiate(&entry.exec, entry.graph, 0);
                    if (e != cudaSuccess) rc = fail(kStepFailed, "cannot instantiate the graph: %s", cudaGetErrorString(e));
                }
                entry.launches = g_launches - before;
                g_launches = before;
            }
            if (rc == 0) {
                if (static_cast<int>(m.graphs.size()) >= m.max_graphs && !m.graph_order.empty()) {
                    auto oldest = m.graphs.find(m.graph_order.front());
                    if (oldest != m.graphs.end()) {
                        cudaGraphExecDestroy(oldest->second.exec);
                        cudaGraphDestroy(oldest->second.graph);
                        m.graphs.erase(oldest);
                    }
                    m.graph_order.erase(m.graph_order.begin());
                }
                found = m.graphs.emplace(key, entry).first;
                m.graph_order.push_back(key);
                info->captured = 1;
            } else {
                if (entry.exec) cudaGraphExecDestroy(entry.exec);
                if (entry.graph) cudaGraphDestroy(entry.graph);
            }
        }
        if (rc == 0) {
            const cudaError_t e = cudaGraphLaunch(found->second.exec, stream);
            if (e != cudaSuccess) rc = fail(kStepFailed, "launching the graph failed: %s", cudaGetErrorString(e));
            else g_launches += found->second.launches;
        }
    } else if (rc == 0) {
        rc = run_program(*program, vars);
    }
    info->launches = g_launches - launches_before;
    if (rc != 0) {
        // Device work had begun: the ledger is rolled back and the model refuses everything from now on.
        const std::string why = std::string("a step failed after its device work had begun: ") + g_error;
        mlr_cache_discard(m.cache);
        m.poisoned = true;
        m.poison_reason = why;
        return fail(kStepFailed, "%s", why.c_str());
    }
    // Lengths and page maps are published when the work is enqueued, so that the next step can be
    // launched behind it; a fault a kernel reports in the status word is read with the step's results
    // and poisons the model before a token of that step is handed out.
    mlr_cache_commit(m.cache);
    return kStepOk;
}

// For tests of the host logic: an op target that writes its first `count` integer arguments and its
// first float argument to a log.
static std::vector<int64_t> g_recorded;
int mlr_test_record(int64_t a0, int64_t a1, int64_t a2, int64_t a3, int64_t a4, int64_t a5, int64_t a6, int64_t a7, float f0) {
    const int64_t values[8] = {a0, a1, a2, a3, a4, a5, a6, a7};
    g_recorded.insert(g_recorded.end(), values, values + 8);
    g_recorded.push_back(static_cast<int64_t>(f0 * 1000.0f));
    return a0 == -7 ? 1 : 0;          // a first argument of -7 makes the "launch" fail
}
const char* mlr_test_record_error() { return "the recording op was told to fail"; }
long long mlr_test_recorded(int64_t* out, long long capacity) {
    const long long n = std::min<long long>(capacity, static_cast<long long>(g_recorded.size()));
    std::copy(g_recorded.begin(), g_recorded.begin() + n, out);
    const long long total = static_cast<long long>(g_recorded.size());
    g_recorded.clear();
    return total;
}

}  // extern "C"
