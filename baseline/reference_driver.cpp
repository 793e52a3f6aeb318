// Drives the UNMODIFIED CUDA runtime of lilong555/mini-llm-runtime (src/minillm/cuda/*.cpp, *.cu,
// compiled from copies of its files) through its own public API, minillm::cuda::CudaRuntime
// (include/minillm/cuda/runtime.h:85-106), for the reference arm of bench.py.  Nothing of
// mini-llm-runtime_b200 is linked or loaded here.
//
// Two classes of the reference need llama.cpp, which its checkout does not carry
// (third_party/ is absent): minillm::GgufModel and minillm::Tokenizer.  They are replaced by
// stand-ins with the same interface (include/minillm/gguf_model.h:23-42, tokenizer.h:14-29):
// the model stand-in MAKES a Qwen3 model of the requested sizes in memory, float32 weights
// from a seeded generator (matrices about N(0, 0.02), norm weights about 1), instead of
// reading a GGUF file; the tokenizer stand-in knows the vocabulary size and nothing else.
// The model "path" carries the sizes:  synthetic:H:L:Hq:Hkv:D:I:V:CTX:SEED:TIED
//
// Workloads, all at the reference's own limits (4 sequences, 2048 positions, 128 rows a step,
// float32 products: include/minillm/cuda/runtime.h:18-23, include/minillm/cuda/kv_layout.h:29-31):
//   decode   S sequences are filled to `context - steps - warmup` tokens in portions of 128, then
//            `warmup` untimed and `steps` timed forwards of S rows each (one token a sequence)
//   prefill  one sequence, 128 tokens in one forward, repeated
// Each forward is the reference's host-synchronous step (it uploads the rows, runs, reads the ids
// back and synchronises), timed with the host clock around the call and with its own CUDA events.
// Output: one JSON object on standard output.
#include "minillm/cuda/runtime.h"
#include "minillm/gguf_model.h"
#include "minillm/tokenizer.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace minillm {

namespace {
struct Sizes {
    std::size_t H, L, Hq, Hkv, D, I, V, context, seed, tied;
};
Sizes parse_sizes(const std::string& path) {
    if (path.rfind("synthetic:", 0) != 0) throw std::runtime_error("the stand-in model wants a path synthetic:H:L:Hq:Hkv:D:I:V:CTX:SEED:TIED");
    std::vector<std::size_t> v;
    std::stringstream in(path.substr(10));
    std::string item;
    while (std::getline(in, item, ':')) v.push_back(static_cast<std::size_t>(std::stoull(item)));
    if (v.size() != 10) throw std::runtime_error("the stand-in model wants ten sizes");
    return {v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9]};
}
// xorshift64* and the sum of four uniforms: close enough to a normal for weights.
struct Generator {
    std::uint64_t s;
    explicit Generator(std::uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x2545F4914F6CDD1Dull) {}
    float uniform() {
        s ^= s >> 12;
        s ^= s << 25;
        s ^= s >> 27;
        return static_cast<float>((s * 0x2545F4914F6CDD1Dull) >> 40) * (1.0f / 16777216.0f);
    }
    float normal() { return (uniform() + uniform() + uniform() + uniform() - 2.0f) * 1.7320508f; }
};
}  // namespace

struct GgufModel::Impl {
    Sizes sizes;
    struct Tensor {
        std::size_t rows, columns;
        std::vector<float> data;
    };
    std::map<std::string, Tensor> tensors;
    std::map<std::string, std::uint64_t> integers;
    std::map<std::string, float> floats;
    std::size_t bytes = 0;
    void add(const std::string& name, std::size_t rows, std::size_t columns, bool norm, std::uint64_t seed) {
        Tensor t{rows, columns, {}};
        t.data.resize(rows * columns);
        Generator g(seed);
        for (auto& x : t.data) x = norm ? 1.0f + 0.01f * g.normal() : 0.02f * g.normal();
        bytes += t.data.size() * 4;
        tensors.emplace(name, std::move(t));
    }
};

GgufModel::GgufModel(const std::string& path) : impl_(std::make_unique<Impl>()) {
    const Sizes z = parse_sizes(path);
    impl_->sizes = z;
    impl_->integers = {{"qwen3.embedding_length", z.H}, {"qwen3.block_count", z.L}, {"qwen3.attention.head_count", z.Hq},
                       {"qwen3.attention.head_count_kv", z.Hkv}, {"qwen3.attention.key_length", z.D},
                       {"qwen3.attention.value_length", z.D}, {"qwen3.feed_forward_length", z.I},
                       {"qwen3.context_length", z.context}};
    impl_->floats = {{"qwen3.attention.layer_norm_rms_epsilon", 1e-6f}, {"qwen3.rope.freq_base", 1000000.0f}};
    std::uint64_t n = z.seed * 1000003ull;
    impl_->add("token_embd.weight", z.V, z.H, false, ++n);
    impl_->add("output_norm.weight", 1, z.H, true, ++n);
    if (!z.tied) impl_->add("output.weight", z.V, z.H, false, ++n);
    for (std::size_t i = 0; i < z.L; ++i) {
        const std::string p = "blk." + std::to_string(i) + ".";
        impl_->add(p + "attn_norm.weight", 1, z.H, true, ++n);
        impl_->add(p + "attn_q.weight", z.Hq * z.D, z.H, false, ++n);
        impl_->add(p + "attn_k.weight", z.Hkv * z.D, z.H, false, ++n);
        impl_->add(p + "attn_v.weight", z.Hkv * z.D, z.H, false, ++n);
        impl_->add(p + "attn_q_norm.weight", 1, z.D, true, ++n);
        impl_->add(p + "attn_k_norm.weight", 1, z.D, true, ++n);
        impl_->add(p + "attn_output.weight", z.H, z.Hq * z.D, false, ++n);
        impl_->add(p + "ffn_norm.weight", 1, z.H, true, ++n);
        impl_->add(p + "ffn_gate.weight", z.I, z.H, false, ++n);
        impl_->add(p + "ffn_up.weight", z.I, z.H, false, ++n);
        impl_->add(p + "ffn_down.weight", z.H, z.I, false, ++n);
    }
}
GgufModel::~GgufModel() = default;
std::string GgufModel::string_value(const std::string& key) const {
    if (key == "general.architecture") return "qwen3";
    throw std::out_of_range("the stand-in model has no string " + key);
}
std::uint64_t GgufModel::integer_value(const std::string& key) const { return impl_->integers.at(key); }
float GgufModel::float_value(const std::string& key) const { return impl_->floats.at(key); }
bool GgufModel::contains(const std::string& key) const {
    return key == "general.architecture" || impl_->integers.count(key) || impl_->floats.count(key);
}
bool GgufModel::has_tensor(const std::string& name) const { return impl_->tensors.count(name) != 0; }
TensorView GgufModel::tensor(const std::string& name) const {
    const auto found = impl_->tensors.find(name);
    if (found == impl_->tensors.end()) throw std::runtime_error("missing GGUF tensor: " + name);
    const auto& t = found->second;
    return {reinterpret_cast<const std::byte*>(t.data.data()), WeightType::f32, t.columns, t.rows, t.columns * 4};
}
std::size_t GgufModel::tensor_count() const { return impl_->tensors.size(); }
std::size_t GgufModel::file_bytes() const { return impl_->bytes; }
std::uint32_t GgufModel::version() const { return 3; }

const std::byte* TensorView::row(std::size_t index) const {
    if (index >= rows) throw std::out_of_range("tensor row index");
    return data + index * stride;
}
std::vector<float> TensorView::vector() const {
    if (rows != 1) throw std::runtime_error("expected a one-dimensional tensor");
    std::vector<float> values(columns);
    decode_row(type, data, values.data(), columns);
    return values;
}

struct Tokenizer::Impl {
    std::size_t vocabulary;
};
Tokenizer::Tokenizer(const std::string&, std::size_t expected) : impl_(std::make_unique<Impl>(Impl{expected})) {}
Tokenizer::~Tokenizer() = default;
std::size_t Tokenizer::vocabulary_size() const noexcept { return impl_->vocabulary; }
std::vector<std::int32_t> Tokenizer::tokenize(std::string_view) const { return {}; }
std::string Tokenizer::token_piece(std::int32_t) const { return {}; }
bool Tokenizer::is_eog(std::int32_t) const { return false; }

}  // namespace minillm

namespace {
using Clock = std::chrono::steady_clock;
double ms_since(Clock::time_point start) { return std::chrono::duration<double, std::milli>(Clock::now() - start).count(); }

struct Timing {
    double wall_ms = 0, device_ms = 0;
    int forwards = 0;
};

// `sequences` requests at `context` tokens: fill, warm up, then time `steps` decode forwards.
Timing decode(minillm::cuda::CudaRuntime& runtime, int sequences, int context, int steps, int warmup, std::size_t vocab,
              std::vector<std::int32_t>& last_tokens) {
    const int filled = context - steps - warmup;
    if (filled < 1) throw std::invalid_argument("context too short for the steps asked for");
    std::uint64_t s = 88172645463325252ull;
    auto next_token = [&] {
        s ^= s << 13;
        s ^= s >> 7;
        s ^= s << 17;
        return static_cast<std::int32_t>(s % vocab);
    };
    for (int seq = 0; seq < sequences; ++seq) {
        runtime.clear_sequence(seq);
        for (int begin = 0; begin < filled; begin += 128) {
            std::vector<minillm::InputToken> batch;
            for (int p = begin; p < std::min(filled, begin + 128); ++p) batch.push_back({next_token(), p, seq, false});
            runtime.forward(batch);
        }
    }
    Timing t;
    last_tokens.assign(static_cast<std::size_t>(sequences), 1);
    for (int step = 0; step < warmup + steps; ++step) {
        std::vector<minillm::InputToken> batch;
        for (int seq = 0; seq < sequences; ++seq) batch.push_back({last_tokens[static_cast<std::size_t>(seq)], filled + step, seq, true});
        const auto start = Clock::now();
        const auto result = runtime.forward(batch, minillm::cuda::CudaOutputMode::greedy, true);
        const double wall = ms_since(start);
        for (const auto& sample : result.samples) last_tokens[static_cast<std::size_t>(sample.sequence)] = sample.token;
        if (step >= warmup) {
            t.wall_ms += wall;
            t.device_ms += result.device_elapsed_ms.value_or(0.0);
            ++t.forwards;
        }
    }
    for (int seq = 0; seq < sequences; ++seq) runtime.clear_sequence(seq);
    return t;
}

Timing prefill(minillm::cuda::CudaRuntime& runtime, int tokens, int repeats, int warmup, std::size_t vocab) {
    Timing t;
    for (int r = 0; r < warmup + repeats; ++r) {
        runtime.clear_sequence(0);
        std::vector<minillm::InputToken> batch;
        for (int p = 0; p < tokens; ++p) batch.push_back({static_cast<std::int32_t>((p * 7919 + r) % static_cast<int>(vocab)), p, 0, p + 1 == tokens});
        const auto start = Clock::now();
        const auto result = runtime.forward(batch, minillm::cuda::CudaOutputMode::greedy, true);
        const double wall = ms_since(start);
        if (r >= warmup) {
            t.wall_ms += wall;
            t.device_ms += result.device_elapsed_ms.value_or(0.0);
            ++t.forwards;
        }
    }
    runtime.clear_sequence(0);
    return t;
}
}  // namespace

// usage: ref_bench MODEL_SPEC STEPS WARMUP CONTEXT BATCH
int main(int argc, char** argv) {
    if (argc != 6) {
        std::fprintf(stderr, "usage: ref_bench synthetic:H:L:Hq:Hkv:D:I:V:CTX:SEED:TIED STEPS WARMUP CONTEXT BATCH\n");
        return 2;
    }
    try {
        const int steps = std::atoi(argv[2]), warmup = std::atoi(argv[3]), context = std::atoi(argv[4]), batch = std::atoi(argv[5]);
        minillm::cuda::CudaRuntimeConfig config;
        config.model_path = argv[1];
        config.max_sequences = 4;
        config.max_model_len = static_cast<std::size_t>(context);
        config.batch_tokens = 128;
        const auto load_start = Clock::now();
        minillm::cuda::CudaRuntime runtime(config);
        const double load_ms = ms_since(load_start);
        const std::size_t vocab = runtime.dimensions().vocabulary;
        std::vector<std::int32_t> tokens;
        const Timing main_point = decode(runtime, batch, context, steps, warmup, vocab, tokens);
        const Timing one = decode(runtime, 1, context, steps, warmup, vocab, tokens);
        const Timing portion = prefill(runtime, 128, 5, 2, vocab);
        const auto diagnostics = runtime.diagnostics();
        std::printf("{\"decode\": {\"batch\": %d, \"context\": %d, \"steps\": %d, \"wall_ms\": %.6f, \"device_ms\": %.6f}, "
                    "\"decode_b1\": {\"steps\": %d, \"wall_ms\": %.6f, \"device_ms\": %.6f}, "
                    "\"prefill_128\": {\"repeats\": %d, \"wall_ms\": %.6f, \"device_ms\": %.6f}, "
                    "\"load_ms\": %.1f, \"weights_bytes\": %zu, \"kv_bytes\": %zu, \"poisoned\": %s, \"last_token\": %d}\n",
                    batch, context, main_point.forwards, main_point.wall_ms, main_point.device_ms, one.forwards, one.wall_ms,
                    one.device_ms, portion.forwards, portion.wall_ms, portion.device_ms, load_ms, diagnostics.resident.weights_bytes,
                    diagnostics.resident.kv_bytes, runtime.state() == minillm::cuda::CudaRuntimeState::poisoned ? "true" : "false",
                    tokens.empty() ? -1 : tokens[0]);
        return 0;
    } catch (const std::exception& error) {
        std::fprintf(stderr, "ref_bench: %s\n", error.what());
        return 1;
    }
}
