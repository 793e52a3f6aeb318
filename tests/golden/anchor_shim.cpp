// Stand-ins for the two classes of lilong555/mini-llm-runtime that need llama.cpp
// (minillm::GgufModel, minillm::Tokenizer), so that the project's own CPU forward pass
// (src/minillm/runtime.cpp, qwen3_model.cpp, paged_kv.cpp, kernels.cpp, parallel.cpp) can
// be compiled UNCHANGED from its source tree and run on a tiny random model.  The model
// comes from a flat file written by make_reference_golden.py:
//
//   int32 n_meta;  n_meta x { str key; int32 kind (0 int, 1 float, 2 string); value }
//   int32 n_tensors;  n_tensors x { str name; int32 rows; int32 columns; float32 data[rows*columns] }
//   str = int32 length + bytes
//
// main() feeds one token sequence through minillm::Runtime::forward in the given portions
// with logits at every position and writes them as float32.
#include "minillm/gguf_model.h"
#include "minillm/runtime.h"
#include "minillm/tokenizer.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace minillm {

struct GgufModel::Impl {
    std::map<std::string, std::uint64_t> integers;
    std::map<std::string, float> floats;
    std::map<std::string, std::string> strings;
    struct Tensor {
        std::size_t rows, columns;
        std::vector<float> data;
    };
    std::map<std::string, Tensor> tensors;
    std::size_t bytes = 0;
};

namespace {
std::string read_string(std::ifstream& in) {
    std::int32_t n = 0;
    in.read(reinterpret_cast<char*>(&n), 4);
    std::string s(static_cast<std::size_t>(n), '\0');
    in.read(s.data(), n);
    return s;
}
}  // namespace

GgufModel::GgufModel(const std::string& path) : impl_(std::make_unique<Impl>()) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw std::runtime_error("cannot open " + path);
    std::int32_t n_meta = 0;
    in.read(reinterpret_cast<char*>(&n_meta), 4);
    for (int i = 0; i < n_meta; ++i) {
        const auto key = read_string(in);
        std::int32_t kind = 0;
        in.read(reinterpret_cast<char*>(&kind), 4);
        if (kind == 0) {
            std::int64_t v = 0;
            in.read(reinterpret_cast<char*>(&v), 8);
            impl_->integers[key] = static_cast<std::uint64_t>(v);
        } else if (kind == 1) {
            float v = 0;
            in.read(reinterpret_cast<char*>(&v), 4);
            impl_->floats[key] = v;
        } else {
            impl_->strings[key] = read_string(in);
        }
    }
    std::int32_t n_tensors = 0;
    in.read(reinterpret_cast<char*>(&n_tensors), 4);
    for (int i = 0; i < n_tensors; ++i) {
        const auto name = read_string(in);
        std::int32_t rows = 0, columns = 0;
        in.read(reinterpret_cast<char*>(&rows), 4);
        in.read(reinterpret_cast<char*>(&columns), 4);
        Impl::Tensor t{static_cast<std::size_t>(rows), static_cast<std::size_t>(columns), {}};
        t.data.resize(t.rows * t.columns);
        in.read(reinterpret_cast<char*>(t.data.data()), static_cast<std::streamsize>(t.data.size() * 4));
        impl_->bytes += t.data.size() * 4;
        impl_->tensors.emplace(name, std::move(t));
    }
    if (!in) throw std::runtime_error("short model file " + path);
}
GgufModel::~GgufModel() = default;
std::string GgufModel::string_value(const std::string& key) const { return impl_->strings.at(key); }
std::uint64_t GgufModel::integer_value(const std::string& key) const { return impl_->integers.at(key); }
float GgufModel::float_value(const std::string& key) const { return impl_->floats.at(key); }
bool GgufModel::contains(const std::string& key) const {
    return impl_->integers.count(key) || impl_->floats.count(key) || impl_->strings.count(key);
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

// usage: anchor MODEL.bin CONTEXT PAGE OUT.f32 PORTION token token ...
int main(int argc, char** argv) {
    if (argc < 7) {
        std::fprintf(stderr, "usage: anchor MODEL.bin CONTEXT PAGE OUT.f32 PORTION tokens...\n");
        return 2;
    }
    try {
        minillm::RuntimeConfig config;
        config.model_path = argv[1];
        config.context_tokens = static_cast<std::size_t>(std::atoi(argv[2]));
        config.page_tokens = static_cast<std::size_t>(std::atoi(argv[3]));
        config.max_sequences = 2;
        config.batch_tokens = config.context_tokens;
        config.threads = 2;
        config.kernels = minillm::KernelMode::scalar;
        const std::size_t portion = static_cast<std::size_t>(std::atoi(argv[5]));
        std::vector<std::int32_t> tokens;
        for (int i = 6; i < argc; ++i) tokens.push_back(std::atoi(argv[i]));
        minillm::Runtime runtime(config);
        std::ofstream out(argv[4], std::ios::binary);
        for (std::size_t begin = 0; begin < tokens.size(); begin += portion) {
            std::vector<minillm::InputToken> batch;
            for (std::size_t p = begin; p < std::min(tokens.size(), begin + portion); ++p)
                batch.push_back({tokens[p], static_cast<std::int32_t>(p), 0, true});
            for (const auto& row : runtime.forward(batch))
                out.write(reinterpret_cast<const char*>(row.values.data()), static_cast<std::streamsize>(row.values.size() * 4));
        }
        return 0;
    } catch (const std::exception& error) {
        std::fprintf(stderr, "anchor: %s\n", error.what());
        return 1;
    }
}
