#include "sovereigngrad/serialization.hpp"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <vector>

namespace sovereigngrad {
namespace serialization {
namespace {

const char kMagic[4] = {'S', 'G', 'R', 'D'};

int dtype_code(DType d) {
    switch (d) {
        case DType::Float32: return 0;
        case DType::Float16: return 1;
        case DType::Int32: return 2;
        case DType::Int64: return 3;
        case DType::Int8: return 4;
        case DType::UInt8: return 5;
    }
    return 0;
}

DType dtype_of(int code, const std::string& file) {
    switch (code) {
        case 0: return DType::Float32;
        case 1: return DType::Float16;
        case 2: return DType::Int32;
        case 3: return DType::Int64;
        case 4: return DType::Int8;
        case 5: return DType::UInt8;
    }
    throw std::runtime_error("Invalid dtype code " + std::to_string(code) + " in checkpoint: " + file);
}

template <typename T>
void put(std::ofstream& out, T v) { out.write(reinterpret_cast<const char*>(&v), sizeof(T)); }

template <typename T>
T get(std::ifstream& in, const std::string& file) {
    T v{};
    if (!in.read(reinterpret_cast<char*>(&v), sizeof(T))) throw std::runtime_error("Truncated checkpoint file: " + file);
    return v;
}

}  // namespace

void save_checkpoint(const StateDict& state_dict, const std::string& filepath) {
    std::ofstream out(filepath, std::ios::binary);
    if (!out.is_open()) throw std::runtime_error("Failed to open file for writing checkpoint: " + filepath);
    std::vector<std::string> names;
    bool all_f32 = true;
    for (const auto& kv : state_dict) {
        if (!kv.second.is_defined()) throw std::runtime_error("Undefined tensor in state dict: " + kv.first);
        names.push_back(kv.first);
        all_f32 = all_f32 && kv.second.dtype() == DType::Float32;
    }
    std::sort(names.begin(), names.end());
    const uint32_t version = all_f32 ? 1u : 2u;
    out.write(kMagic, 4);
    put<uint32_t>(out, version);
    put<uint32_t>(out, static_cast<uint32_t>(names.size()));
    for (const std::string& name : names) {
        Tensor t = state_dict.at(name).to(Device::CPU).contiguous();
        put<uint32_t>(out, static_cast<uint32_t>(name.size()));
        out.write(name.data(), static_cast<std::streamsize>(name.size()));
        if (version == 2) put<uint8_t>(out, static_cast<uint8_t>(dtype_code(t.dtype())));
        put<uint32_t>(out, static_cast<uint32_t>(t.shape().size()));
        for (int64_t d : t.shape()) put<int64_t>(out, d);
        const int64_t bytes = t.numel() * static_cast<int64_t>(dtype_size(t.dtype()));
        put<int64_t>(out, version == 1 ? t.numel() : bytes);
        if (bytes) out.write(static_cast<const char*>(t.raw()), bytes);
    }
    if (!out) throw std::runtime_error("Failed to write checkpoint: " + filepath);
}

StateDict load_checkpoint(const std::string& filepath, Device device) {
    std::ifstream in(filepath, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error("Failed to open file for reading checkpoint: " + filepath);
    char magic[4];
    if (!in.read(magic, 4) || std::memcmp(magic, kMagic, 4) != 0)
        throw std::runtime_error("Invalid checkpoint file format or corrupted magic header in: " + filepath);
    const uint32_t version = get<uint32_t>(in, filepath);
    if (version != 1 && version != 2) throw std::runtime_error("Unsupported checkpoint format version: " + std::to_string(version));
    const uint32_t count = get<uint32_t>(in, filepath);
    StateDict result;
    for (uint32_t i = 0; i < count; ++i) {
        const uint32_t name_len = get<uint32_t>(in, filepath);
        if (name_len > (1u << 20)) throw std::runtime_error("Corrupted tensor name in checkpoint: " + filepath);
        std::string name(name_len, '\0');
        if (name_len && !in.read(&name[0], name_len)) throw std::runtime_error("Truncated checkpoint file: " + filepath);
        const DType dt = version == 2 ? dtype_of(get<uint8_t>(in, filepath), filepath) : DType::Float32;
        const uint32_t rank = get<uint32_t>(in, filepath);
        if (rank > 16) throw std::runtime_error("Corrupted tensor rank in checkpoint: " + filepath);
        std::vector<int64_t> shape(rank);
        int64_t numel = 1;
        for (uint32_t r = 0; r < rank; ++r) {
            shape[r] = get<int64_t>(in, filepath);
            if (shape[r] < 0) throw std::runtime_error("Negative dimension in checkpoint: " + filepath);
            numel *= shape[r];
        }
        const int64_t stored = get<int64_t>(in, filepath);
        const int64_t bytes = numel * static_cast<int64_t>(dtype_size(dt));
        if (stored != (version == 1 ? numel : bytes))
            throw std::runtime_error("Tensor '" + name + "' has a payload that does not match its shape in: " + filepath);
        Tensor host = Tensor::empty(shape, Device::CPU, dt);
        if (bytes && !in.read(static_cast<char*>(host.raw()), bytes)) throw std::runtime_error("Truncated checkpoint file: " + filepath);
        result[name] = device == Device::CPU ? host : host.to(device);
    }
    return result;
}

void put_quantized(const std::string& prefix, const quantization::QuantizedTensor& q, StateDict* state_dict) {
    std::ostringstream ss;
    ss << "bits=" << q.bits << ";group=" << q.group_size << ";scheme=" << static_cast<int>(q.scheme)
       << ";layout=" << (q.layout == quantization::WeightLayout::NK ? "NK" : "KN") << ";shape=";
    for (size_t i = 0; i < q.original_shape.size(); ++i) ss << (i ? "," : "") << q.original_shape[i];
    const std::string text = ss.str();
    Tensor meta = Tensor::empty({static_cast<int64_t>(text.size())}, Device::CPU, DType::UInt8);
    std::memcpy(meta.raw(), text.data(), text.size());
    (*state_dict)[prefix + ".qdata"] = q.qdata;
    (*state_dict)[prefix + ".scales"] = q.scales;
    (*state_dict)[prefix + ".qmeta"] = meta;
}

quantization::QuantizedTensor get_quantized(const std::string& prefix, const StateDict& state_dict) {
    auto tensor = [&](const std::string& k) -> const Tensor& {
        auto it = state_dict.find(prefix + k);
        if (it == state_dict.end()) throw std::runtime_error("checkpoint: missing tensor " + prefix + k);
        return it->second;
    };
    quantization::QuantizedTensor q;
    q.qdata = tensor(".qdata");
    q.scales = tensor(".scales");
    Tensor meta = tensor(".qmeta").to(Device::CPU);
    if (meta.dtype() != DType::UInt8) throw std::runtime_error("checkpoint: " + prefix + ".qmeta is not a byte string");
    const std::string text(static_cast<const char*>(meta.raw()), static_cast<size_t>(meta.numel()));
    bool have_bits = false, have_shape = false;
    std::stringstream fields(text);
    std::string field;
    while (std::getline(fields, field, ';')) {
        const size_t eq = field.find('=');
        if (eq == std::string::npos) throw std::runtime_error("checkpoint: malformed " + prefix + ".qmeta");
        const std::string key = field.substr(0, eq), val = field.substr(eq + 1);
        if (key == "bits") { q.bits = std::stoi(val); have_bits = true; }
        else if (key == "group") q.group_size = std::stoll(val);
        else if (key == "scheme") q.scheme = static_cast<quantization::QuantizationScheme>(std::stoi(val));
        else if (key == "layout") q.layout = val == "NK" ? quantization::WeightLayout::NK : quantization::WeightLayout::KN;
        else if (key == "shape") {
            std::stringstream dims(val);
            std::string d;
            while (std::getline(dims, d, ',')) q.original_shape.push_back(std::stoll(d));
            have_shape = true;
        }
    }
    int64_t numel = 1;
    for (int64_t d : q.original_shape) numel *= d;
    const int64_t want = q.bits == 4 ? (numel + 1) / 2 : numel;
    const DType want_dt = q.bits == 4 ? DType::UInt8 : DType::Int8;
    if (!have_bits || !have_shape || (q.bits != 4 && q.bits != 8) || q.qdata.dtype() != want_dt || q.qdata.numel() != want ||
        q.scales.dtype() != DType::Float32)
        throw std::runtime_error("checkpoint: " + prefix + " does not hold a consistent quantized tensor");
    return q;
}

}  // namespace serialization
}  // namespace sovereigngrad
