// SafeTensors reader/writer with 8-bit dtypes for packed quantized weights (see the header).
#include "sovereigngrad/safetensors.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace sovereigngrad {
namespace safetensors {
namespace {

const char* dtype_str(DType d) {
    switch (d) {
        case DType::Float32: return "F32";
        case DType::Float16: return "F16";
        case DType::Int32: return "I32";
        case DType::Int64: return "I64";
        case DType::Int8: return "I8";
        case DType::UInt8: return "U8";
    }
    return "F32";
}

DType dtype_from(const std::string& s) {
    if (s == "F32") return DType::Float32;
    if (s == "F16") return DType::Float16;
    if (s == "I32") return DType::Int32;
    if (s == "I64") return DType::Int64;
    if (s == "I8") return DType::Int8;
    if (s == "U8") return DType::UInt8;
    throw std::runtime_error("safetensors: unsupported dtype " + s);
}

std::string escape(const std::string& s) {
    std::string o;
    for (char c : s) {
        if (c == '"' || c == '\\') { o += '\\'; o += c; }
        else if (c == '\n') o += "\\n";
        else if (c == '\t') o += "\\t";
        else if (static_cast<unsigned char>(c) < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += c;
    }
    return o;
}

// A small recursive-descent reader for the JSON subset a SafeTensors header uses: objects, arrays of
// integers, strings, integers.
struct Json {
    const std::string& s;
    size_t p = 0;
    explicit Json(const std::string& str) : s(str) {}
    [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("safetensors: bad header: ") + what); }
    void ws() { while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\r' || s[p] == '\t')) ++p; }
    bool eat(char c) { ws(); if (p < s.size() && s[p] == c) { ++p; return true; } return false; }
    void expect(char c) { if (!eat(c)) fail("unexpected character"); }
    std::string str() {
        ws();
        if (p >= s.size() || s[p] != '"') fail("string expected");
        ++p;
        std::string o;
        while (p < s.size() && s[p] != '"') {
            if (s[p] == '\\') {
                if (++p >= s.size()) fail("dangling escape");
                switch (s[p]) {
                    case 'n': o += '\n'; break;
                    case 't': o += '\t'; break;
                    case 'r': o += '\r'; break;
                    case 'b': o += '\b'; break;
                    case 'f': o += '\f'; break;
                    case 'u': {
                        if (p + 4 >= s.size()) fail("short \\u escape");
                        const unsigned v = static_cast<unsigned>(std::stoul(s.substr(p + 1, 4), nullptr, 16));
                        if (v < 0x80) o += static_cast<char>(v);
                        else if (v < 0x800) { o += static_cast<char>(0xC0 | (v >> 6)); o += static_cast<char>(0x80 | (v & 0x3F)); }
                        else { o += static_cast<char>(0xE0 | (v >> 12)); o += static_cast<char>(0x80 | ((v >> 6) & 0x3F)); o += static_cast<char>(0x80 | (v & 0x3F)); }
                        p += 4;
                        break;
                    }
                    default: o += s[p];
                }
                ++p;
            } else {
                o += s[p++];
            }
        }
        if (p >= s.size()) fail("unterminated string");
        ++p;
        return o;
    }
    int64_t integer() {
        ws();
        size_t q = p;
        if (q < s.size() && s[q] == '-') ++q;
        while (q < s.size() && s[q] >= '0' && s[q] <= '9') ++q;
        if (q == p) fail("integer expected");
        const int64_t v = std::stoll(s.substr(p, q - p));
        p = q;
        return v;
    }
    std::vector<int64_t> int_array() {
        std::vector<int64_t> v;
        expect('[');
        if (eat(']')) return v;
        do v.push_back(integer()); while (eat(','));
        expect(']');
        return v;
    }
};

struct Header {
    std::unordered_map<std::string, TensorMeta> tensors;
    Metadata metadata;
    size_t data_start = 0;
};

Header read_header(std::ifstream& f, const std::string& path) {
    if (!f) throw std::runtime_error("safetensors: cannot open " + path);
    unsigned char lenb[8];
    f.read(reinterpret_cast<char*>(lenb), 8);
    if (f.gcount() != 8) throw std::runtime_error("safetensors: file too short: " + path);
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | lenb[i];
    if (n == 0 || n > (1ull << 30)) throw std::runtime_error("safetensors: implausible header length in " + path);
    std::string js(n, '\0');
    f.read(&js[0], static_cast<std::streamsize>(n));
    if (static_cast<uint64_t>(f.gcount()) != n) throw std::runtime_error("safetensors: truncated header in " + path);
    Header h;
    h.data_start = 8 + n;
    Json j(js);
    j.expect('{');
    if (!j.eat('}')) {
        do {
            const std::string name = j.str();
            j.expect(':');
            j.expect('{');
            if (name == "__metadata__") {
                if (!j.eat('}')) {
                    do {
                        const std::string k = j.str();
                        j.expect(':');
                        h.metadata[k] = j.str();
                    } while (j.eat(','));
                    j.expect('}');
                }
                continue;
            }
            TensorMeta m;
            bool have_offsets = false;
            if (!j.eat('}')) {
                do {
                    const std::string k = j.str();
                    j.expect(':');
                    if (k == "dtype") m.dtype = j.str();
                    else if (k == "shape") m.shape = j.int_array();
                    else if (k == "data_offsets") {
                        const auto o = j.int_array();
                        if (o.size() != 2 || o[0] < 0 || o[1] < o[0]) j.fail("bad data_offsets");
                        m.data_offset_start = static_cast<size_t>(o[0]);
                        m.data_offset_end = static_cast<size_t>(o[1]);
                        have_offsets = true;
                    } else j.fail("unknown tensor field");
                } while (j.eat(','));
                j.expect('}');
            }
            if (m.dtype.empty() || !have_offsets) j.fail("tensor entry without dtype or data_offsets");
            h.tensors[name] = m;
        } while (j.eat(','));
        j.expect('}');
    }
    return h;
}

std::string join_shape(const std::vector<int64_t>& s) {
    std::string o;
    for (size_t i = 0; i < s.size(); ++i) o += (i ? "," : "") + std::to_string(s[i]);
    return o;
}

}  // namespace

void save_file(const StateDict& state_dict, const std::string& filepath, const Metadata& metadata) {
    std::vector<std::string> names;
    for (const auto& kv : state_dict) names.push_back(kv.first);
    std::sort(names.begin(), names.end());
    std::vector<Tensor> host;
    std::ostringstream js;
    js << "{";
    size_t off = 0;
    bool first = true;
    if (!metadata.empty()) {
        js << "\"__metadata__\":{";
        bool f2 = true;
        for (const auto& kv : metadata) {
            js << (f2 ? "" : ",") << "\"" << escape(kv.first) << "\":\"" << escape(kv.second) << "\"";
            f2 = false;
        }
        js << "}";
        first = false;
    }
    for (const auto& name : names) {
        const Tensor& t = state_dict.at(name);
        if (!t.is_defined()) throw std::runtime_error("safetensors: undefined tensor " + name);
        Tensor h = t.device() == Device::CPU ? t.contiguous() : t.contiguous().to(Device::CPU);
        const size_t bytes = static_cast<size_t>(h.numel()) * dtype_size(h.dtype());
        js << (first ? "" : ",") << "\"" << escape(name) << "\":{\"dtype\":\"" << dtype_str(h.dtype()) << "\",\"shape\":[";
        for (size_t i = 0; i < h.shape().size(); ++i) js << (i ? "," : "") << h.shape()[i];
        js << "],\"data_offsets\":[" << off << "," << off + bytes << "]}";
        off += bytes;
        first = false;
        host.push_back(h);
    }
    js << "}";
    std::string header = js.str();
    while (header.size() % 8) header += ' ';                  // the data section starts 8-byte aligned
    std::ofstream f(filepath, std::ios::binary | std::ios::trunc);
    if (!f) throw std::runtime_error("safetensors: cannot create " + filepath);
    uint64_t n = header.size();
    unsigned char lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = static_cast<unsigned char>((n >> (8 * i)) & 0xFF);
    f.write(reinterpret_cast<const char*>(lenb), 8);
    f.write(header.data(), static_cast<std::streamsize>(header.size()));
    for (const Tensor& h : host) {
        const size_t bytes = static_cast<size_t>(h.numel()) * dtype_size(h.dtype());
        if (bytes) f.write(static_cast<const char*>(h.raw()), static_cast<std::streamsize>(bytes));
    }
    if (!f) throw std::runtime_error("safetensors: write failed: " + filepath);
}

std::unordered_map<std::string, TensorMeta> inspect_file(const std::string& filepath, Metadata* metadata) {
    std::ifstream f(filepath, std::ios::binary);
    Header h = read_header(f, filepath);
    if (metadata) *metadata = h.metadata;
    return h.tensors;
}

StateDict load_file(const std::string& filepath, Device device, Metadata* metadata) {
    std::ifstream f(filepath, std::ios::binary);
    Header h = read_header(f, filepath);
    if (metadata) *metadata = h.metadata;
    f.seekg(0, std::ios::end);
    const size_t file_size = static_cast<size_t>(f.tellg());
    StateDict out;
    for (const auto& kv : h.tensors) {
        const TensorMeta& m = kv.second;
        const DType dt = dtype_from(m.dtype);
        int64_t numel = 1;
        for (int64_t d : m.shape) {
            if (d < 0) throw std::runtime_error("safetensors: negative dimension in " + kv.first);
            numel *= d;
        }
        const size_t bytes = static_cast<size_t>(numel) * dtype_size(dt);
        if (m.data_offset_end - m.data_offset_start != bytes || h.data_start + m.data_offset_end > file_size)
            throw std::runtime_error("safetensors: data_offsets of " + kv.first + " do not match its shape or the file size");
        Tensor host = Tensor::empty(m.shape, Device::CPU, dt);
        if (bytes) {
            f.seekg(static_cast<std::streamoff>(h.data_start + m.data_offset_start));
            f.read(static_cast<char*>(host.raw()), static_cast<std::streamsize>(bytes));
            if (static_cast<size_t>(f.gcount()) != bytes) throw std::runtime_error("safetensors: truncated data for " + kv.first);
        }
        out[kv.first] = device == Device::CPU ? host : host.to(device);
    }
    return out;
}

void put_quantized(const std::string& prefix, const quantization::QuantizedTensor& q, StateDict* state_dict, Metadata* metadata) {
    (*state_dict)[prefix + ".qdata"] = q.qdata;
    (*state_dict)[prefix + ".scales"] = q.scales;
    (*metadata)[prefix + ".bits"] = std::to_string(q.bits);
    (*metadata)[prefix + ".group_size"] = std::to_string(q.group_size);
    (*metadata)[prefix + ".scheme"] = std::to_string(static_cast<int>(q.scheme));
    (*metadata)[prefix + ".layout"] = q.layout == quantization::WeightLayout::NK ? "NK" : "KN";
    (*metadata)[prefix + ".original_shape"] = join_shape(q.original_shape);
}

quantization::QuantizedTensor get_quantized(const std::string& prefix, const StateDict& state_dict, const Metadata& metadata) {
    auto need = [&](const std::string& k) -> const std::string& {
        auto it = metadata.find(prefix + k);
        if (it == metadata.end()) throw std::runtime_error("safetensors: missing metadata " + prefix + k);
        return it->second;
    };
    auto tensor = [&](const std::string& k) -> const Tensor& {
        auto it = state_dict.find(prefix + k);
        if (it == state_dict.end()) throw std::runtime_error("safetensors: missing tensor " + prefix + k);
        return it->second;
    };
    quantization::QuantizedTensor q;
    q.qdata = tensor(".qdata");
    q.scales = tensor(".scales");
    q.bits = std::stoi(need(".bits"));
    q.group_size = std::stoll(need(".group_size"));
    q.scheme = static_cast<quantization::QuantizationScheme>(std::stoi(need(".scheme")));
    q.layout = need(".layout") == "NK" ? quantization::WeightLayout::NK : quantization::WeightLayout::KN;
    std::stringstream ss(need(".original_shape"));
    std::string part;
    while (std::getline(ss, part, ',')) q.original_shape.push_back(std::stoll(part));
    int64_t numel = 1;
    for (int64_t d : q.original_shape) numel *= d;
    const int64_t want = q.bits == 4 ? (numel + 1) / 2 : numel;
    const DType want_dt = q.bits == 4 ? DType::UInt8 : DType::Int8;
    if ((q.bits != 4 && q.bits != 8) || q.qdata.dtype() != want_dt || q.qdata.numel() != want || q.scales.dtype() != DType::Float32)
        throw std::runtime_error("safetensors: " + prefix + " does not hold a consistent quantized tensor");
    return q;
}

}  // namespace safetensors
}  // namespace sovereigngrad
