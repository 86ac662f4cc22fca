// Packed-weight checkpoints: the reference's SafeTensors reader/writer interface
// (include/sovereigngrad/safetensors.hpp, src/safetensors.cpp:15-41,174-300) extended with the
// two 8-bit dtypes, so that a quantized layer is stored as its packed codes (I8, or U8 nibble
// pairs for INT4) + fp32 scales + a few metadata strings instead of one fp32 per code, which is what
// the reference writes (src/module.cpp:94-112): 4x (INT8) / 8x (INT4) smaller, and loadable
// straight into device storage from the pool.
//
// File format: standard SafeTensors — 8-byte little-endian header length, a JSON header
// {"<name>": {"dtype": "F32|F16|I32|I64|I8|U8", "shape": [...], "data_offsets": [begin, end]}, ...,
//  "__metadata__": {"<key>": "<string>", ...}}, then the raw little-endian tensor bytes.
#pragma once

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "sovereigngrad/quantization.hpp"
#include "sovereigngrad/tensor.hpp"

namespace sovereigngrad {
namespace safetensors {

struct TensorMeta {
    std::string dtype;
    std::vector<int64_t> shape;
    size_t data_offset_start = 0;
    size_t data_offset_end = 0;
};

using StateDict = std::unordered_map<std::string, Tensor>;
using Metadata = std::map<std::string, std::string>;

// Tensors may live on either device (device tensors are copied to the host first); non-contiguous
// tensors are made contiguous.  Names are written in sorted order: equal inputs give equal files.
void save_file(const StateDict& state_dict, const std::string& filepath, const Metadata& metadata = {});

// Loads every tensor into storage of `device` (CUDA: from the pool).  `metadata` (optional)
// receives the "__metadata__" strings.  Throws std::runtime_error on a malformed file.
StateDict load_file(const std::string& filepath, Device device = Device::CPU, Metadata* metadata = nullptr);

// Header only.
std::unordered_map<std::string, TensorMeta> inspect_file(const std::string& filepath, Metadata* metadata = nullptr);

// A quantized tensor as entries "<prefix>.qdata" (I8 / U8) and "<prefix>.scales" (F32) plus metadata
// "<prefix>.bits", ".group_size", ".scheme", ".layout", ".original_shape" (comma separated).
void put_quantized(const std::string& prefix, const quantization::QuantizedTensor& q, StateDict* state_dict, Metadata* metadata);
quantization::QuantizedTensor get_quantized(const std::string& prefix, const StateDict& state_dict, const Metadata& metadata);

}  // namespace safetensors
}  // namespace sovereigngrad
