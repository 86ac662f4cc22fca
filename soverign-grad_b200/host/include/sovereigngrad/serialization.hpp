// The reference's native checkpoint format (".sgrd": src/serialization.cpp:11-47 writes it, :49-107
// reads it) extended to packed quantized weights.
//
// Version 1 is the reference's own layout and holds fp32 tensors only:
//   "SGRD", u32 version = 1, u32 tensor count, then per tensor
//   u32 name length, name, u32 rank, rank x i64 dims, i64 numel, numel x fp32.
// A state dict of fp32 tensors is written as version 1, byte for byte what the reference writes for
// the same tensors in the same order, so the reference's load_checkpoint reads it.
//
// Version 2 (written whenever a tensor is not fp32) adds one dtype byte per tensor and counts the
// payload in bytes:
//   "SGRD", u32 version = 2, u32 tensor count, then per tensor
//   u32 name length, name, u8 dtype (0 F32, 1 F16, 2 I32, 3 I64, 4 I8, 5 U8), u32 rank, rank x i64 dims,
//   i64 payload bytes, payload.
// A quantized tensor is three entries: "<prefix>.qdata" (I8, or U8 nibble pairs), "<prefix>.scales"
// (F32) and "<prefix>.qmeta" (U8: the text "bits=..;group=..;scheme=..;layout=..;shape=a,b").  The
// reference stores the same layer as one fp32 per code (src/module.cpp:94-112): 4x / 8x larger.
// Both versions are read.  Names are written in sorted order: equal inputs give equal files.
#pragma once

#include <string>
#include <unordered_map>

#include "sovereigngrad/quantization.hpp"
#include "sovereigngrad/tensor.hpp"

namespace sovereigngrad {
namespace serialization {

using StateDict = std::unordered_map<std::string, Tensor>;

void save_checkpoint(const StateDict& state_dict, const std::string& filepath);

// Loads every tensor into storage of `device` (CUDA: straight into pool storage).
StateDict load_checkpoint(const std::string& filepath, Device device = Device::CPU);

void put_quantized(const std::string& prefix, const quantization::QuantizedTensor& q, StateDict* state_dict);
quantization::QuantizedTensor get_quantized(const std::string& prefix, const StateDict& state_dict);

}  // namespace serialization
}  // namespace sovereigngrad
