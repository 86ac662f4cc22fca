// Host side of the B200 quantization path: the reference's quantization API
// (include/sovereigngrad/quantization.hpp:11-37) over the C ABI of include/sgq.h.
//
// Same names, argument meaning and error behaviour (std::runtime_error), with these documented
// differences:
//   * `qdata` holds packed codes — DType::Int8 of the original shape, or DType::UInt8 with
//     ceil(numel/2) bytes for INT4 (low nibble = even element) — instead of one fp32 per code;
//     codes_as_float() gives the reference's fp32 view.
//   * tensors must live on Device::CUDA: the kernels are sm_100a only and there is no CPU path
//     (the reference bounces every call through the host, src/quantization.cpp:12,40,110).
//   * no autograd graph is recorded; the gradient the reference's graph would send into x
//     (MatmulNode, src/ops.cpp:362-375) is available as quantized_matmul_backward_x().
//   * `layout` says how a 2-D weight is stored: KN = [in, out] (the reference's own convention,
//     y = x*W), NK = [out, in] (y = x*W^T).  It is recorded in the QuantizedTensor by
//     quantize_*() callers through set_layout(); default KN.
#pragma once

#include <cstdint>
#include <vector>

#include "sovereigngrad/tensor.hpp"

namespace sovereigngrad {
namespace quantization {

enum class QuantizationScheme { PerTensorSymmetric, PerChannelSymmetric, GroupedAsymmetric };
enum class WeightLayout { KN = 0, NK = 1 };
// which kernel family the forward uses; Auto picks by shape (see sgq.h SGQ_PATH_*)
enum class ForwardPath { Auto = 0, Simt = 1, Decode = 2, TensorCoreBf16 = 3, TensorCoreInt8 = 4 };

struct QuantizedTensor {
    Tensor qdata;        // packed codes (Int8 / UInt8)
    Tensor scales;       // fp32 scaling factors, reference order
    Tensor zero_points;  // never written (the reference's "GroupedAsymmetric" is symmetric too)
    QuantizationScheme scheme = QuantizationScheme::PerTensorSymmetric;
    std::vector<int64_t> original_shape;
    int64_t group_size = 0;   // INT8: numel (as the reference sets it); INT4: group
    int bits = 8;
    WeightLayout layout = WeightLayout::KN;

    QuantizedTensor& set_layout(WeightLayout l) { layout = l; return *this; }
    Tensor codes_as_float() const;   // the reference's `qdata`: integer codes as fp32, original shape
};

QuantizedTensor quantize_int8(const Tensor& x, QuantizationScheme scheme = QuantizationScheme::PerChannelSymmetric);
Tensor dequantize_int8(const QuantizedTensor& qx);

QuantizedTensor quantize_int4(const Tensor& x, int64_t group_size = 32);
Tensor dequantize_int4(const QuantizedTensor& qx);

Tensor quantized_matmul_int8(const Tensor& x, const QuantizedTensor& q_weight, const Tensor& bias = Tensor(),
                             ForwardPath path = ForwardPath::Auto);
Tensor quantized_matmul_int4(const Tensor& x, const QuantizedTensor& q_weight, const Tensor& bias = Tensor(),
                             ForwardPath path = ForwardPath::Auto);

// grad_x of quantized_matmul_int8 / _int4(x, q_weight): grad_output[M,N] * deq(W)^T, what the reference's
// autograd computes when x requires a gradient (src/ops.cpp:367-370).  Weights are frozen codes.
Tensor quantized_matmul_backward_x(const Tensor& grad_output, const QuantizedTensor& q_weight,
                                   ForwardPath path = ForwardPath::Auto);

// Dynamic activation quantization: one scale per row (token) of x[tokens, features] — the reference's
// per-channel quantizer (src/quantization.cpp:42-75) applied to activations.
QuantizedTensor quantize_activations_int8(const Tensor& x);

}  // namespace quantization
}  // namespace sovereigngrad
