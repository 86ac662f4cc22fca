// nn::Linear (as the source of float weights) and the quantized layers of the reference
// (include/sovereigngrad/nn.hpp:18-39, 927-1001) over the sm_100a kernels.
//
// Differences from the reference, all on purpose:
//   * the constructors do not draw a random weight and quantize it only to throw it away in
//     from_float() (nn.hpp:935-954): a layer is built from real weights or starts empty;
//   * nn::QuantizedLinear::from_float keeps the reference's default (one INT8 scale per row of the
//     stored [in, out] weight) and takes the scheme as an optional argument;
//   * Linear::forward is a plain host loop (a float reference for tests), not a GPU kernel:
//     fp32 GEMM is not part of this path.
#pragma once

#include <cmath>
#include <memory>

#include "sovereigngrad/module.hpp"
#include "sovereigngrad/quantization.hpp"

namespace sovereigngrad {
namespace nn {

class Linear : public Module {
public:
    Tensor W;   // [in_features, out_features]
    Tensor b;   // [1, out_features]

    Linear(int64_t in_features, int64_t out_features, Device device = Device::CPU, uint64_t seed = 0) {
        const float std = std::sqrt(2.0f / static_cast<float>(in_features + out_features));   // nn.hpp:24
        W = Tensor::randn({in_features, out_features}, 0.0f, std, device, true, seed);
        b = Tensor::zeros({1, out_features}, device, true);
        register_parameter("weight", W);
        register_parameter("bias", b);
    }

    Tensor forward(const Tensor& x) override;   // y = x*W + b on the host
};

class QuantizedLinear : public Module {
public:
    quantization::QuantizedTensor q_weight;
    Tensor bias;
    int64_t in_features;
    int64_t out_features;

    QuantizedLinear(int64_t in_features, int64_t out_features) : in_features(in_features), out_features(out_features) {
        register_all();
    }

    static std::shared_ptr<QuantizedLinear> from_float(
        const Linear& float_linear,
        quantization::QuantizationScheme scheme = quantization::QuantizationScheme::PerChannelSymmetric) {
        auto ql = std::make_shared<QuantizedLinear>(float_linear.W.shape()[0], float_linear.W.shape()[1]);
        ql->q_weight = quantization::quantize_int8(float_linear.W.to(Device::CUDA), scheme);
        ql->bias = float_linear.b.to(Device::CUDA).clone();
        return ql;
    }

    Tensor forward(const Tensor& x) override { return quantization::quantized_matmul_int8(x, q_weight, bias); }

protected:
    void register_all() {
        register_parameter("qdata", q_weight.qdata);
        register_parameter("scales", q_weight.scales);
        register_parameter("bias", bias);
    }
};

class QuantizedLinear4Bit : public Module {
public:
    quantization::QuantizedTensor q_weight;
    Tensor bias;
    int64_t in_features;
    int64_t out_features;
    int64_t group_size;

    QuantizedLinear4Bit(int64_t in_features, int64_t out_features, int64_t group_size = 32)
        : in_features(in_features), out_features(out_features), group_size(group_size) {
        register_parameter("qdata", q_weight.qdata);
        register_parameter("scales", q_weight.scales);
        register_parameter("bias", bias);
    }

    static std::shared_ptr<QuantizedLinear4Bit> from_float(const Linear& float_linear, int64_t group_size = 32) {
        auto ql = std::make_shared<QuantizedLinear4Bit>(float_linear.W.shape()[0], float_linear.W.shape()[1], group_size);
        ql->q_weight = quantization::quantize_int4(float_linear.W.to(Device::CUDA), group_size);
        ql->bias = float_linear.b.to(Device::CUDA).clone();
        return ql;
    }

    // Weight given as [out, in] (y = x*W^T): INT4 groups then run along the input dimension, which is
    // what the decode and tensor-core kernels stream.
    static std::shared_ptr<QuantizedLinear4Bit> from_weight_nk(const Tensor& w_nk, const Tensor& bias, int64_t group_size = 32) {
        auto ql = std::make_shared<QuantizedLinear4Bit>(w_nk.shape()[1], w_nk.shape()[0], group_size);
        ql->q_weight = quantization::quantize_int4(w_nk.to(Device::CUDA), group_size);
        ql->q_weight.set_layout(quantization::WeightLayout::NK);
        if (bias.is_defined()) ql->bias = bias.to(Device::CUDA).clone();
        return ql;
    }

    Tensor forward(const Tensor& x) override { return quantization::quantized_matmul_int4(x, q_weight, bias); }
};

}  // namespace nn
}  // namespace sovereigngrad
