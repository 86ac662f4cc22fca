#include "sovereigngrad/quantization.hpp"

#include <stdexcept>
#include <string>

#include <cuda_runtime_api.h>

#include "sgq.h"

namespace sovereigngrad {
namespace quantization {
namespace {

void check(int status, const char* what) {
    if (status != SGQ_OK)
        throw std::runtime_error(std::string(what) + ": " + sgq_status_string(status) + " (" + sgq_last_error() + ")");
}

void require_cuda(const Tensor& t, const char* what) {
    if (!t.is_defined()) throw std::runtime_error(std::string(what) + ": undefined tensor");
    if (t.device() != Device::CUDA)
        throw std::runtime_error(std::string(what) + ": tensor must be on Device::CUDA (this build has no CPU path)");
}

Tensor f32_contiguous(const Tensor& t) {
    if (t.dtype() != DType::Float32) throw std::runtime_error("expected a Float32 tensor");
    return t.contiguous();
}

bool per_tensor(const QuantizedTensor& q) {
    return q.scheme == QuantizationScheme::PerTensorSymmetric || q.scales.numel() == 1;   // src/quantization.cpp:91
}

// scratch for the forward; grows on demand, protected by the pool's own locking
struct Workspace {
    Tensor buf;
    void* get(size_t bytes, size_t* have) {
        if (bytes == 0) { *have = 0; return nullptr; }
        if (!buf.is_defined() || static_cast<size_t>(buf.numel()) < bytes)
            buf = Tensor::empty({static_cast<int64_t>(bytes)}, Device::CUDA, DType::UInt8);
        *have = static_cast<size_t>(buf.numel());
        return buf.raw();
    }
};
// One per calling thread (entry points are re-entrant) AND per device: a thread that switches the
// current device must never hand one GPU's kernels a scratch buffer that lives on another.
constexpr int kMaxDevices = 64;
thread_local Workspace g_workspaces[kMaxDevices];
Workspace& workspace_of_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) dev = 0;
    return g_workspaces[dev];
}

Tensor forward(const Tensor& x_in, const QuantizedTensor& q, const Tensor& bias, ForwardPath path) {
    require_cuda(x_in, "quantized_matmul");
    require_cuda(q.qdata, "quantized_matmul");
    if (x_in.shape().size() != 2 || q.original_shape.size() != 2)
        throw std::runtime_error("matmul currently requires 2D tensors!");               // src/ops.cpp:380-382
    const bool kn = q.layout == WeightLayout::KN;
    const int64_t K = kn ? q.original_shape[0] : q.original_shape[1];
    const int64_t N = kn ? q.original_shape[1] : q.original_shape[0];
    const int64_t M = x_in.shape()[0];
    if (x_in.shape()[1] != K) throw std::runtime_error("Matrix inner dimensions must match for matmul!");   // :387-389
    Tensor x = f32_contiguous(x_in);
    const float* bias_ptr = nullptr;
    Tensor b;
    if (bias.is_defined()) {                                                             // undefined bias = skip (:193,202)
        if (bias.device() != Device::CUDA) throw std::runtime_error("Device mismatch in add!");
        if (bias.numel() != N) throw std::runtime_error("Incompatible shapes for broadcasting!");
        b = f32_contiguous(bias);
        bias_ptr = b.data();
    }
    Tensor y = Tensor::empty({M, N}, Device::CUDA);
    const int layout = kn ? SGQ_LAYOUT_KN : SGQ_LAYOUT_NK;
    size_t have = 0;
    void* ws = workspace_of_current_device().get(sgq_linear_workspace_bytes(q.bits, M, K, N, layout, static_cast<int>(path)), &have);
    int rc;
    if (q.bits == 4) {
        rc = sgq_linear_int4(x.data(), M, K, N, static_cast<const uint8_t*>(q.qdata.raw()), q.scales.data(), layout,
                             q.group_size, bias_ptr, y.data(), N, static_cast<int>(path), ws, have, nullptr);
    } else {
        rc = sgq_linear_int8(x.data(), M, K, N, static_cast<const int8_t*>(q.qdata.raw()), q.scales.data(), layout,
                             per_tensor(q) ? SGQ_PER_TENSOR : SGQ_PER_ROW, bias_ptr, y.data(), N, static_cast<int>(path), ws,
                             have, nullptr);
    }
    check(rc, "quantized_matmul");
    return y;
}

}  // namespace

Tensor QuantizedTensor::codes_as_float() const {
    require_cuda(qdata, "codes_as_float");
    Tensor out = Tensor::empty(original_shape, Device::CUDA);
    const int64_t n = out.numel();
    check(bits == 8 ? sgq_codes_to_f32_int8(static_cast<const int8_t*>(qdata.raw()), n, out.data(), nullptr)
                    : sgq_codes_to_f32_int4(static_cast<const uint8_t*>(qdata.raw()), n, out.data(), nullptr),
          "codes_as_float");
    return out;
}

QuantizedTensor quantize_int8(const Tensor& x_in, QuantizationScheme scheme) {
    require_cuda(x_in, "quantize_int8");
    Tensor x = f32_contiguous(x_in);
    const int64_t total = x.numel();
    QuantizedTensor r;
    r.original_shape = x.shape();
    r.scheme = scheme;
    r.bits = 8;
    r.group_size = total;                                                                 // src/quantization.cpp:20
    r.qdata = Tensor::empty(x.shape(), Device::CUDA, DType::Int8);
    const bool tensor_wide = scheme == QuantizationScheme::PerTensorSymmetric || x.shape().size() < 2;   // :22
    const int64_t rows = tensor_wide ? 1 : x.shape()[0];
    const int64_t cols = rows ? total / rows : 0;
    r.scales = Tensor::empty({tensor_wide ? 1 : rows}, Device::CUDA);
    check(sgq_quantize_int8(x.data(), rows, cols, tensor_wide ? SGQ_PER_TENSOR : SGQ_PER_ROW,
                            static_cast<int8_t*>(r.qdata.raw()), r.scales.data(), nullptr),
          "quantize_int8");
    return r;
}

Tensor dequantize_int8(const QuantizedTensor& q) {
    require_cuda(q.qdata, "dequantize_int8");
    Tensor out = Tensor::empty(q.original_shape, Device::CUDA);
    const int64_t total = out.numel();
    const bool tensor_wide = per_tensor(q);
    const int64_t rows = tensor_wide ? 1 : q.original_shape[0];
    check(sgq_dequantize_int8(static_cast<const int8_t*>(q.qdata.raw()), q.scales.data(), rows, rows ? total / rows : 0,
                              tensor_wide ? SGQ_PER_TENSOR : SGQ_PER_ROW, out.data(), nullptr),
          "dequantize_int8");
    return out;
}

QuantizedTensor quantize_int4(const Tensor& x_in, int64_t group_size) {
    require_cuda(x_in, "quantize_int4");
    Tensor x = f32_contiguous(x_in);
    if (group_size <= 0) group_size = 32;                                                 // src/quantization.cpp:118
    const int64_t total = x.numel();
    QuantizedTensor r;
    r.original_shape = x.shape();
    r.scheme = QuantizationScheme::GroupedAsymmetric;                                     // :123 (the math is symmetric)
    r.bits = 4;
    r.group_size = group_size;
    r.qdata = Tensor::empty({(total + 1) / 2}, Device::CUDA, DType::UInt8);
    r.scales = Tensor::empty({(total + group_size - 1) / group_size}, Device::CUDA);
    check(sgq_quantize_int4(x.data(), total, group_size, static_cast<uint8_t*>(r.qdata.raw()), r.scales.data(), nullptr),
          "quantize_int4");
    return r;
}

Tensor dequantize_int4(const QuantizedTensor& q) {
    require_cuda(q.qdata, "dequantize_int4");
    Tensor out = Tensor::empty(q.original_shape, Device::CUDA);
    check(sgq_dequantize_int4(static_cast<const uint8_t*>(q.qdata.raw()), q.scales.data(), out.numel(), q.group_size,
                              out.data(), nullptr),
          "dequantize_int4");
    return out;
}

Tensor quantized_matmul_backward_x(const Tensor& grad_in, const QuantizedTensor& q, ForwardPath path) {
    require_cuda(grad_in, "quantized_matmul_backward_x");
    require_cuda(q.qdata, "quantized_matmul_backward_x");
    if (grad_in.shape().size() != 2 || q.original_shape.size() != 2)
        throw std::runtime_error("matmul currently requires 2D tensors!");
    const bool kn = q.layout == WeightLayout::KN;
    const int64_t K = kn ? q.original_shape[0] : q.original_shape[1];
    const int64_t N = kn ? q.original_shape[1] : q.original_shape[0];
    const int64_t M = grad_in.shape()[0];
    if (grad_in.shape()[1] != N) throw std::runtime_error("Matrix inner dimensions must match for matmul!");
    Tensor dy = f32_contiguous(grad_in);
    Tensor dx = Tensor::empty({M, K}, Device::CUDA);
    const int layout = kn ? SGQ_LAYOUT_KN : SGQ_LAYOUT_NK;
    size_t have = 0;
    void* ws = workspace_of_current_device().get(
        sgq_linear_backward_x_workspace_bytes(q.bits, M, K, N, layout, static_cast<int>(path)), &have);
    const int rc = q.bits == 4
        ? sgq_linear_int4_backward_x(dy.data(), M, K, N, static_cast<const uint8_t*>(q.qdata.raw()), q.scales.data(), layout,
                                     q.group_size, dx.data(), K, static_cast<int>(path), ws, have, nullptr)
        : sgq_linear_int8_backward_x(dy.data(), M, K, N, static_cast<const int8_t*>(q.qdata.raw()), q.scales.data(), layout,
                                     per_tensor(q) ? SGQ_PER_TENSOR : SGQ_PER_ROW, dx.data(), K, static_cast<int>(path), ws, have,
                                     nullptr);
    check(rc, "quantized_matmul_backward_x");
    return dx;
}

QuantizedTensor quantize_activations_int8(const Tensor& x) {
    if (x.shape().size() != 2) throw std::runtime_error("quantize_activations_int8: expected [tokens, features]");
    return quantize_int8(x, QuantizationScheme::PerChannelSymmetric);
}

Tensor quantized_matmul_int8(const Tensor& x, const QuantizedTensor& q, const Tensor& bias, ForwardPath path) {
    if (q.bits != 8) throw std::runtime_error("quantized_matmul_int8: weight is not INT8");
    return forward(x, q, bias, path);
}

Tensor quantized_matmul_int4(const Tensor& x, const QuantizedTensor& q, const Tensor& bias, ForwardPath path) {
    if (q.bits != 4) throw std::runtime_error("quantized_matmul_int4: weight is not INT4");
    return forward(x, q, bias, path);
}

}  // namespace quantization
}  // namespace sovereigngrad
