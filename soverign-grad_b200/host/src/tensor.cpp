#include "sovereigngrad/tensor.hpp"

#include <cuda_runtime.h>

#include <cstring>
#include <random>
#include <stdexcept>

namespace sovereigngrad {

namespace {
void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA Error: ") + cudaGetErrorString(e) + " in " + what);
}
}  // namespace

std::vector<int64_t> default_strides(const std::vector<int64_t>& shape) {
    std::vector<int64_t> s(shape.size());
    int64_t acc = 1;
    for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) {
        s[i] = acc;
        acc *= shape[i];
    }
    return s;
}

int64_t compute_numel(const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
}

Storage::Storage(size_t size, Device device, bool zero) : size(size), device(device) {
    ptr = MemoryAllocator::instance().allocate(size, device);
    if (ptr && size > 0 && zero) {
        if (device == Device::CPU) std::memset(ptr, 0, size);
        else cuda_check(cudaMemset(ptr, 0, size), "Storage");
    }
}

Storage::~Storage() { MemoryAllocator::instance().free(ptr, device); }

TensorImpl::TensorImpl(const std::vector<int64_t>& shape, Device device, DType dtype, bool zero)
    : shape(shape), strides(default_strides(shape)), device(device), dtype(dtype) {
    storage = std::make_shared<Storage>(static_cast<size_t>(compute_numel(shape)) * dtype_size(dtype), device, zero);
}

int64_t TensorImpl::numel() const { return compute_numel(shape); }

bool TensorImpl::is_contiguous() const { return shape.empty() || strides == default_strides(shape); }

Tensor::Tensor(const std::vector<int64_t>& shape, Device device, bool requires_grad)
    : impl(std::make_shared<TensorImpl>(shape, device, DType::Float32, true)) {
    impl->requires_grad = requires_grad;
}

Tensor::Tensor(const std::vector<int64_t>& shape, Device device, DType dtype, bool requires_grad)
    : impl(std::make_shared<TensorImpl>(shape, device, dtype, true)) {
    impl->requires_grad = requires_grad;
}

Tensor::Tensor(const std::vector<float>& data, const std::vector<int64_t>& shape, Device device, bool requires_grad) {
    const int64_t total = compute_numel(shape);
    if (data.size() != static_cast<size_t>(total)) throw std::runtime_error("Data size does not match shape!");
    impl = std::make_shared<TensorImpl>(shape, device, DType::Float32, false);
    impl->requires_grad = requires_grad;
    if (total == 0) return;
    if (device == Device::CPU) std::memcpy(impl->raw(), data.data(), sizeof(float) * total);
    else cuda_check(cudaMemcpy(impl->raw(), data.data(), sizeof(float) * total, cudaMemcpyHostToDevice), "Tensor(vector)");
}

Tensor Tensor::empty(const std::vector<int64_t>& shape, Device device, DType dtype) {
    return Tensor(std::make_shared<TensorImpl>(shape, device, dtype, false));
}

Tensor Tensor::zeros(const std::vector<int64_t>& shape, Device device, bool requires_grad) {
    return Tensor(shape, device, requires_grad);
}

Tensor Tensor::full(const std::vector<int64_t>& shape, float value, Device device, bool requires_grad) {
    return Tensor(std::vector<float>(static_cast<size_t>(compute_numel(shape)), value), shape, device, requires_grad);
}

Tensor Tensor::randn(const std::vector<int64_t>& shape, float mean, float std, Device device, bool requires_grad,
                     uint64_t seed) {
    std::mt19937 gen(seed ? static_cast<uint32_t>(seed) : std::random_device{}());
    std::normal_distribution<float> dist(mean, std);
    std::vector<float> v(static_cast<size_t>(compute_numel(shape)));
    for (auto& e : v) e = dist(gen);
    return Tensor(v, shape, device, requires_grad);
}

Tensor Tensor::clone() const {
    if (!impl) return Tensor();
    Tensor src = contiguous();
    Tensor out = Tensor::empty(shape(), device(), dtype());
    const size_t bytes = static_cast<size_t>(numel()) * dtype_size(dtype());
    if (bytes) {
        if (device() == Device::CPU) std::memcpy(out.raw(), src.raw(), bytes);
        else cuda_check(cudaMemcpy(out.raw(), src.raw(), bytes, cudaMemcpyDeviceToDevice), "clone");
    }
    out.impl->requires_grad = impl->requires_grad;
    return out;
}

Tensor Tensor::transpose(int dim0, int dim1) const {
    auto t = std::make_shared<TensorImpl>(*impl);   // shares the storage
    std::swap(t->shape[dim0], t->shape[dim1]);
    std::swap(t->strides[dim0], t->strides[dim1]);
    return Tensor(t);
}

Tensor Tensor::contiguous() const {
    if (!impl || is_contiguous()) return *this;
    // strided gather on the host (on CUDA: through a host copy, as the reference does,
    // src/tensor.cpp:486-510); not on the hot path
    if (dtype() != DType::Float32) throw std::runtime_error("contiguous(): only Float32 views are supported");
    auto base = std::make_shared<TensorImpl>(*impl);
    base->shape = {static_cast<int64_t>(impl->storage->size / sizeof(float))};
    base->strides = {1};
    base->offset = 0;
    std::vector<float> host = Tensor(base).to(Device::CPU).to_vector();
    std::vector<float> out(static_cast<size_t>(numel()));
    const auto& sh = shape();
    const auto& st = strides();
    std::vector<int64_t> idx(sh.size(), 0);
    for (size_t i = 0; i < out.size(); ++i) {
        int64_t off = impl->offset;
        for (size_t d = 0; d < sh.size(); ++d) off += idx[d] * st[d];
        out[i] = host[static_cast<size_t>(off)];
        for (int d = static_cast<int>(sh.size()) - 1; d >= 0; --d) {
            if (++idx[d] < sh[d]) break;
            idx[d] = 0;
        }
    }
    return Tensor(out, sh, device(), requires_grad());
}

Tensor Tensor::to(Device target) const {
    if (!impl) return Tensor();
    if (target == device()) return *this;
    Tensor src = contiguous();
    Tensor out = Tensor::empty(shape(), target, dtype());
    const size_t bytes = static_cast<size_t>(numel()) * dtype_size(dtype());
    if (bytes)
        cuda_check(cudaMemcpy(out.raw(), src.raw(), bytes,
                              target == Device::CUDA ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost), "to");
    out.impl->requires_grad = impl->requires_grad;
    return out;
}

std::vector<float> Tensor::to_vector() const {
    if (dtype() != DType::Float32) throw std::runtime_error("to_vector(): Float32 only");
    Tensor h = contiguous().to(Device::CPU);
    const float* p = h.data();
    return std::vector<float>(p, p + h.numel());
}

Tensor Tensor::operator-(const Tensor& other) const {
    if (shape() != other.shape()) throw std::runtime_error("Incompatible shapes for broadcasting!");
    std::vector<float> a = to_vector(), b = other.to_vector();
    for (size_t i = 0; i < a.size(); ++i) a[i] -= b[i];
    return Tensor(a, shape(), device());
}

float Tensor::get_element(const std::vector<int64_t>& indices) const {
    int64_t off = impl->offset;
    for (size_t d = 0; d < indices.size(); ++d) off += indices[d] * impl->strides[d];
    const float* base = static_cast<const float*>(impl->storage->ptr);
    if (device() == Device::CPU) return base[off];
    float v = 0.0f;
    cuda_check(cudaMemcpy(&v, base + off, sizeof(float), cudaMemcpyDeviceToHost), "get_element");
    return v;
}

}  // namespace sovereigngrad
