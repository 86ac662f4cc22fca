// Host side of the B200 quantization path: the part of the reference's Tensor / Storage
// (include/sovereigngrad/tensor.hpp:13-206, src/tensor.cpp) that the quantized-linear path
// touches — device storage from the pool, shape/stride metadata, host<->device transfer,
// clone/contiguous/transpose — plus the two 8-bit dtypes that packed codes need (the
// reference's DType stops at 16 bits and keeps codes as fp32).  Autograd, the op library and
// everything else of the reference's Tensor are outside this path.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "sovereigngrad/allocator.hpp"

namespace sovereigngrad {

enum class DType { Float32, Float16, Int32, Int64, Int8, UInt8 };

inline std::string dtype_to_string(DType d) {
    switch (d) {
        case DType::Float32: return "Float32";
        case DType::Float16: return "Float16";
        case DType::Int32: return "Int32";
        case DType::Int64: return "Int64";
        case DType::Int8: return "Int8";
        case DType::UInt8: return "UInt8";
        default: return "Unknown";
    }
}

inline size_t dtype_size(DType d) {
    switch (d) {
        case DType::Float16: return 2;
        case DType::Int64: return 8;
        case DType::Int8:
        case DType::UInt8: return 1;
        default: return 4;
    }
}

// Owns `size` bytes from MemoryAllocator::instance(); zero-filled like the reference's
// (src/tensor.cpp:33-42) unless `zero` is false (outputs that a kernel overwrites entirely).
struct Storage {
    void* ptr = nullptr;
    size_t size = 0;
    Device device = Device::CPU;

    Storage(size_t size, Device device, bool zero = true);
    ~Storage();
    Storage(const Storage&) = delete;
    Storage& operator=(const Storage&) = delete;
};

struct TensorImpl {
    std::shared_ptr<Storage> storage;
    std::vector<int64_t> shape;
    std::vector<int64_t> strides;
    int64_t offset = 0;   // in elements of dtype
    Device device = Device::CPU;
    DType dtype = DType::Float32;
    bool requires_grad = false;   // kept for interface parity; this path is inference only

    TensorImpl(const std::vector<int64_t>& shape, Device device, DType dtype, bool zero);

    void* raw() const {
        if (!storage || !storage->ptr) return nullptr;
        return static_cast<char*>(storage->ptr) + offset * static_cast<int64_t>(dtype_size(dtype));
    }
    float* data() const { return static_cast<float*>(raw()); }   // meaningful for Float32 only
    int64_t numel() const;
    bool is_contiguous() const;
};

class Tensor {
public:
    std::shared_ptr<TensorImpl> impl;

    Tensor() : impl(nullptr) {}
    explicit Tensor(std::shared_ptr<TensorImpl> impl) : impl(std::move(impl)) {}
    Tensor(const std::vector<int64_t>& shape, Device device = Device::CPU, bool requires_grad = false);
    Tensor(const std::vector<int64_t>& shape, Device device, DType dtype, bool requires_grad = false);
    Tensor(const std::vector<float>& data, const std::vector<int64_t>& shape, Device device = Device::CPU,
           bool requires_grad = false);

    // uninitialised storage: for outputs a kernel writes completely
    static Tensor empty(const std::vector<int64_t>& shape, Device device, DType dtype = DType::Float32);
    static Tensor zeros(const std::vector<int64_t>& shape, Device device = Device::CPU, bool requires_grad = false);
    static Tensor full(const std::vector<int64_t>& shape, float value, Device device = Device::CPU,
                       bool requires_grad = false);
    // N(mean, std); unlike the reference (src/tensor.cpp:136-153, seeded from random_device on
    // every call) a non-zero `seed` makes the draw reproducible.
    static Tensor randn(const std::vector<int64_t>& shape, float mean = 0.0f, float std = 1.0f,
                        Device device = Device::CPU, bool requires_grad = false, uint64_t seed = 0);

    const std::vector<int64_t>& shape() const { return impl->shape; }
    const std::vector<int64_t>& strides() const { return impl->strides; }
    Device device() const { return impl->device; }
    DType dtype() const { return impl ? impl->dtype : DType::Float32; }
    int64_t numel() const { return impl ? impl->numel() : 0; }
    bool is_contiguous() const { return impl ? impl->is_contiguous() : true; }
    bool is_defined() const { return impl != nullptr; }
    bool defined() const { return impl != nullptr; }
    float* data() const { return impl ? impl->data() : nullptr; }
    void* raw() const { return impl ? impl->raw() : nullptr; }
    bool requires_grad() const { return impl ? impl->requires_grad : false; }

    Tensor clone() const;
    Tensor contiguous() const;
    Tensor transpose(int dim0, int dim1) const;
    Tensor to(Device device) const;   // synchronous copy, like the reference (src/tensor.cpp:330-350)
    Tensor cpu() const { return to(Device::CPU); }
    Tensor cuda() const { return to(Device::CUDA); }

    Tensor operator-(const Tensor& other) const;   // same-shape fp32, computed on the host

    float get_element(const std::vector<int64_t>& indices) const;   // host read (copies one value off the device)
    std::vector<float> to_vector() const;                          // contiguous fp32 copy on the host
};

std::vector<int64_t> default_strides(const std::vector<int64_t>& shape);
int64_t compute_numel(const std::vector<int64_t>& shape);

}  // namespace sovereigngrad
