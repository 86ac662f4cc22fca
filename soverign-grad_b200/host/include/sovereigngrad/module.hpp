// The slice of the reference's nn::Module (include/sovereigngrad/module.hpp:12-49) that the quantized
// layers use: named parameter registration (`qdata`, `scales`, `bias`) and device placement.
#pragma once

#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "sovereigngrad/tensor.hpp"

namespace sovereigngrad {
namespace nn {

class Module {
public:
    Module() = default;
    virtual ~Module() = default;

    virtual void to(Device device) {
        for (auto& kv : parameters_)
            if (kv.second->is_defined()) *kv.second = kv.second->to(device);
    }
    void cpu() { to(Device::CPU); }
    void cuda() { to(Device::CUDA); }

    virtual Tensor forward(const Tensor& input) { return input; }
    virtual Tensor operator()(const Tensor& input) { return forward(input); }

    void register_parameter(const std::string& name, Tensor& param) { parameters_[name] = &param; }

    std::vector<std::pair<std::string, Tensor>> named_parameters() const {
        std::vector<std::pair<std::string, Tensor>> out;
        for (const auto& kv : parameters_) out.emplace_back(kv.first, *kv.second);
        return out;
    }

protected:
    std::unordered_map<std::string, Tensor*> parameters_;
};

}  // namespace nn
}  // namespace sovereigngrad
