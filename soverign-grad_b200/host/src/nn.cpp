#include "sovereigngrad/nn.hpp"

#include <stdexcept>

namespace sovereigngrad {
namespace nn {

Tensor Linear::forward(const Tensor& x) {
    if (x.shape().size() != 2) throw std::runtime_error("matmul currently requires 2D tensors!");
    const int64_t M = x.shape()[0], K = x.shape()[1], N = W.shape()[1];
    if (K != W.shape()[0]) throw std::runtime_error("Matrix inner dimensions must match for matmul!");
    const std::vector<float> xv = x.to_vector(), wv = W.to_vector(), bv = b.to_vector();
    std::vector<float> out(static_cast<size_t>(M * N));
    for (int64_t i = 0; i < M; ++i)
        for (int64_t j = 0; j < N; ++j) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc = std::fmaf(xv[i * K + k], wv[k * N + j], acc);
            out[i * N + j] = acc + bv[j];
        }
    return Tensor(out, {M, N}, x.device());
}

}  // namespace nn
}  // namespace sovereigngrad
