// TEST INFRASTRUCTURE — not part of the shipped library.
//
// C-ABI driver around the UNMODIFIED SovereignGrad reference sources.  The
// recipe in oracle/Makefile compiles the reference's own .cpp files from where
// they lie (REF=<path to the reference checkout>) together with this file into
// oracle/_ref/libsgref.so.  Nothing from the reference is copied: this file
// only *calls* its public API
//   sovereigngrad::quantization::quantize_int8 / quantize_int4
//   sovereigngrad::quantization::dequantize_int8 / dequantize_int4
//   sovereigngrad::quantization::quantized_matmul_int8 / _int4
//   sovereigngrad::nn::Linear, nn::QuantizedLinear(4Bit)::from_float / forward
// on caller-provided seeded data (the reference's own Tensor::randn cannot be
// seeded, src/tensor.cpp:136-153).
//
// Users: tests/ (checker), tests/golden/make_golden.py (fixture generator) and
// the `cpu_baseline` / `--impl reference` legs of bench.py (timed baseline).
#include "sovereigngrad/nn.hpp"
#include "sovereigngrad/quantization.hpp"
#include "sovereigngrad/safetensors.hpp"
#include "sovereigngrad/serialization.hpp"
#include "sovereigngrad/tensor.hpp"

#include <chrono>
#include <cstdint>
#include <cstring>
#include <exception>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

using namespace sovereigngrad;
namespace q = sovereigngrad::quantization;

namespace {
thread_local std::string g_err;

Tensor from_raw(const float* p, const std::vector<int64_t>& shape) {
    Tensor t(shape, Device::CPU, false);
    std::memcpy(t.impl->data(), p, sizeof(float) * static_cast<size_t>(t.numel()));
    return t;
}
void to_raw(const Tensor& t, float* out) {
    Tensor c = t.to(Device::CPU).contiguous();
    std::memcpy(out, c.impl->data(), sizeof(float) * static_cast<size_t>(c.numel()));
}
q::QuantizationScheme scheme_of(int s) {
    return s == 0 ? q::QuantizationScheme::PerTensorSymmetric : q::QuantizationScheme::PerChannelSymmetric;
}
std::vector<int64_t> shape_of(const int64_t* s, int nd) { return std::vector<int64_t>(s, s + nd); }

struct LinearHandle {
    q::QuantizedTensor qw;   // as produced by the reference quantizer
    Tensor w_t_deq;          // only for layout NK: unused (dequant is redone per call like the reference)
    Tensor bias;             // undefined => no bias
    int bits = 4;
    int layout = 0;          // 0 = [K,N] (module native), 1 = [N,K] (y = x * deq(W)^T)
    int64_t K = 0, N = 0;
};

Tensor forward(const LinearHandle& h, const Tensor& x, bool with_bias) {
    Tensor b = with_bias ? h.bias : Tensor();
    if (h.layout == 0) {
        return h.bits == 8 ? q::quantized_matmul_int8(x, h.qw, b) : q::quantized_matmul_int4(x, h.qw, b);
    }
    // [N,K] convention: the reference API only multiplies by a [K,N] weight, so the
    // dequantized tensor is transposed first; the dequantization still runs per call.
    Tensor deq = h.bits == 8 ? q::dequantize_int8(h.qw) : q::dequantize_int4(h.qw);
    Tensor out = x.matmul(deq.transpose(0, 1).contiguous());
    if (b.is_defined()) out = out + b;
    return out;
}
}  // namespace

#define SGREF_TRY try {
#define SGREF_CATCH                      \
    }                                    \
    catch (const std::exception& e) {    \
        g_err = e.what();                \
        return -1;                       \
    }                                    \
    catch (...) {                        \
        g_err = "unknown exception";     \
        return -1;                       \
    }                                    \
    return 0;

extern "C" {

const char* sgref_last_error() { return g_err.c_str(); }

int sgref_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void sgref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// codes_out: numel floats (the reference keeps integer codes in an fp32 tensor).
// scales_out: 1 (scheme 0 or ndim < 2) or shape[0] floats.  *nscales receives the count.
int sgref_quantize_int8(const float* x, const int64_t* shape, int ndim, int scheme, float* codes_out,
                        float* scales_out, int64_t* nscales) {
    SGREF_TRY
    Tensor t = from_raw(x, shape_of(shape, ndim));
    q::QuantizedTensor r = q::quantize_int8(t, scheme_of(scheme));
    to_raw(r.qdata, codes_out);
    to_raw(r.scales, scales_out);
    if (nscales) *nscales = r.scales.numel();
    SGREF_CATCH
}

int sgref_quantize_int4(const float* x, const int64_t* shape, int ndim, int64_t group, float* codes_out,
                        float* scales_out, int64_t* nscales) {
    SGREF_TRY
    Tensor t = from_raw(x, shape_of(shape, ndim));
    q::QuantizedTensor r = q::quantize_int4(t, group);
    to_raw(r.qdata, codes_out);
    to_raw(r.scales, scales_out);
    if (nscales) *nscales = r.scales.numel();
    SGREF_CATCH
}

int sgref_dequantize_int8(const float* codes, const float* scales, int64_t nscales, const int64_t* shape,
                          int ndim, int scheme, float* out) {
    SGREF_TRY
    q::QuantizedTensor r;
    r.original_shape = shape_of(shape, ndim);
    r.qdata = from_raw(codes, r.original_shape);
    r.scales = from_raw(scales, {nscales});
    r.scheme = scheme_of(scheme);
    r.bits = 8;
    r.group_size = r.qdata.numel();
    to_raw(q::dequantize_int8(r), out);
    SGREF_CATCH
}

int sgref_dequantize_int4(const float* codes, const float* scales, int64_t nscales, const int64_t* shape,
                          int ndim, int64_t group, float* out) {
    SGREF_TRY
    q::QuantizedTensor r;
    r.original_shape = shape_of(shape, ndim);
    r.qdata = from_raw(codes, r.original_shape);
    r.scales = from_raw(scales, {nscales});
    r.scheme = q::QuantizationScheme::GroupedAsymmetric;
    r.bits = 4;
    r.group_size = group <= 0 ? 32 : group;
    to_raw(q::dequantize_int4(r), out);
    SGREF_CATCH
}

// Build a quantized linear from an fp32 weight.
//   layout 0: w is [K,N]; layout 1: w is [N,K].
//   bits 8: scheme 0 per-tensor / 1 per-row of the stored tensor; bits 4: group.
//   bias: N floats or NULL.
// via_module != 0 (layout 0 only) goes through nn::Linear + nn::QuantizedLinear(4Bit)::from_float,
// the path a user of the reference takes (INT8 there is always per-row, nn.hpp:948).
void* sgref_linear_create(const float* w, int layout, int64_t K, int64_t N, int bits, int scheme, int64_t group,
                          const float* bias, int via_module) {
    try {
        auto* h = new LinearHandle();
        h->bits = bits;
        h->layout = layout;
        h->K = K;
        h->N = N;
        std::vector<int64_t> wshape = layout == 0 ? std::vector<int64_t>{K, N} : std::vector<int64_t>{N, K};
        Tensor W = from_raw(w, wshape);
        if (bias) h->bias = from_raw(bias, {1, N});
        if (via_module && layout == 0) {
            nn::Linear lin(K, N, Device::CPU);
            std::memcpy(lin.W.impl->data(), w, sizeof(float) * static_cast<size_t>(K * N));
            if (bias) std::memcpy(lin.b.impl->data(), bias, sizeof(float) * static_cast<size_t>(N));
            if (bits == 8) {
                auto m = nn::QuantizedLinear::from_float(lin);
                h->qw = m->q_weight;
                h->bias = m->bias;
            } else {
                auto m = nn::QuantizedLinear4Bit::from_float(lin, group);
                h->qw = m->q_weight;
                h->bias = m->bias;
            }
        } else {
            h->qw = bits == 8 ? q::quantize_int8(W, scheme_of(scheme)) : q::quantize_int4(W, group);
        }
        return h;
    } catch (const std::exception& e) {
        g_err = e.what();
        return nullptr;
    }
}

void sgref_linear_destroy(void* handle) { delete static_cast<LinearHandle*>(handle); }

int64_t sgref_linear_num_scales(void* handle) { return static_cast<LinearHandle*>(handle)->qw.scales.numel(); }

int sgref_linear_codes(void* handle, float* codes_out, float* scales_out) {
    SGREF_TRY
    auto* h = static_cast<LinearHandle*>(handle);
    to_raw(h->qw.qdata, codes_out);
    to_raw(h->qw.scales, scales_out);
    SGREF_CATCH
}

// y[M,N] = forward(x[M,K]).  The dequantization of the whole weight runs inside every call,
// exactly as in the reference (src/quantization.cpp:189-206).
int sgref_linear_forward(void* handle, const float* x, int64_t M, int with_bias, float* y) {
    SGREF_TRY
    auto* h = static_cast<LinearHandle*>(handle);
    Tensor X = from_raw(x, {M, h->K});
    to_raw(forward(*h, X, with_bias != 0), y);
    SGREF_CATCH
}

// dx[M,K] = gradient of sum(forward(x) * dy) with respect to x, through the reference's own autograd:
// x.requires_grad makes matmul attach a MatmulNode (src/ops.cpp:451-453) whose backward computes
// grad_output.matmul(B^T contiguous) (src/ops.cpp:367-370), B being the dequantized weight.
int sgref_linear_backward_x(void* handle, const float* x, int64_t M, const float* dy, float* dx) {
    SGREF_TRY
    auto* h = static_cast<LinearHandle*>(handle);
    Tensor X = from_raw(x, {M, h->K});
    X.set_requires_grad(true);
    Tensor Y = forward(*h, X, false);
    Tensor DY = from_raw(dy, {M, h->N});
    Tensor loss = sum(Y * DY);
    loss.backward();
    to_raw(X.grad(), dx);
    SGREF_CATCH
}

// Reads one fp32 tensor out of a checkpoint with the reference's own readers: kind 0 = its native format
// (serialization::load_checkpoint, src/serialization.cpp:49-107), kind 1 = SafeTensors
// (safetensors::load_file, src/safetensors.cpp:236-287).  *numel receives the element count.
int sgref_read_tensor(int kind, const char* path, const char* name, float* out, int64_t capacity, int64_t* numel) {
    SGREF_TRY
    std::unordered_map<std::string, Tensor> sd =
        kind == 0 ? serialization::load_checkpoint(path, Device::CPU) : safetensors::load_file(path, Device::CPU);
    auto it = sd.find(name);
    if (it == sd.end()) throw std::runtime_error(std::string("tensor not in file: ") + name);
    if (numel) *numel = it->second.numel();
    if (it->second.numel() > capacity) throw std::runtime_error("output buffer too small");
    to_raw(it->second, out);
    SGREF_CATCH
}

// Times `iters` forwards after one warm-up; returns seconds per forward (<0 on error).
double sgref_linear_time(void* handle, const float* x, int64_t M, int with_bias, int iters) {
    try {
        auto* h = static_cast<LinearHandle*>(handle);
        Tensor X = from_raw(x, {M, h->K});
        Tensor y = forward(*h, X, with_bias != 0);
        auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < iters; ++i) y = forward(*h, X, with_bias != 0);
        auto t1 = std::chrono::steady_clock::now();
        return std::chrono::duration<double>(t1 - t0).count() / (iters > 0 ? iters : 1);
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1.0;
    }
}

// Times the reference quantizer alone; returns seconds per call (<0 on error).
double sgref_quantize_time(const float* x, const int64_t* shape, int ndim, int bits, int scheme, int64_t group,
                           int iters) {
    try {
        Tensor t = from_raw(x, shape_of(shape, ndim));
        auto run = [&]() { return bits == 8 ? q::quantize_int8(t, scheme_of(scheme)) : q::quantize_int4(t, group); };
        q::QuantizedTensor r = run();
        auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < iters; ++i) r = run();
        auto t1 = std::chrono::steady_clock::now();
        return std::chrono::duration<double>(t1 - t0).count() / (iters > 0 ? iters : 1);
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1.0;
    }
}


// ---- decode-glue ops of the reference (used to pin the numpy restatement in oracle/nanollama_oracle.py)
// sovereigngrad::rms_norm (src/ops.cpp:1532), silu (:561), softmax (:2101),
// nn::RotaryEmbedding tables + rotary_embedding (include/sovereigngrad/nn.hpp:583, src/ops.cpp:1714).
int sgref_rms_norm(const float* x, int64_t rows, int64_t D, const float* gamma, float eps, float* out) {
    SGREF_TRY
    to_raw(rms_norm(from_raw(x, {rows, D}), from_raw(gamma, {D}), eps), out);
    SGREF_CATCH
}

int sgref_silu(const float* x, int64_t n, float* out) {
    SGREF_TRY
    to_raw(silu(from_raw(x, {n})), out);
    SGREF_CATCH
}

int sgref_softmax_rows(const float* x, int64_t rows, int64_t cols, float* out) {
    SGREF_TRY
    to_raw(softmax(from_raw(x, {rows, cols}), -1), out);
    SGREF_CATCH
}

int sgref_rope_tables(int64_t head_dim, int64_t max_seq, float base, float* cos_out, float* sin_out) {
    SGREF_TRY
    nn::RotaryEmbedding r(head_dim, max_seq, base, Device::CPU);
    to_raw(r.cos_cached, cos_out);
    to_raw(r.sin_cached, sin_out);
    SGREF_CATCH
}

// x is [T, head_dim] with T <= max_seq, so that the reference's flat table index is the position.
int sgref_rope(const float* x, int64_t T, int64_t head_dim, int64_t max_seq, float base, float* out) {
    SGREF_TRY
    nn::RotaryEmbedding r(head_dim, max_seq, base, Device::CPU);
    to_raw(r.forward(from_raw(x, {T, head_dim})), out);
    SGREF_CATCH
}

// nn::SwiGLU (include/sovereigngrad/nn.hpp:138-160) with caller-provided float weights stored [in, out].
int sgref_swiglu(const float* x, int64_t M, int64_t D, int64_t H, const float* w_gate, const float* w_up,
                 const float* w_down, float* out) {
    SGREF_TRY
    nn::SwiGLU m(D, H, Device::CPU);
    std::memcpy(m.w_gate->W.impl->data(), w_gate, sizeof(float) * D * H);
    std::memcpy(m.w_up->W.impl->data(), w_up, sizeof(float) * D * H);
    std::memcpy(m.w_down->W.impl->data(), w_down, sizeof(float) * D * H);
    to_raw(m.forward(from_raw(x, {M, D})), out);
    SGREF_CATCH
}

}  // extern "C"
