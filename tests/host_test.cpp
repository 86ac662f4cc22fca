// Test driver of the C++ host layer (built by build.py into lib/sgq_host_test).
//
//   sgq_host_test cpu
//       allocator pool on a host-memory stand-in for the device, Tensor metadata, error behaviour.
//       Needs no GPU.  Prints "ok" lines; exit code 0 on success.
//   sgq_host_test gpu <dir> <M> <K> <N> <group>
//       reads <dir>/w.bin ([K,N] fp32), b.bin ([N]), x.bin ([M,K]); runs the flow of the reference's
//       own quantization test (src/test_suite.cpp:672-726): nn::Linear -> QuantizedLinear(4Bit)::
//       from_float -> forward; writes codes, scales and outputs for the caller to compare.
#include <cassert>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include "sovereigngrad/nn.hpp"
#include "sovereigngrad/safetensors.hpp"
#include "sovereigngrad/serialization.hpp"

using namespace sovereigngrad;
namespace q = sovereigngrad::quantization;

#define CHECK(cond)                                                                   \
    do {                                                                              \
        if (!(cond)) {                                                                \
            std::fprintf(stderr, "CHECK failed at %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                             \
        }                                                                             \
    } while (0)

template <typename F>
static bool throws(F f) {
    try {
        f();
    } catch (const std::exception&) {
        return true;
    }
    return false;
}

// ---- a host-memory stand-in for cudaMalloc/cudaFree ------------------------------------------
static size_t g_fake_live = 0, g_fake_calls = 0, g_fake_limit = size_t(1) << 40;
static void* fake_alloc(size_t bytes, int* ordinal) {
    if (g_fake_live + bytes > g_fake_limit) return nullptr;
    *ordinal = 0;
    g_fake_live += bytes;
    ++g_fake_calls;
    void* p = std::aligned_alloc(512, bytes);
    std::memcpy(p, &bytes, sizeof(bytes));   // remember the size for release
    return p;
}
static void fake_release(void* p, int) {
    size_t bytes;
    std::memcpy(&bytes, p, sizeof(bytes));
    g_fake_live -= bytes;
    std::free(p);
}
static const char* fake_error() { return "out of fake device memory"; }

static int run_cpu() {
    auto& A = MemoryAllocator::instance();
    RawBackend fake;
    fake.alloc = fake_alloc;
    fake.release = fake_release;
    fake.last_error = fake_error;
    A.set_cuda_backend(fake);

    // the reference's allocator test (src/test_suite.cpp:52-68), on the CPU pool
    A.reset_peak_memory_stats();
    {
        Tensor a({100, 100}, Device::CPU);
        Tensor b({200, 200}, Device::CPU);
        CHECK(A.active_allocations(Device::CPU) >= 2);
    }
    CHECK(A.cached_allocations(Device::CPU) >= 1);
    CHECK(A.peak_memory_allocated(Device::CPU) > 0);
    CHECK(!A.get_memory_summary(Device::CPU).empty());
    std::puts("ok cpu pool statistics");

    // device pool on the stand-in: segments of 2 MiB, 512-byte alignment, best fit, split, coalesce
    void* p1 = A.allocate(1000, Device::CUDA);
    CHECK(p1 && (reinterpret_cast<uintptr_t>(p1) % 512) == 0);
    CHECK(g_fake_calls == 1 && A.total_memory_allocated(Device::CUDA) == (2u << 20));
    void* p2 = A.allocate(300000, Device::CUDA);
    void* p3 = A.allocate(5000, Device::CUDA);
    CHECK(g_fake_calls == 1);                       // all carved from the first segment
    CHECK(static_cast<char*>(p2) == static_cast<char*>(p1) + 1024);   // 1000 rounds up to 1024
    CHECK(A.active_allocations(Device::CUDA) == 3 && A.cached_allocations(Device::CUDA) == 1);
    A.free(p2, Device::CUDA);
    CHECK(A.cached_allocations(Device::CUDA) == 2);  // hole between p1 and p3 + tail
    void* p4 = A.allocate(200000, Device::CUDA);     // best fit: the hole, not the large tail
    CHECK(p4 == p2);
    A.free(p4, Device::CUDA);
    A.free(p1, Device::CUDA);
    A.free(p3, Device::CUDA);
    CHECK(A.active_allocations(Device::CUDA) == 0);
    CHECK(A.cached_allocations(Device::CUDA) == 1);  // everything merged back into one block
    CHECK(A.peak_memory_allocated(Device::CUDA) >= 1024 + 300032 + 5120);
    void* big = A.allocate(size_t(100) << 20, Device::CUDA);   // own segment
    CHECK(big && g_fake_calls == 2);
    A.free(big, Device::CUDA);
    A.free(big, Device::CUDA);                       // double free and unknown pointers are ignored
    A.free(reinterpret_cast<void*>(0x1234), Device::CUDA);
    CHECK(A.allocate(0, Device::CUDA) == nullptr);
    // out of memory: cached segments go back to the driver, then a runtime_error with the reference's wording
    g_fake_limit = g_fake_live + (1u << 20);
    bool oom = false;
    try {
        A.allocate(size_t(512) << 20, Device::CUDA);
    } catch (const std::runtime_error& e) {
        oom = std::string(e.what()).find("CUDA Allocator Out of Memory") != std::string::npos;
    }
    CHECK(oom);
    CHECK(g_fake_live == 0);                         // the retry released both cached segments
    g_fake_limit = size_t(1) << 40;
    A.release_all();
    CHECK(A.total_memory_allocated(Device::CUDA) == 0 && g_fake_live == 0);
    A.reset_cuda_backend();
    std::puts("ok device pool on the stand-in backend");

    // Tensor metadata on the host
    Tensor t(std::vector<float>{1, 2, 3, 4, 5, 6}, {2, 3});
    CHECK(t.numel() == 6 && t.is_contiguous() && t.strides()[0] == 3);
    Tensor tt = t.transpose(0, 1);
    CHECK(!tt.is_contiguous() && tt.shape()[0] == 3);
    Tensor tc = tt.contiguous();
    CHECK(tc.to_vector() == (std::vector<float>{1, 4, 2, 5, 3, 6}));
    CHECK(t.get_element({1, 2}) == 6.0f);
    CHECK((t - t.clone()).to_vector() == std::vector<float>(6, 0.0f));
    CHECK(throws([] { Tensor(std::vector<float>{1, 2}, {3}); }));            // "Data size does not match shape!"
    CHECK(dtype_size(DType::Int8) == 1 && dtype_size(DType::UInt8) == 1 && dtype_size(DType::Float16) == 2);
    Tensor r1 = Tensor::randn({4, 4}, 0.f, 1.f, Device::CPU, false, 7), r2 = Tensor::randn({4, 4}, 0.f, 1.f, Device::CPU, false, 7);
    CHECK(r1.to_vector() == r2.to_vector());                                 // seeded draws repeat
    std::puts("ok tensor metadata");

    // no CPU path: quantizing a host tensor fails loudly
    CHECK(throws([&] { q::quantize_int4(t, 32); }));
    CHECK(throws([&] { q::quantize_int8(t); }));
    nn::Linear lin(8, 4, Device::CPU, 3);
    CHECK(lin.named_parameters().size() == 2);
    Tensor y = lin.forward(Tensor(std::vector<float>(16, 1.0f), {2, 8}));
    CHECK(y.shape() == (std::vector<int64_t>{2, 4}));
    std::puts("ok no cpu fallback");

    // packed-weight checkpoint: an INT4 and an INT8 tensor as packed codes + scales + metadata
    {
        namespace st = safetensors;
        const std::string path = "/tmp/sgq_host_test_ckpt.safetensors";
        q::QuantizedTensor q4, q8;
        q4.bits = 4; q4.group_size = 32; q4.original_shape = {8, 64}; q4.layout = q::WeightLayout::NK;
        q4.scheme = q::QuantizationScheme::GroupedAsymmetric;
        q4.qdata = Tensor::empty({8 * 64 / 2}, Device::CPU, DType::UInt8);
        q4.scales = Tensor::empty({8 * 64 / 32}, Device::CPU);
        for (int i = 0; i < 256; ++i) static_cast<uint8_t*>(q4.qdata.raw())[i] = static_cast<uint8_t>(i * 37 + 5);
        for (int i = 0; i < 16; ++i) q4.scales.data()[i] = 0.001f * static_cast<float>(i + 1);
        q8.bits = 8; q8.group_size = 15; q8.original_shape = {3, 5};
        q8.scheme = q::QuantizationScheme::PerChannelSymmetric;
        q8.qdata = Tensor::empty({3, 5}, Device::CPU, DType::Int8);
        q8.scales = Tensor::empty({3}, Device::CPU);
        for (int i = 0; i < 15; ++i) static_cast<int8_t*>(q8.qdata.raw())[i] = static_cast<int8_t>(i * 17 - 127);
        for (int i = 0; i < 3; ++i) q8.scales.data()[i] = 0.5f + static_cast<float>(i);
        st::StateDict sd;
        st::Metadata md;
        md["format"] = "sgq \"packed\" v1";
        st::put_quantized("layers.0.w", q4, &sd, &md);
        st::put_quantized("head", q8, &sd, &md);
        sd["bias"] = Tensor(std::vector<float>{1.f, -2.f, 3.5f}, {3});
        st::save_file(sd, path, md);
        st::Metadata md2;
        auto meta = st::inspect_file(path, &md2);
        CHECK(meta.size() == 5 && meta.at("layers.0.w.qdata").dtype == "U8" && meta.at("head.qdata").dtype == "I8");
        CHECK(meta.at("head.qdata").shape == (std::vector<int64_t>{3, 5}) && md2 == md);
        CHECK(meta.at("layers.0.w.qdata").data_offset_end - meta.at("layers.0.w.qdata").data_offset_start == 256);   // 8x less than fp32 codes
        st::Metadata md3;
        st::StateDict back = st::load_file(path, Device::CPU, &md3);
        q::QuantizedTensor r4 = st::get_quantized("layers.0.w", back, md3), r8 = st::get_quantized("head", back, md3);
        CHECK(r4.bits == 4 && r4.group_size == 32 && r4.layout == q::WeightLayout::NK && r4.original_shape == q4.original_shape);
        CHECK(std::memcmp(r4.qdata.raw(), q4.qdata.raw(), 256) == 0 && std::memcmp(r4.scales.raw(), q4.scales.raw(), 64) == 0);
        CHECK(r8.bits == 8 && r8.scheme == q::QuantizationScheme::PerChannelSymmetric && r8.layout == q::WeightLayout::KN);
        CHECK(std::memcmp(r8.qdata.raw(), q8.qdata.raw(), 15) == 0 && r8.scales.to_vector() == q8.scales.to_vector());
        CHECK(back.at("bias").to_vector() == (std::vector<float>{1.f, -2.f, 3.5f}));
        // equal inputs give equal files; malformed files are refused
        st::save_file(sd, path + ".2", md);
        std::ifstream fa(path, std::ios::binary), fb(path + ".2", std::ios::binary);
        std::string ca((std::istreambuf_iterator<char>(fa)), std::istreambuf_iterator<char>());
        std::string cb((std::istreambuf_iterator<char>(fb)), std::istreambuf_iterator<char>());
        CHECK(ca == cb && ca.size() > 8);
        { std::ofstream cut(path + ".3", std::ios::binary); cut.write(ca.data(), static_cast<std::streamsize>(ca.size() - 5)); }
        CHECK(throws([&] { st::load_file(path + ".3"); }));
        CHECK(throws([&] { st::load_file("/tmp/sgq_no_such_file.safetensors"); }));
        md3.erase("head.bits");
        CHECK(throws([&] { st::get_quantized("head", back, md3); }));
        std::remove(path.c_str()); std::remove((path + ".2").c_str()); std::remove((path + ".3").c_str());
        std::puts("ok packed checkpoint");
    }

    // the reference's native ".sgrd" format: version 1 for fp32 state dicts, version 2 with packed tensors
    {
        namespace sz = serialization;
        const std::string path = "/tmp/sgq_host_test_ckpt.sgrd";
        sz::StateDict f32;
        f32["linear.W"] = Tensor(std::vector<float>{1.f, 2.f, 3.f, 4.f, 5.f, 6.f}, {2, 3});
        f32["linear.b"] = Tensor(std::vector<float>{-0.5f, 0.25f, 8.f}, {1, 3});
        sz::save_checkpoint(f32, path);
        {
            std::ifstream f(path, std::ios::binary);
            std::string c((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
            uint32_t version = 0;
            std::memcpy(&version, c.data() + 4, 4);
            CHECK(c.compare(0, 4, "SGRD") == 0 && version == 1);          // what the reference's reader accepts
            // header 12 + (4 + 8 + 4 + 2*8 + 8 + 24) + (4 + 8 + 4 + 2*8 + 8 + 12)
            CHECK(c.size() == 12 + 64 + 52);
        }
        sz::StateDict back = sz::load_checkpoint(path);
        CHECK(back.size() == 2 && back.at("linear.W").shape() == (std::vector<int64_t>{2, 3}));
        CHECK(back.at("linear.W").to_vector() == f32.at("linear.W").to_vector() && back.at("linear.b").to_vector() == f32.at("linear.b").to_vector());

        q::QuantizedTensor q4;
        q4.bits = 4; q4.group_size = 32; q4.original_shape = {4, 64}; q4.layout = q::WeightLayout::NK;
        q4.scheme = q::QuantizationScheme::GroupedAsymmetric;
        q4.qdata = Tensor::empty({4 * 64 / 2}, Device::CPU, DType::UInt8);
        q4.scales = Tensor::empty({4 * 64 / 32}, Device::CPU);
        for (int i = 0; i < 128; ++i) static_cast<uint8_t*>(q4.qdata.raw())[i] = static_cast<uint8_t>(i * 29 + 3);
        for (int i = 0; i < 8; ++i) q4.scales.data()[i] = 0.002f * static_cast<float>(i + 1);
        sz::StateDict packed = f32;
        sz::put_quantized("layers.0.w", q4, &packed);
        sz::save_checkpoint(packed, path + ".2");
        {
            std::ifstream f(path + ".2", std::ios::binary);
            std::string c((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
            uint32_t version = 0;
            std::memcpy(&version, c.data() + 4, 4);
            CHECK(version == 2);
        }
        sz::StateDict pb = sz::load_checkpoint(path + ".2");
        q::QuantizedTensor r4 = sz::get_quantized("layers.0.w", pb);
        CHECK(r4.bits == 4 && r4.group_size == 32 && r4.layout == q::WeightLayout::NK && r4.original_shape == q4.original_shape);
        CHECK(r4.scheme == q::QuantizationScheme::GroupedAsymmetric);
        CHECK(std::memcmp(r4.qdata.raw(), q4.qdata.raw(), 128) == 0 && std::memcmp(r4.scales.raw(), q4.scales.raw(), 32) == 0);
        CHECK(pb.at("linear.b").to_vector() == f32.at("linear.b").to_vector());
        // equal inputs give equal files; malformed files are refused
        sz::save_checkpoint(packed, path + ".3");
        std::ifstream fa(path + ".2", std::ios::binary), fb(path + ".3", std::ios::binary);
        std::string ca((std::istreambuf_iterator<char>(fa)), std::istreambuf_iterator<char>());
        std::string cb((std::istreambuf_iterator<char>(fb)), std::istreambuf_iterator<char>());
        CHECK(ca == cb);
        { std::ofstream cut(path + ".4", std::ios::binary); cut.write(ca.data(), static_cast<std::streamsize>(ca.size() - 7)); }
        CHECK(throws([&] { sz::load_checkpoint(path + ".4"); }));
        { std::ofstream bad(path + ".5", std::ios::binary); bad.write("SGRX\1\0\0\0\0\0\0\0", 12); }
        CHECK(throws([&] { sz::load_checkpoint(path + ".5"); }));
        pb.erase("layers.0.w.qmeta");
        CHECK(throws([&] { sz::get_quantized("layers.0.w", pb); }));
        for (const char* suffix : {"", ".2", ".3", ".4", ".5"}) std::remove((path + suffix).c_str());
        std::puts("ok sgrd checkpoint");
    }
    return 0;
}

// Writes, into `dir`, checkpoints whose fp32 tensors the REFERENCE's own readers must be able to read:
// a version-1 .sgrd file, and a SafeTensors file that also carries a packed INT4 tensor.
static int run_compat(const std::string& dir) {
    namespace sz = serialization;
    namespace st = safetensors;
    sz::StateDict f32;
    std::vector<float> w(6 * 5), b(5);
    for (size_t i = 0; i < w.size(); ++i) w[i] = 0.125f * static_cast<float>(i) - 1.5f;
    for (size_t i = 0; i < b.size(); ++i) b[i] = 1.0f / static_cast<float>(i + 1);
    f32["linear.W"] = Tensor(w, {6, 5});
    f32["linear.b"] = Tensor(b, {1, 5});
    sz::save_checkpoint(f32, dir + "/f32.sgrd");
    st::StateDict sd(f32.begin(), f32.end());
    st::Metadata md;
    q::QuantizedTensor q4;
    q4.bits = 4; q4.group_size = 32; q4.original_shape = {2, 64}; q4.layout = q::WeightLayout::NK;
    q4.scheme = q::QuantizationScheme::GroupedAsymmetric;
    q4.qdata = Tensor::empty({64}, Device::CPU, DType::UInt8);
    q4.scales = Tensor::empty({4}, Device::CPU);
    for (int i = 0; i < 64; ++i) static_cast<uint8_t*>(q4.qdata.raw())[i] = static_cast<uint8_t>(i * 13 + 1);
    for (int i = 0; i < 4; ++i) q4.scales.data()[i] = 0.01f * static_cast<float>(i + 1);
    st::put_quantized("packed.w", q4, &sd, &md);
    st::save_file(sd, dir + "/mixed.safetensors", md);
    std::puts("ok compat files");
    return 0;
}

static std::vector<float> read_f32(const std::string& path, size_t n) {
    std::vector<float> v(n);
    std::ifstream f(path, std::ios::binary);
    if (!f.read(reinterpret_cast<char*>(v.data()), n * sizeof(float))) throw std::runtime_error("cannot read " + path);
    return v;
}
static void write_bytes(const std::string& path, const void* p, size_t n) {
    std::ofstream f(path, std::ios::binary);
    f.write(static_cast<const char*>(p), n);
}
static void dump(const std::string& path, const Tensor& t) {
    Tensor h = t.to(Device::CPU);
    write_bytes(path, h.raw(), static_cast<size_t>(h.numel()) * dtype_size(h.dtype()));
}

static int run_gpu(const std::string& dir, int64_t M, int64_t K, int64_t N, int64_t group) {
    nn::Linear lin(K, N, Device::CPU);
    lin.W = Tensor(read_f32(dir + "/w.bin", K * N), {K, N}, Device::CUDA);
    lin.b = Tensor(read_f32(dir + "/b.bin", N), {1, N}, Device::CUDA);
    Tensor x(read_f32(dir + "/x.bin", M * K), {M, K}, Device::CUDA);

    auto ql8 = nn::QuantizedLinear::from_float(lin);
    auto ql4 = nn::QuantizedLinear4Bit::from_float(lin, group);
    CHECK(ql8->named_parameters().size() == 3 && ql4->named_parameters().size() == 3);
    Tensor y8 = ql8->forward(x), y4 = (*ql4)(x);
    CHECK(y8.shape() == (std::vector<int64_t>{M, N}) && y4.shape() == y8.shape());
    dump(dir + "/q8_codes.bin", ql8->q_weight.qdata);
    dump(dir + "/q8_scales.bin", ql8->q_weight.scales);
    dump(dir + "/q4_packed.bin", ql4->q_weight.qdata);
    dump(dir + "/q4_scales.bin", ql4->q_weight.scales);
    dump(dir + "/y8.bin", y8);
    dump(dir + "/y4.bin", y4);
    dump(dir + "/q4_codes_f32.bin", ql4->q_weight.codes_as_float());
    dump(dir + "/deq8.bin", q::dequantize_int8(ql8->q_weight));
    dump(dir + "/deq4.bin", q::dequantize_int4(ql4->q_weight));

    // per-tensor INT8 and the [N,K] convention through the same API
    auto qt = q::quantize_int8(lin.W, q::QuantizationScheme::PerTensorSymmetric);
    dump(dir + "/q8t_scales.bin", qt.scales);
    dump(dir + "/y8t.bin", q::quantized_matmul_int8(x, qt, lin.b));
    Tensor w_nk = lin.W.transpose(0, 1).contiguous();
    auto nk = nn::QuantizedLinear4Bit::from_weight_nk(w_nk, lin.b, 32);
    dump(dir + "/y4_nk.bin", nk->forward(x));
    dump(dir + "/q4_nk_packed.bin", nk->q_weight.qdata);

    // gradient into x through the frozen layers (upstream gradient: the forward's own output) and dynamic
    // activation quantization
    dump(dir + "/dx4.bin", q::quantized_matmul_backward_x(y4, ql4->q_weight));
    dump(dir + "/dx8.bin", q::quantized_matmul_backward_x(y8, ql8->q_weight, q::ForwardPath::Simt));
    dump(dir + "/dx4_nk.bin", q::quantized_matmul_backward_x(y4, nk->q_weight));
    auto xa = q::quantize_activations_int8(x);
    dump(dir + "/xa_codes.bin", xa.qdata);
    dump(dir + "/xa_scales.bin", xa.scales);
    CHECK(throws([&] { q::quantized_matmul_backward_x(Tensor({M, N + 1}, Device::CUDA), ql4->q_weight); }));

    // packed checkpoints, both container formats: saved from device tensors, loaded straight into pool storage
    // on the device, and the loaded layer computes the same bits
    {
        const size_t before = MemoryAllocator::instance().active_allocations(Device::CUDA);
        serialization::StateDict sd;
        serialization::put_quantized("proj", ql4->q_weight, &sd);
        sd["proj.bias"] = ql4->bias;
        serialization::save_checkpoint(sd, dir + "/packed.sgrd");
        serialization::StateDict back = serialization::load_checkpoint(dir + "/packed.sgrd", Device::CUDA);
        q::QuantizedTensor lq = serialization::get_quantized("proj", back);
        CHECK(lq.qdata.device() == Device::CUDA && lq.scales.device() == Device::CUDA && back.at("proj.bias").device() == Device::CUDA);
        CHECK(MemoryAllocator::instance().active_allocations(Device::CUDA) > before);      // it lives in the device pool
        Tensor y_loaded = q::quantized_matmul_int4(x, lq, back.at("proj.bias"));
        CHECK(y_loaded.to_vector() == y4.to_vector());
        safetensors::StateDict sd2;
        safetensors::Metadata md;
        safetensors::put_quantized("proj", ql8->q_weight, &sd2, &md);
        safetensors::save_file(sd2, dir + "/packed.safetensors", md);
        safetensors::Metadata md2;
        safetensors::StateDict back2 = safetensors::load_file(dir + "/packed.safetensors", Device::CUDA, &md2);
        q::QuantizedTensor lq8 = safetensors::get_quantized("proj", back2, md2);
        CHECK(lq8.qdata.device() == Device::CUDA);
        CHECK(q::quantized_matmul_int8(x, lq8, lin.b).to_vector() == y8.to_vector());
        std::puts("ok packed checkpoints on the device");
    }

    // the tolerance checks of the reference's test (element 0 only, src/test_suite.cpp:719-722)
    Tensor fy = lin.forward(x);
    const float d8 = std::abs((fy - y8).to_vector()[0]), d4 = std::abs((fy - y4).to_vector()[0]);
    std::printf("reference-style check: |float - int8|[0] = %g, |float - int4|[0] = %g\n", d8, d4);
    CHECK(d8 < 0.15f && d4 < 0.35f);

    // error behaviour on the device
    CHECK(throws([&] { q::quantized_matmul_int4(Tensor({M, K + 1}, Device::CUDA), ql4->q_weight, Tensor()); }));
    CHECK(throws([&] { q::quantized_matmul_int4(x, ql8->q_weight, Tensor()); }));
    CHECK(throws([&] { q::quantized_matmul_int8(x, ql8->q_weight, Tensor({1, N + 1}, Device::CUDA)); }));
    std::printf("%s\n", MemoryAllocator::instance().get_memory_summary(Device::CUDA).c_str());
    CHECK(MemoryAllocator::instance().active_allocations(Device::CUDA) > 0);
    std::puts("ok gpu");
    return 0;
}

int main(int argc, char** argv) {
    try {
        if (argc >= 2 && std::string(argv[1]) == "cpu") return run_cpu();
        if (argc >= 3 && std::string(argv[1]) == "compat") return run_compat(argv[2]);
        if (argc >= 7 && std::string(argv[1]) == "gpu")
            return run_gpu(argv[2], std::atoll(argv[3]), std::atoll(argv[4]), std::atoll(argv[5]), std::atoll(argv[6]));
    } catch (const std::exception& e) {
        std::fprintf(stderr, "exception: %s\n", e.what());
        return 2;
    }
    std::fprintf(stderr, "usage: sgq_host_test cpu | compat <dir> | gpu <dir> M K N group\n");
    return 64;
}
