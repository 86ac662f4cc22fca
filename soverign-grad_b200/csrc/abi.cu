// extern "C" entry points of include/sgq.h: argument validation, path selection, launches.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <set>
#include <utility>

#include "sgq_common.cuh"
#include "sm100_ptx.cuh"

namespace sgq {

cudaError_t read_status_gemv(uint32_t* v, bool clear);
cudaError_t read_status_gemm(uint32_t* v, bool clear);
cudaError_t read_status_peer(uint32_t* v, bool clear);
cudaError_t read_status_gemv_i8(uint32_t* v, bool clear);

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return SGQ_ERR_CUDA;
}

namespace {
struct DeviceInfo {
    int sms = 0;
    int major = 0;
    bool known = false;
};
DeviceInfo g_devices[64];
std::mutex g_devices_mutex;

const DeviceInfo& device_info() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::lock_guard<std::mutex> lock(g_devices_mutex);
    DeviceInfo& d = g_devices[dev];
    if (!d.known) {
        cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev);
        if (d.sms <= 0) d.sms = 148;
        d.known = true;
    }
    return d;
}
}  // namespace

int sm_count() { return device_info().sms; }

bool make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint32_t rank, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<EncodeFn>(fn);
    });
    if (!encode) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return false;
    }
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], estr[5];
    for (uint32_t i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) st[i] = strides_bytes[i];
    }
    CUresult r = encode(map, dtype, rank, const_cast<void*>(base), d, st, b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (rank=%u dims=%llu,%llu box=%u,%u pitch=%llu)",
                  static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]),
                  static_cast<unsigned long long>(dims[1]), box[0], box[1], static_cast<unsigned long long>(strides_bytes[0]));
        return false;
    }
    return true;
}

bool make_tensor_map_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t inner, uint64_t outer,
                        uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
    const uint64_t dims[2] = {inner, outer};
    const uint64_t strides[1] = {row_pitch_bytes};
    const uint32_t box[2] = {box_inner, box_outer};
    return make_tensor_map(map, dtype, base, 2, dims, strides, box, swizzle);
}

namespace {
int g_stream_overlap = 0;
unsigned int g_peer_wait_budget = 1u << 21;     // about half a second with the back-off of the wait loop
}
unsigned int peer_wait_budget() { return __atomic_load_n(&g_peer_wait_budget, __ATOMIC_RELAXED); }
bool stream_overlap_enabled() { return __atomic_load_n(&g_stream_overlap, __ATOMIC_RELAXED) != 0; }
bool stream_overlap_compact() { return __atomic_load_n(&g_stream_overlap, __ATOMIC_RELAXED) == 2; }

void prefer_max_shared(const void* kernel) {
    static std::mutex mu;
    static std::set<std::pair<int, const void*>> done;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return;
    std::lock_guard<std::mutex> lock(mu);
    if (!done.insert({dev, kernel}).second) return;
    // a preference, not a requirement: a failure changes timing only
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        (void)cudaGetLastError();
}

int check_device() {
    if (device_info().major != 10) {
        set_error("this library contains sm_100a code only; current device is compute capability %d.x",
                  device_info().major);
        return SGQ_ERR_DEVICE;
    }
    return SGQ_OK;
}

int bad(int code, const char* msg) {
    set_error("%s", msg);
    return code;
}

namespace {

int validate_linear(const LinearArgs& a, int path) {
    if (a.M < 0 || a.K < 0 || a.N < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative dimension");
    if (a.ldy < a.N) return bad(SGQ_ERR_BAD_SHAPE, "ldy < N");
    if (a.layout != SGQ_LAYOUT_KN && a.layout != SGQ_LAYOUT_NK) return bad(SGQ_ERR_BAD_ARGUMENT, "unknown layout");
    if (a.bits == 8 && a.scheme != SGQ_PER_TENSOR && a.scheme != SGQ_PER_ROW)
        return bad(SGQ_ERR_BAD_ARGUMENT, "unknown scheme");
    if (path < SGQ_PATH_AUTO || path > SGQ_PATH_TC_I8) return bad(SGQ_ERR_BAD_ARGUMENT, "unknown path");
    if (a.M == 0 || a.N == 0) return SGQ_OK;
    if (!a.y) return bad(SGQ_ERR_NULL_POINTER, "y is NULL");
    if (a.K > 0 && (!a.x || !a.wq || !a.scales)) return bad(SGQ_ERR_NULL_POINTER, "x, weights or scales is NULL");
    if (a.workspace && !aligned(a.workspace, 256)) return bad(SGQ_ERR_WORKSPACE, "workspace is not 256-byte aligned");
    return SGQ_OK;
}

// would AUTO send this (decode-sized) problem to one of the streaming decode kernels?
bool decode_path_ready(const LinearArgs& a) {
    return gemv_supported(a) ||
           (gemv_i8_supported(a) && a.workspace && aligned(a.workspace, 256) && a.workspace_bytes >= gemv_i8_workspace_bytes(a.M, a.K)) ||
           (kn_decode_supported(a) && a.workspace && aligned(a.workspace, 256) &&
            a.workspace_bytes >= kn_decode_workspace_bytes(a.bits, a.M, a.K, a.N));
}

constexpr int64_t kDecodeRows = 16;       // rows one decode launch sequence takes
constexpr int64_t kTensorCoreRows = 64;   // from here on AUTO prefers the tensor-core kernels

int run_linear(LinearArgs a, int path) {
    int rc = validate_linear(a, path);
    if (rc != SGQ_OK) return rc;
    if (a.M == 0 || a.N == 0) return SGQ_OK;
    if ((rc = check_device()) != SGQ_OK) return rc;
    if (a.K == 0) return launch_linear_simt(a);  // y = bias
    if (path == SGQ_PATH_AUTO && a.M > kDecodeRows && a.M < kTensorCoreRows) {
        // Batches between the decode kernels' 16 rows and the tensor-core kernels' 64: blocks of 16 rows on the
        // decode kernels (each block streams the weights once; same fp32 contract as a decode batch) rather
        // than the any-shape kernel.  The blocks run one after the other on the stream and share the workspace.
        LinearArgs blk = a;
        blk.M = kDecodeRows;
        if (decode_path_ready(blk)) {
            for (int64_t m0 = 0; m0 < a.M; m0 += kDecodeRows) {
                LinearArgs sub = a;
                sub.M = a.M - m0 < kDecodeRows ? a.M - m0 : kDecodeRows;
                sub.x = a.x + m0 * a.K;
                sub.y = a.y + m0 * a.ldy;
                if (!decode_path_ready(sub)) return launch_linear_simt(a);      // (cannot happen: fewer rows need less)
                if ((rc = run_linear(sub, SGQ_PATH_GEMV)) != SGQ_OK) return rc;
            }
            return SGQ_OK;
        }
    }
    if (path == SGQ_PATH_AUTO) {
        if (gemv_supported(a) || (gemv_i8_supported(a) && a.workspace && aligned(a.workspace, 256) &&
                                  a.workspace_bytes >= gemv_i8_workspace_bytes(a.M, a.K)) ||
            (kn_decode_supported(a) && a.workspace && aligned(a.workspace, 256) &&
             a.workspace_bytes >= kn_decode_workspace_bytes(a.bits, a.M, a.K, a.N)))
            path = SGQ_PATH_GEMV;
        else if (a.M >= 64 && tc_bf16_supported(a.bits, a.M, a.K, a.N, a.layout, a.group) &&
                 a.workspace && a.workspace_bytes >= tc_bf16_min_workspace_bytes(a.bits, a.M, a.K, a.N, a.layout, a.group) &&
                 aligned(a.wq, 16) && aligned(a.scales, 16) && aligned(a.x, 16))
            path = SGQ_PATH_TC_BF16;
        else
            path = SGQ_PATH_SIMT;
    }
    switch (path) {
        case SGQ_PATH_SIMT:
            return launch_linear_simt(a);
        case SGQ_PATH_GEMV:
            if (a.layout == SGQ_LAYOUT_KN) return launch_linear_kn_decode(a);
            return a.bits == 8 ? launch_linear_gemv_i8(a) : launch_linear_gemv(a);
        case SGQ_PATH_TC_BF16:
            return launch_linear_tc_bf16(a);
        case SGQ_PATH_TC_I8:
            if (a.bits != 8 || a.layout != SGQ_LAYOUT_NK)
                return bad(SGQ_ERR_UNSUPPORTED, "kind::i8 path needs INT8 weights stored [N,K]");
            return launch_linear_w8a8(a, nullptr, nullptr, nullptr);
    }
    return bad(SGQ_ERR_BAD_ARGUMENT, "unknown path");
}

}  // namespace
}  // namespace sgq

using namespace sgq;

extern "C" {

const char* sgq_status_string(int status) {
    switch (status) {
        case SGQ_OK: return "ok";
        case SGQ_ERR_NULL_POINTER: return "null pointer";
        case SGQ_ERR_BAD_SHAPE: return "bad shape";
        case SGQ_ERR_BAD_ARGUMENT: return "bad argument";
        case SGQ_ERR_UNSUPPORTED: return "unsupported by the requested path";
        case SGQ_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
        case SGQ_ERR_ALIGNMENT: return "misaligned pointer";
        case SGQ_ERR_CUDA: return "CUDA error";
        case SGQ_ERR_DEVICE: return "device is not sm_100";
        case SGQ_ERR_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

const char* sgq_last_error(void) { return g_error; }

int sgq_abi_version(void) { return SGQ_ABI_VERSION; }

int sgq_set_stream_overlap(int enabled) {
    return __atomic_exchange_n(&g_stream_overlap, enabled == 2 ? 2 : (enabled ? 1 : 0), __ATOMIC_RELAXED);
}

unsigned int sgq_set_peer_wait_budget(unsigned int polls) {
    return __atomic_exchange_n(&g_peer_wait_budget, polls < 16u ? 16u : polls, __ATOMIC_RELAXED);
}

int sgq_device_status(unsigned int* word, int clear) {
    uint32_t a = 0, b = 0, c = 0, d = 0;
    SGQ_CUDA_TRY(read_status_gemv(&a, clear != 0));
    SGQ_CUDA_TRY(read_status_gemm(&b, clear != 0));
    SGQ_CUDA_TRY(read_status_peer(&c, clear != 0));
    SGQ_CUDA_TRY(read_status_gemv_i8(&d, clear != 0));
    const uint32_t v = a ? a : (b ? b : (c ? c : d));
    if (word) *word = v;
    if (v != 0) {
        set_error("device status word 0x%08x (code %u, detail %u)", v, v >> 24, v & 0xFFFFFFu);
        return SGQ_ERR_TIMEOUT;
    }
    return SGQ_OK;
}

int sgq_quantize_int8(const float* x, int64_t rows, int64_t cols, int scheme, int8_t* codes, float* scales,
                      void* stream) {
    if (rows < 0 || cols < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative dimension");
    if (scheme != SGQ_PER_TENSOR && scheme != SGQ_PER_ROW) return bad(SGQ_ERR_BAD_ARGUMENT, "unknown scheme");
    if (!scales && (scheme == SGQ_PER_TENSOR || rows > 0)) return bad(SGQ_ERR_NULL_POINTER, "scales is NULL");
    if (rows * cols > 0 && (!x || !codes)) return bad(SGQ_ERR_NULL_POINTER, "x or codes is NULL");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    return launch_quantize_int8(x, rows, cols, scheme, codes, scales, static_cast<cudaStream_t>(stream));
}

int sgq_quantize_int4(const float* x, int64_t numel, int64_t group, uint8_t* packed, float* scales, void* stream) {
    if (numel < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative element count");
    if (group <= 0) group = 32;  // src/quantization.cpp:118
    if (numel > 0 && (!x || !packed || !scales)) return bad(SGQ_ERR_NULL_POINTER, "x, packed or scales is NULL");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    return launch_quantize_int4(x, numel, group, packed, scales, static_cast<cudaStream_t>(stream));
}

int sgq_dequantize_int8(const int8_t* codes, const float* scales, int64_t rows, int64_t cols, int scheme, float* out,
                        void* stream) {
    if (rows < 0 || cols < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative dimension");
    if (scheme != SGQ_PER_TENSOR && scheme != SGQ_PER_ROW) return bad(SGQ_ERR_BAD_ARGUMENT, "unknown scheme");
    if (rows * cols > 0 && (!codes || !scales || !out)) return bad(SGQ_ERR_NULL_POINTER, "codes, scales or out is NULL");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    return launch_dequantize_int8(codes, scales, rows, cols, scheme, out, static_cast<cudaStream_t>(stream));
}

int sgq_dequantize_int4(const uint8_t* packed, const float* scales, int64_t numel, int64_t group, float* out,
                        void* stream) {
    if (numel < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative element count");
    if (group <= 0) group = 32;
    if (numel > 0 && (!packed || !scales || !out)) return bad(SGQ_ERR_NULL_POINTER, "packed, scales or out is NULL");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    return launch_dequantize_int4(packed, scales, numel, group, out, static_cast<cudaStream_t>(stream));
}

static int codes_view(int bits, bool to_f32, const void* src, int64_t numel, void* dst, void* stream) {
    if (numel < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative element count");
    if (numel > 0 && (!src || !dst)) return bad(SGQ_ERR_NULL_POINTER, "source or destination is NULL");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return to_f32 ? launch_codes_to_f32(bits, src, numel, static_cast<float*>(dst), s)
                  : launch_codes_from_f32(bits, static_cast<const float*>(src), numel, dst, s);
}

int sgq_codes_to_f32_int8(const int8_t* codes, int64_t numel, float* out, void* stream) {
    return codes_view(8, true, codes, numel, out, stream);
}
int sgq_codes_to_f32_int4(const uint8_t* packed, int64_t numel, float* out, void* stream) {
    return codes_view(4, true, packed, numel, out, stream);
}
int sgq_codes_from_f32_int8(const float* codes_f32, int64_t numel, int8_t* codes, void* stream) {
    return codes_view(8, false, codes_f32, numel, codes, stream);
}
int sgq_codes_from_f32_int4(const float* codes_f32, int64_t numel, uint8_t* packed, void* stream) {
    return codes_view(4, false, codes_f32, numel, packed, stream);
}

size_t sgq_linear_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout, int path) {
    if (M <= 0 || K <= 0 || N <= 0) return 0;
    switch (path) {
        case SGQ_PATH_SIMT: return 0;
        case SGQ_PATH_GEMV:
            if (layout == SGQ_LAYOUT_KN) return kn_decode_workspace_bytes(bits, M, K, N);
            return bits == 8 ? gemv_i8_workspace_bytes(M, K) : gemv_workspace_bytes(bits, M, K, N, layout);
        case SGQ_PATH_TC_BF16: return tc_bf16_workspace_bytes(bits, M, K, N, layout);
        case SGQ_PATH_TC_I8: return tc_i8_workspace_bytes(M, K, N);
        default: {  // AUTO: enough for whichever path AUTO may take
            if (M > 16 && M < 64) M = 16;       // runs as blocks of 16 rows that share the scratch
            size_t a = layout == SGQ_LAYOUT_KN ? kn_decode_workspace_bytes(bits, M, K, N)
                                               : (bits == 8 ? gemv_i8_workspace_bytes(M, K) : gemv_workspace_bytes(bits, M, K, N, layout));
            size_t b = M >= 64 ? tc_bf16_workspace_bytes(bits, M, K, N, layout) : 0;
            return a > b ? a : b;
        }
    }
}

int sgq_linear_int4(const float* x, int64_t M, int64_t K, int64_t N, const uint8_t* packed, const float* scales,
                    int layout, int64_t group, const float* bias, float* y, int64_t ldy, int path, void* workspace,
                    size_t workspace_bytes, void* stream) {
    if (group <= 0) group = 32;
    LinearArgs a{x, M, K, N, packed, scales, 4, layout, group, SGQ_PER_TENSOR, bias, y, ldy, workspace, workspace_bytes,
                 static_cast<cudaStream_t>(stream)};
    return run_linear(a, path);
}

int sgq_linear_int8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* codes, const float* scales,
                    int layout, int scheme, const float* bias, float* y, int64_t ldy, int path, void* workspace,
                    size_t workspace_bytes, void* stream) {
    LinearArgs a{x, M, K, N, codes, scales, 8, layout, 0, scheme, bias, y, ldy, workspace, workspace_bytes,
                 static_cast<cudaStream_t>(stream)};
    return run_linear(a, path);
}

// dx = dy * deq(W) (layout NK) or dy * deq(W)^T (layout KN): the forward of the same stored tensor read with the
// other layout flag (the contraction then runs over the output features N and produces the K input features).
int sgq_linear_int4_backward_x(const float* dy, int64_t M, int64_t K, int64_t N, const uint8_t* packed, const float* scales,
                               int layout, int64_t group, float* dx, int64_t ldx, int path, void* workspace,
                               size_t workspace_bytes, void* stream) {
    if (layout != SGQ_LAYOUT_KN && layout != SGQ_LAYOUT_NK) return bad(SGQ_ERR_BAD_ARGUMENT, "unknown layout");
    return sgq_linear_int4(dy, M, N, K, packed, scales, layout == SGQ_LAYOUT_KN ? SGQ_LAYOUT_NK : SGQ_LAYOUT_KN, group, nullptr, dx,
                           ldx, path, workspace, workspace_bytes, stream);
}

int sgq_linear_int8_backward_x(const float* dy, int64_t M, int64_t K, int64_t N, const int8_t* codes, const float* scales,
                               int layout, int scheme, float* dx, int64_t ldx, int path, void* workspace, size_t workspace_bytes,
                               void* stream) {
    if (layout != SGQ_LAYOUT_KN && layout != SGQ_LAYOUT_NK) return bad(SGQ_ERR_BAD_ARGUMENT, "unknown layout");
    return sgq_linear_int8(dy, M, N, K, codes, scales, layout == SGQ_LAYOUT_KN ? SGQ_LAYOUT_NK : SGQ_LAYOUT_KN, scheme, nullptr, dx,
                           ldx, path, workspace, workspace_bytes, stream);
}

size_t sgq_linear_backward_x_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout, int path) {
    return sgq_linear_workspace_bytes(bits, M, N, K, layout == SGQ_LAYOUT_KN ? SGQ_LAYOUT_NK : SGQ_LAYOUT_KN, path);
}

int sgq_quantize_activations_int8(const float* x, int64_t M, int64_t K, int8_t* xq, float* sx, void* stream) {
    return sgq_quantize_int8(x, M, K, SGQ_PER_ROW, xq, sx, stream);
}

int sgq_linear_int4_decode_noalloc(const float* x, int64_t M, int64_t K, int64_t N, const uint8_t* packed,
                                   const float* scales, const float* bias, float* y, int64_t ldy, void* stream) {
    LinearArgs a{x, M, K, N, packed, scales, 4, SGQ_LAYOUT_NK, 32, SGQ_PER_TENSOR, bias, y, ldy, nullptr, 0,
                 static_cast<cudaStream_t>(stream)};
    int rc = validate_linear(a, SGQ_PATH_GEMV);
    if (rc != SGQ_OK) return rc;
    if (M == 0 || N == 0) return SGQ_OK;
    if ((rc = check_device()) != SGQ_OK) return rc;
    return launch_linear_gemv_static(a);
}

size_t sgq_linear_w8a8_workspace_bytes(int64_t M, int64_t K, int64_t N) {
    if (M <= 0 || K <= 0 || N <= 0) return 0;
    return tc_i8_workspace_bytes(M, K, N);
}

int sgq_linear_w8a8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* codes, const float* scales,
                    int scheme, const float* bias, float* y, int64_t ldy, int8_t* xq_out, float* sx_out,
                    int32_t* acc_out, void* workspace, size_t workspace_bytes, void* stream) {
    LinearArgs a{x, M, K, N, codes, scales, 8, SGQ_LAYOUT_NK, 0, scheme, bias, y, ldy, workspace, workspace_bytes,
                 static_cast<cudaStream_t>(stream)};
    int rc = validate_linear(a, SGQ_PATH_TC_I8);
    if (rc != SGQ_OK) return rc;
    if (M == 0 || N == 0) return SGQ_OK;
    if ((rc = check_device()) != SGQ_OK) return rc;
    return launch_linear_w8a8(a, xq_out, sx_out, acc_out);
}

size_t sgq_prepared_x_bytes(int64_t M, int64_t K) { return gemv_prepared_bytes(M, K); }

int sgq_prepare_x(const float* x, int64_t M, int64_t K, void* prepared, size_t prepared_bytes, void* stream) {
    if (M < 0 || K < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative dimension");
    if (M == 0) return SGQ_OK;
    const size_t need = gemv_prepared_bytes(M, K);
    if (need == 0) return bad(SGQ_ERR_UNSUPPORTED, "no prepared-activation form for this (M, K): M <= 16, K % 256 == 0");
    if (!x || !prepared) return bad(SGQ_ERR_NULL_POINTER, "x or prepared is NULL");
    if (prepared_bytes < need || !aligned(prepared, 256)) return bad(SGQ_ERR_WORKSPACE, "prepared buffer too small or not 256-byte aligned");
    if (!aligned(x, 16)) return bad(SGQ_ERR_ALIGNMENT, "x must be 16-byte aligned");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    return launch_prepare_x(x, M, K, prepared, static_cast<cudaStream_t>(stream));
}

int sgq_linear_int4_prepared(const void* prepared, size_t prepared_bytes, int64_t M, int64_t K, int64_t N, const uint8_t* packed,
                             const float* scales, const float* bias, float* y, int64_t ldy, void* stream) {
    if (M < 0 || K < 0 || N < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative dimension");
    if (ldy < N) return bad(SGQ_ERR_BAD_SHAPE, "ldy < N");
    if (M == 0 || N == 0) return SGQ_OK;
    const size_t need = gemv_prepared_bytes(M, K);
    if (need == 0) return bad(SGQ_ERR_UNSUPPORTED, "no prepared-activation form for this (M, K): M <= 16, K % 256 == 0");
    if (!prepared || !packed || !scales || !y) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    if (prepared_bytes < need || !aligned(prepared, 256)) return bad(SGQ_ERR_WORKSPACE, "prepared buffer too small or not 256-byte aligned");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    LinearArgs a = {};
    a.x = nullptr; a.M = M; a.K = K; a.N = N; a.wq = packed; a.scales = scales; a.bits = 4; a.layout = SGQ_LAYOUT_NK;
    a.group = 32; a.scheme = 0; a.bias = bias; a.y = y; a.ldy = ldy;
    a.workspace = const_cast<void*>(prepared); a.workspace_bytes = prepared_bytes;
    a.stream = static_cast<cudaStream_t>(stream);
    return launch_linear_gemv_prepared(a);
}

static int linear_int4_allgather(const float* x, int64_t M, int64_t K, int64_t N_local, const uint8_t* packed, const float* scales,
                                 const float* bias, float* const* y_ranks, int world, int64_t ldy, int64_t n_offset, void* workspace,
                                 size_t workspace_bytes, void* const* signals, int rank, void* local_state, void* stream, int deferred) {
    if (world < 1 || world > kMaxPeers) return bad(SGQ_ERR_BAD_ARGUMENT, "world must be 1..8");
    if (n_offset < 0 || ldy < n_offset + N_local) return bad(SGQ_ERR_BAD_SHAPE, "ldy < n_offset + N_local");
    if (!y_ranks) return bad(SGQ_ERR_NULL_POINTER, "y_ranks is NULL");
    LinearArgs a{x, M, K, N_local, packed, scales, 4, SGQ_LAYOUT_NK, 32, SGQ_PER_TENSOR, bias, y_ranks[0], ldy, workspace,
                 workspace_bytes, static_cast<cudaStream_t>(stream)};
    for (int r = 0; r < world; ++r) {
        if (!y_ranks[r]) return bad(SGQ_ERR_NULL_POINTER, "an output pointer is NULL");
        a.peers.p[r] = y_ranks[r] + n_offset;
    }
    a.peers.n = world;
    if (signals) {
        if (rank < 0 || rank >= world || !local_state || !aligned(local_state, 8)) return bad(SGQ_ERR_BAD_ARGUMENT, "bad rank or local_state");
        for (int r = 0; r < world; ++r) {
            if (!signals[r] || !aligned(signals[r], 8)) return bad(SGQ_ERR_NULL_POINTER, "a signal array is NULL or misaligned");
            a.peers.sig[r] = static_cast<unsigned long long*>(signals[r]);
        }
        a.peers.rank = rank;
        a.peers.state = static_cast<unsigned long long*>(local_state);
        a.peers.poll_budget = peer_wait_budget();
        a.peers.deferred = deferred;
    } else if (deferred) {
        return bad(SGQ_ERR_NULL_POINTER, "the deferred exchange needs signals and local_state");
    }
    a.y = a.peers.p[0];
    a.ldy = ldy;
    // validate_linear wants ldy >= N for the single-output case; here rows are ldy apart and N_local wide
    if (M >= kTensorCoreRows && tc_bf16_supported(4, M, K, N_local, SGQ_LAYOUT_NK, 32) && workspace &&
        workspace_bytes >= tc_bf16_min_workspace_bytes(4, M, K, N_local, SGQ_LAYOUT_NK, 32)) {
        // Prefill-sized batches: the tcgen05 GEMM's epilogue stores its tiles into every rank's output.  It has no
        // barrier of its own: with signals the barrier kernel follows it on the stream; the deferred form is for
        // decode batches only (its wait sits in the decode kernel's prologue).
        if (deferred) return bad(SGQ_ERR_UNSUPPORTED, "the deferred exchange takes decode batches (M <= 16) only");
        a.peers.sig[0] = nullptr;
        const int rc = run_linear(a, SGQ_PATH_TC_BF16);
        if (rc != SGQ_OK || !signals) return rc;
        return sgq_peer_barrier(signals, rank, world, local_state, stream);
    }
    return run_linear(a, SGQ_PATH_GEMV);
}

int sgq_linear_int4_allgather(const float* x, int64_t M, int64_t K, int64_t N_local, const uint8_t* packed, const float* scales,
                              const float* bias, float* const* y_ranks, int world, int64_t ldy, int64_t n_offset, void* workspace,
                              size_t workspace_bytes, void* const* signals, int rank, void* local_state, void* stream) {
    return linear_int4_allgather(x, M, K, N_local, packed, scales, bias, y_ranks, world, ldy, n_offset, workspace, workspace_bytes,
                                 signals, rank, local_state, stream, 0);
}

int sgq_linear_int4_allgather_deferred(const float* x, int64_t M, int64_t K, int64_t N_local, const uint8_t* packed,
                                       const float* scales, const float* bias, float* const* y_ranks, int world, int64_t ldy,
                                       int64_t n_offset, void* workspace, size_t workspace_bytes, void* const* signals, int rank,
                                       void* local_state, void* stream) {
    return linear_int4_allgather(x, M, K, N_local, packed, scales, bias, y_ranks, world, ldy, n_offset, workspace, workspace_bytes,
                                 signals, rank, local_state, stream, 1);
}

int sgq_interleave_slices(const float* src, int64_t world, int64_t M, int64_t n_local, float* dst, int64_t ldd,
                          void* stream) {
    if (world < 0 || M < 0 || n_local < 0 || ldd < world * n_local) return bad(SGQ_ERR_BAD_SHAPE, "bad slice shape");
    if (world * M * n_local > 0 && (!src || !dst)) return bad(SGQ_ERR_NULL_POINTER, "src or dst is NULL");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    return launch_interleave(src, world, M, n_local, dst, ldd, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
