// Shared helpers of the sm_100a kernels behind include/sgq.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sgq.h"

namespace sgq {

// ---- host side ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);  // records the message, returns SGQ_ERR_CUDA
int sm_count();                                   // SMs of the current device (cached per device)
int check_device();                               // SGQ_ERR_DEVICE unless the current device is compute capability 10.x
int bad(int code, const char* msg);               // records msg, returns code

#define SGQ_CUDA_TRY(expr)                                              \
    do {                                                                \
        cudaError_t _e = (expr);                                        \
        if (_e != cudaSuccess) return ::sgq::cuda_fail(_e, #expr);      \
    } while (0)

#define SGQ_LAUNCH_CHECK(name)                                          \
    do {                                                                \
        cudaError_t _e = cudaGetLastError();                            \
        if (_e != cudaSuccess) return ::sgq::cuda_fail(_e, name);       \
    } while (0)

// Runs cudaFuncSetAttribute(max dynamic shared memory) once per (kernel, device); later calls,
// including those made while a stream is being captured into a graph, touch no CUDA API.
struct SmemOptIn {
    unsigned long long done_mask = 0;   // bit d = attribute set on device d (guarded by the caller's call_once-like use)
    template <typename Kernel>
    cudaError_t ensure(Kernel kernel, int bytes) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const unsigned long long bit = 1ull << (dev & 63);
        if (__atomic_load_n(&done_mask, __ATOMIC_ACQUIRE) & bit) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess) __atomic_fetch_or(&done_mask, bit, __ATOMIC_RELEASE);
        return e;
    }
};

// Process-wide switch (sgq_set_stream_overlap): kernels are launched with programmatic stream
// serialization, so that a kernel's prologue, and for the decode kernel its first weight tiles,
// overlap the tail of the kernel before it in the stream.
bool stream_overlap_enabled();
bool stream_overlap_compact();     // mode 2: the decode kernel also takes its two-CTAs-per-SM form

#ifdef __CUDACC__
// An SM splits one memory between L1 and shared memory, and a CTA cannot join an SM whose running CTAs were placed
// under another split.  A small kernel that a large-shared-memory kernel is meant to run BESIDE (the weight
// expansion in front of the prefill GEMM) must therefore prefer the largest shared-memory split too.  Not applied to
// every kernel: a streaming kernel loses with the small L1 it leaves (the cache attention: 14.8 -> 18 us).  Once
// per kernel and device; a hint only.
void prefer_max_shared(const void* kernel);

// kernel<<<grid, block, smem, stream>>>(args...) with the programmatic-serialization attribute when `overlap`.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool overlap,
                          Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// launchers implemented in the individual .cu files
int launch_quantize_int8(const float* x, int64_t rows, int64_t cols, int scheme, int8_t* codes, float* scales,
                         cudaStream_t s);
int launch_quantize_int4(const float* x, int64_t n, int64_t group, uint8_t* packed, float* scales, cudaStream_t s);
int launch_dequantize_int8(const int8_t* codes, const float* scales, int64_t rows, int64_t cols, int scheme,
                           float* out, cudaStream_t s);
int launch_dequantize_int4(const uint8_t* packed, const float* scales, int64_t n, int64_t group, float* out,
                           cudaStream_t s);
int launch_codes_to_f32(int bits, const void* codes, int64_t n, float* out, cudaStream_t s);
int launch_codes_from_f32(int bits, const float* codes_f32, int64_t n, void* codes, cudaStream_t s);
int launch_interleave(const float* src, int64_t world, int64_t M, int64_t n_local, float* dst, int64_t ldd,
                      cudaStream_t s);

// Output slices written straight into the output buffers of every GPU of the box (this one
// included): y of rank r is p[r].  n == 0: the ordinary single output LinearArgs::y.
constexpr int kMaxPeers = 8;
struct PeerOut {
    float* p[kMaxPeers];
    int n;
    // optional barrier fused into the kernel's tail (sig[0] == nullptr: none): the signal arrays of all
    // ranks, this rank's index, and 16 bytes of local state {u64 epoch, u32 finished-CTA counter}
    unsigned long long* sig[kMaxPeers];
    int rank;
    unsigned long long* state;
    unsigned int poll_budget;   // polls after which a wait for a peer gives up (peer_wait_budget())
    int deferred;               // 1: the tail only signals; the wait for the other ranks happens in the prologue of the
                                // next kernel that uses the same signals (a kernel launched with deferred = 1 itself)
};

// Polls a device-side wait for another GPU may spend before it gives up (sgq_set_peer_wait_budget);
// with the back-off below one poll is 0.1-0.4 us once a wait has lasted more than a few microseconds.
unsigned int peer_wait_budget();

#ifdef __CUDACC__
// The signal slots count: slot [d][r] is the number of signals rank r has sent to rank d, and every rank keeps the
// number it has sent itself (`local_count`; the same on every rank at the same point of the same sequence).
// One warp of ONE CTA: count this CTA's arrival with every rank.  The release makes everything the warp stored
// before (peer stores included: the lanes met at the __syncwarp) visible to a rank that then sees the count, so a
// CTA needs neither a fence of its own nor a last-CTA election, and a rank sees a launch complete as soon as its
// last CTA's count lands.  No waiting.
__device__ __forceinline__ void peer_arrive(unsigned long long* const* sig, int rank, int world, unsigned long long* local_count,
                                            int lane) {
    __syncwarp();
    if (lane < world) asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(sig[lane] + rank), "l"(1ull) : "memory");
    if (lane == 0) atomicAdd(local_count, 1ull);
}

// One warp: wait (bounded) until every rank has published at least the epoch this GPU itself has reached,
// i.e. until every rank has finished the exchanges this GPU has finished.  Returns false on a timeout.
__device__ __forceinline__ bool peer_wait_epoch(const unsigned long long* mine, int world, const unsigned long long* local_epoch,
                                                int lane, unsigned int poll_budget) {
    unsigned long long epoch;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(epoch) : "l"(local_epoch) : "memory");
    bool ok = true;
    if (lane < world) {
        unsigned int polls = 0;
        for (;;) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine + lane) : "memory");
            if (v >= epoch) break;
            if (++polls > poll_budget) {
                ok = false;
                break;
            }
            if (polls > 64) __nanosleep(polls > 4096 ? 400 : 100);
        }
    }
    return __all_sync(0xffffffffu, ok);
}

// One warp: publish this GPU's next epoch to every rank and wait (bounded) until every rank has
// published it here.  Returns false if a peer did not arrive in time.
__device__ __forceinline__ bool peer_signal_and_wait(unsigned long long* const* sig, int rank, int world,
                                                     unsigned long long* local_epoch, int lane, int* late_rank,
                                                     unsigned int poll_budget) {
    unsigned long long epoch = 0;
    if (lane == 0) {
        epoch = *local_epoch + 1;
        *local_epoch = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    __threadfence_system();                       // everything this GPU stored before, peer stores included
    bool ok = true;
    if (lane < world) {
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(sig[lane] + rank), "l"(epoch) : "memory");
        const unsigned long long* mine = sig[rank] + lane;
        unsigned int polls = 0;
        for (;;) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
            if (v >= epoch) break;
            if (++polls > poll_budget) {          // bounded: the caller records the failure and returns
                ok = false;
                *late_rank = lane;
                break;
            }
            if (polls > 64) __nanosleep(polls > 4096 ? 400 : 100);
        }
    }
    return __all_sync(0xffffffffu, ok);
}
#endif

struct LinearArgs {
    const float* x;
    int64_t M, K, N;
    const void* wq;       // packed nibbles (bits 4) or int8 codes (bits 8)
    const float* scales;
    int bits;             // 4 | 8
    int layout;           // SGQ_LAYOUT_*
    int64_t group;        // bits 4: group size (> 0)
    int scheme;           // bits 8: SGQ_PER_*
    const float* bias;    // nullable
    float* y;
    int64_t ldy;
    void* workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
    PeerOut peers;        // decode kernel only
};

int launch_linear_simt(const LinearArgs& a);
bool gemv_supported(const LinearArgs& a);
size_t gemv_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout);
int launch_linear_gemv(const LinearArgs& a);
int launch_linear_gemv_static(LinearArgs a);   // scratch in a file-scope device array
size_t gemv_prepared_bytes(int64_t M, int64_t K);            // 0: no prepared form for this (M, K)
int launch_prepare_x(const float* x, int64_t M, int64_t K, void* prepared, cudaStream_t s);
int launch_linear_gemv_prepared(const LinearArgs& a);        // a.workspace = prepared activations, a.x unused
bool gemv_i8_supported(const LinearArgs& a);                 // INT8 weights stored [N,K], M <= 16
size_t gemv_i8_workspace_bytes(int64_t M, int64_t K);
int launch_linear_gemv_i8(const LinearArgs& a);
bool kn_decode_supported(const LinearArgs& a);               // weights stored [K,N] (the reference module's layout), M <= 16
size_t kn_decode_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N);
int launch_linear_kn_decode(const LinearArgs& a);
bool tc_bf16_supported(int bits, int64_t M, int64_t K, int64_t N, int layout, int64_t group);
size_t tc_bf16_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout);      // preferred (weights expanded)
size_t tc_bf16_min_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout, int64_t group);  // least the path runs with
int launch_linear_tc_bf16(const LinearArgs& a);
bool tc_i8_supported(int64_t M, int64_t K, int64_t N);
size_t tc_i8_workspace_bytes(int64_t M, int64_t K, int64_t N);
int launch_linear_w8a8(const LinearArgs& a, int8_t* xq_out, float* sx_out, int32_t* acc_out);

// ---- device side -------------------------------------------------------------------------
#ifdef __CUDACC__

// std::round: half away from zero.  trunc and the subtraction are exact for every float, so
// this is exact, unlike x + copysign(0.5, x).  NaN and +-Inf pass through.
__device__ __forceinline__ float round_half_away(float v) {
    float t = truncf(v);
    float d = fabsf(v - t);
    return (d >= 0.5f) ? t + copysignf(1.0f, v) : t;
}

// std::max(lo, std::min(hi, v)) with the operand order the reference uses: a NaN becomes +hi.
__device__ __forceinline__ float clamp_like_reference(float v, float lo, float hi) {
    float m = (v < hi) ? v : hi;
    return (lo < m) ? m : lo;
}

// reference: `if (a > max_abs) max_abs = a;` — a NaN never wins; fmaxf has the same property.
__device__ __forceinline__ float absmax_step(float m, float v) { return fmaxf(m, fabsf(v)); }

template <int QMAX, int QMIN>
__device__ __forceinline__ int quantize_code(float v, float inv_scale) {
    float r = round_half_away(__fmul_rn(v, inv_scale));
    return static_cast<int>(clamp_like_reference(r, static_cast<float>(QMIN), static_cast<float>(QMAX)));
}

__device__ __forceinline__ int nibble_signed(uint32_t v4) { return static_cast<int>((v4 & 0xFu) ^ 8u) - 8; }

__device__ __forceinline__ int load_code_int4(const uint8_t* packed, int64_t i) {
    return nibble_signed(static_cast<uint32_t>(packed[i >> 1]) >> ((i & 1) * 4));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

#endif  // __CUDACC__

}  // namespace sgq
