// Exchange of decode outputs between the GPUs of one box without a collective library: the decode
// kernel stores its output slice into every GPU's full-width output buffer (plain peer stores over
// NVLink, no multicast), and sgq_peer_barrier tells every GPU that all slices have landed.
//
// Signals: every rank owns an array of `world` 64-bit slots in memory that all ranks can write;
// slot r of rank q is written only by rank r and counts the signals rank r has sent.  Every rank
// keeps the number it has sent itself in local device memory (so recorded launches stay valid).  A
// barrier adds one to that number, stores it into slot `rank` of every rank and waits until each of
// its own slots has reached it; the deferred form of the fused all-gather (gemv.cu) adds one per
// thread block instead and leaves the waiting to the next kernel.  Ranks must run the same sequence
// of signalling launches.  The wait is bounded (sgq_set_peer_wait_budget): if a peer
// never arrives the kernel records kDevErrPeerWait in the status word and returns; the caller
// reads it on the host (sgq_device_status).
#include "sgq_common.cuh"
#include "sm100_ptx.cuh"

namespace sgq {

__device__ uint32_t g_status_peer = 0;

cudaError_t read_status_peer(uint32_t* v, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(v, g_status_peer, sizeof(uint32_t));
    if (e == cudaSuccess && clear && *v != 0) {
        const uint32_t zero = 0;
        e = cudaMemcpyToSymbol(g_status_peer, &zero, sizeof(zero));
    }
    return e;
}

namespace {

struct PeerSignals {
    unsigned long long* p[kMaxPeers];   // p[r] = the signal array of rank r
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const __grid_constant__ PeerSignals sig, int rank, int world,
                                                          unsigned long long* local_epoch, unsigned int poll_budget) {
    const int lane = threadIdx.x;
    pdl_launch_dependents();      // the next kernel may set itself up (and fetch weights); it still waits for this grid
    pdl_wait();                   // the kernel that stored the slices has finished and its stores are visible here
    int late = 0;
    if (!peer_signal_and_wait(sig.p, rank, world, local_epoch, lane, &late, poll_budget) && lane == 0)
        atomicCAS(&g_status_peer, 0u, (kDevErrPeerWait << 24) | 0x10000u);
}

// src[M, n_local] -> y_r[m * ldy + n] for every rank r (the pointers already include the column offset)
__global__ void __launch_bounds__(256) peer_scatter_kernel(const float* __restrict__ src, int64_t M, int64_t n_local,
                                                           const __grid_constant__ PeerOut peers, int64_t ldy, int vec) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = M * n_local;
    if (vec) {
        for (int64_t i = (blockIdx.x * 256ll + threadIdx.x) * 4; i < total; i += gridDim.x * 1024ll) {
            const int64_t m = i / n_local, n = i - m * n_local;
            const float4 v = *reinterpret_cast<const float4*>(src + i);
            for (int r = 0; r < peers.n; ++r) *reinterpret_cast<float4*>(peers.p[r] + m * ldy + n) = v;
        }
    } else {
        for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
            const int64_t m = i / n_local, n = i - m * n_local;
            const float v = src[i];
            for (int r = 0; r < peers.n; ++r) peers.p[r][m * ldy + n] = v;
        }
    }
}

}  // namespace
}  // namespace sgq

using namespace sgq;

extern "C" {

int sgq_peer_scatter(const float* src, int64_t M, int64_t n_local, float* const* y_ranks, int world, int64_t ldy, int64_t n_offset,
                     void* stream) {
    if (world < 1 || world > kMaxPeers) return bad(SGQ_ERR_BAD_ARGUMENT, "world must be 1..8");
    if (M < 0 || n_local < 0 || n_offset < 0 || ldy < n_offset + n_local) return bad(SGQ_ERR_BAD_SHAPE, "bad slice shape");
    if (M * n_local == 0) return SGQ_OK;
    if (!src || !y_ranks) return bad(SGQ_ERR_NULL_POINTER, "src or y_ranks is NULL");
    PeerOut peers = {};
    bool vec = aligned(src, 16) && (n_offset & 3) == 0 && (n_local & 3) == 0 && (ldy & 3) == 0;
    for (int r = 0; r < world; ++r) {
        if (!y_ranks[r]) return bad(SGQ_ERR_NULL_POINTER, "an output pointer is NULL");
        peers.p[r] = y_ranks[r] + n_offset;
        vec = vec && aligned(y_ranks[r], 16);
    }
    peers.n = world;
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    int64_t blocks = ceil_div(M * n_local, 1024);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    // 128-bit stores when every row on both sides is 16-byte aligned
    SGQ_CUDA_TRY(launch_kernel(peer_scatter_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                               stream_overlap_enabled(), src, M, n_local, peers, ldy, vec ? 1 : 0));
    return SGQ_OK;
}

int sgq_peer_barrier(void* const* signals, int rank, int world, void* local_epoch, void* stream) {
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return bad(SGQ_ERR_BAD_ARGUMENT, "bad rank/world (at most 8 GPUs)");
    if (!signals || !local_epoch) return bad(SGQ_ERR_NULL_POINTER, "signals or local_epoch is NULL");
    PeerSignals sig = {};
    for (int r = 0; r < world; ++r) {
        if (!signals[r] || !aligned(signals[r], 8)) return bad(SGQ_ERR_NULL_POINTER, "a signal array is NULL or misaligned");
        sig.p[r] = static_cast<unsigned long long*>(signals[r]);
    }
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    SGQ_CUDA_TRY(launch_kernel(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), stream_overlap_enabled(),
                               sig, rank, world, static_cast<unsigned long long*>(local_epoch), peer_wait_budget()));
    return SGQ_OK;
}

}  // extern "C"
