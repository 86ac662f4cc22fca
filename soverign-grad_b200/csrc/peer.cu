// Exchange of decode outputs between the GPUs of one box without a collective library: the decode
// kernel stores its output slice into every GPU's full-width output buffer (plain peer stores over
// NVLink, no multicast), and sgq_peer_barrier tells every GPU that all slices have landed.
//
// Signals: every rank owns an array of `world` 64-bit slots in memory that all ranks can write;
// slot r of rank q is written only by rank r.  A barrier publishes this rank's epoch (a counter
// kept in local device memory, +1 per barrier, so recorded launches stay valid) into slot `rank` of
// every rank and waits until each of its own slots has reached the epoch.  Ranks must call the
// barrier the same number of times.  The wait is bounded: if a peer never arrives the kernel
// records kDevErrPeerWait in the status word and returns; the caller reads it on the host.
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
                                                          unsigned long long* local_epoch) {
    const int lane = threadIdx.x;
    pdl_launch_dependents();      // the next kernel may set itself up (and fetch weights); it still waits for this grid
    pdl_wait();                   // the kernel that stored the slices has finished and its stores are visible here
    int late = 0;
    if (!peer_signal_and_wait(sig.p, rank, world, local_epoch, lane, &late) && lane == 0)
        atomicCAS(&g_status_peer, 0u, (kDevErrPeerWait << 24) | 0x10000u);
}

}  // namespace
}  // namespace sgq

using namespace sgq;

extern "C" {

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
                               sig, rank, world, static_cast<unsigned long long*>(local_epoch)));
    return SGQ_OK;
}

}  // extern "C"
