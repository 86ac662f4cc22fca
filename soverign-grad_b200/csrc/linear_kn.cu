// Decode-shape forward (M <= 16) for weights stored [K, N] — the reference module's own layout
// (nn::QuantizedLinear / QuantizedLinear4Bit keep W as [in, out], include/sovereigngrad/nn.hpp:
// 935-1001) — so that a drop-in user who keeps that layout does not fall onto the any-shape kernel.
//
//   INT4: groups of G consecutive elements of the FLAT tensor, i.e. along N inside a row k when
//         N % G == 0: scale[k][n / G].  The scale depends on k, so the k-sum cannot be taken in
//         integers first (as the [N,K] kernels do); every code is turned into fp32 and multiplied by
//         (x[m,k] * scale): y[m,n] = sum_k (x[m,k] * s[k, n/G]) * code[k,n].
//   INT8: one scale per row k of the stored tensor (per "channel" = input feature) or per tensor:
//         y[m,n] = sum_k (x[m,k] * s[k]) * code[k,n].
//
// HBM-bound streaming of W, coalesced along N: a thread owns 16 consecutive output features (8 packed
// bytes of INT4, 16 bytes of INT8 per k), a CTA 2048 of them, and K is split into slices over the
// second grid dimension so that the whole GPU is busy.  Codes become fp32 without a conversion
// instruction (0x4B000000 | (nibble ^ 8) is 8388608 + 8 + code; one subtraction).  Each slice
// writes its partial sums to scratch; a second kernel adds the slices in ascending order (fixed
// order: run-to-run identical) and the bias.  fp32 throughout; the summation order differs from the
// reference's single chain, the result is inside the 1e-3 contract.
#include "sgq_common.cuh"
#include "sm100_ptx.cuh"

namespace sgq {
namespace {

constexpr int kThreads = 128;
constexpr int kColsPerThread = 16;
constexpr int kColsPerBlock = kThreads * kColsPerThread;   // 2048
constexpr int kMaxSliceK = 256;                            // k per slice (x slice of MB rows sits in shared memory)
constexpr int kMaxM = 16;

template <int BITS>
struct Word;
template <>
struct Word<4> {
    using T = uint2;   // 16 nibbles
};
template <>
struct Word<8> {
    using T = uint4;   // 16 bytes
};

// 16 codes of one k as fp32
template <int BITS>
__device__ __forceinline__ void codes_to_float(const typename Word<BITS>::T& w, float (&c)[16]) {
    if constexpr (BITS == 4) {
        const uint32_t words[2] = {w.x, w.y};
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 8; ++j)
                c[8 * h + j] = __uint_as_float(0x4B000000u | (((words[h] >> (4 * j)) & 0xFu) ^ 8u)) - 8388616.0f;
    } else {
        const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int h = 0; h < 4; ++h)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                c[4 * h + j] = __uint_as_float(0x4B000000u | (((words[h] >> (8 * j)) & 0xFFu) ^ 0x80u)) - 8388736.0f;
    }
}

// scale_mode: 0 = INT4 groups (scales[(k * N + n) / group]), 1 = one scale per k, 2 = one scale
template <int BITS, int MB>
__global__ void __launch_bounds__(kThreads) kn_partial_kernel(const float* __restrict__ x, int64_t K, int64_t N,
                                                              const uint8_t* __restrict__ wq, const float* __restrict__ scales,
                                                              int scale_mode, int64_t group, int slice_k, float* __restrict__ part) {
    __shared__ float xs[MB][kMaxSliceK];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t k0 = static_cast<int64_t>(blockIdx.y) * slice_k;
    const int kn = static_cast<int>((K - k0 < slice_k) ? K - k0 : slice_k);
    for (int i = threadIdx.x; i < MB * kn; i += kThreads) {
        const int m = i / kn, kk = i - m * kn;
        xs[m][kk] = x[static_cast<int64_t>(m) * K + k0 + kk];
    }
    __syncthreads();
    const int64_t n0 = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) * kColsPerThread;
    if (n0 >= N) return;                                     // N % 16 == 0: a thread is in or out as a whole
    float acc[MB][16];
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[m][j] = 0.0f;

    using W = typename Word<BITS>::T;
    const int64_t row_bytes = (BITS == 4) ? N / 2 : N;
    const uint8_t* wp = wq + k0 * row_bytes + ((BITS == 4) ? n0 / 2 : n0);
    const float s_all = (scale_mode == 2) ? __ldg(scales) : 1.0f;
    constexpr int U = 4;                                     // k rows in flight per thread
    for (int kk = 0; kk < kn; kk += U) {
        W w[U];
        float s[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kk + u < kn) ? kk + u : kn - 1;   // clamped: the tail reloads a valid row, its x is zeroed below
            w[u] = __ldcs(reinterpret_cast<const W*>(wp + static_cast<int64_t>(k) * row_bytes));
            if (scale_mode == 0)
                s[u] = __ldg(scales + ((k0 + k) * N + n0) / group);
            else if (scale_mode == 1)
                s[u] = __ldg(scales + k0 + k);
            else
                s[u] = s_all;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float c[16];
            codes_to_float<BITS>(w[u], c);
            const bool live = kk + u < kn;
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const float xsv = live ? xs[m][kk + u] * s[u] : 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[m][j] = fmaf(xsv, c[j], acc[m][j]);
            }
        }
    }
    float* out = part + (static_cast<int64_t>(blockIdx.y) * MB) * N + n0;
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
        for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<float4*>(out + static_cast<int64_t>(m) * N + j) =
                make_float4(acc[m][j], acc[m][j + 1], acc[m][j + 2], acc[m][j + 3]);
}

// y[m, n] = sum over slices (ascending) + bias
__global__ void __launch_bounds__(256) kn_reduce_kernel(const float* __restrict__ part, int slices, int mb, int64_t N,
                                                        const float* __restrict__ bias, float* __restrict__ y, int64_t ldy) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t total = static_cast<int64_t>(mb) * N;
    for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
        const int64_t m = i / N, n = i - m * N;
        float v = 0.0f;
        for (int s = 0; s < slices; ++s) v += __ldcg(part + (static_cast<int64_t>(s) * mb + m) * N + n);
        if (bias) v += bias[n];
        y[m * ldy + n] = v;
    }
}

struct KnPlan {
    int mb;          // batch rows per pass (1, 2 or 4)
    int slice_k;     // k per slice
    int slices;
    int nblocks;
};

KnPlan kn_plan(int64_t M, int64_t K, int64_t N) {
    KnPlan p;
    p.mb = M >= 4 ? 4 : (M >= 2 ? 2 : 1);
    p.nblocks = static_cast<int>(ceil_div(N, kColsPerBlock));
    int64_t want_slices = ceil_div(static_cast<int64_t>(6) * sm_count(), p.nblocks);   // ~6 CTAs of 128 threads per SM
    int64_t sk = ceil_div(K, want_slices);
    sk = (sk + 7) / 8 * 8;
    if (sk < 16) sk = 16;
    if (sk > kMaxSliceK) sk = kMaxSliceK;
    p.slice_k = static_cast<int>(sk);
    p.slices = static_cast<int>(ceil_div(K, sk));
    return p;
}

template <int BITS, int MB>
int launch_pass(const LinearArgs& a, const KnPlan& p, int scale_mode, const float* x, float* y, int rows, float* part) {
    const bool overlap = stream_overlap_enabled();
    SGQ_CUDA_TRY(launch_kernel(kn_partial_kernel<BITS, MB>, dim3(static_cast<unsigned>(p.nblocks), static_cast<unsigned>(p.slices)),
                               dim3(kThreads), 0, a.stream, overlap, x, a.K, a.N, static_cast<const uint8_t*>(a.wq), a.scales,
                               scale_mode, a.group, p.slice_k, part));
    int64_t blocks = ceil_div(static_cast<int64_t>(rows) * a.N, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    SGQ_CUDA_TRY(launch_kernel(kn_reduce_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, a.stream, overlap,
                               static_cast<const float*>(part), p.slices, MB, a.N, a.bias, y, a.ldy));
    (void)rows;
    return SGQ_OK;
}

}  // namespace

bool kn_decode_supported(const LinearArgs& a) {
    if (a.layout != SGQ_LAYOUT_KN || a.M < 1 || a.M > kMaxM || a.K < 1 || a.N < 16 || (a.N % 16) != 0) return false;
    if (a.K >= (1LL << 31) || a.N >= (1LL << 31)) return false;
    if (!aligned(a.wq, 16) || !aligned(a.x, 4)) return false;
    if (a.bits == 4) return a.group >= 16 && (a.group % 16) == 0 && (a.N % a.group) == 0;
    return a.bits == 8;
}

size_t kn_decode_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N) {
    (void)bits;
    if (M < 1 || M > kMaxM || K < 1 || N < 16 || (N % 16) != 0) return 0;
    const KnPlan p = kn_plan(M, K, N);
    return (static_cast<size_t>(p.slices) * p.mb * N * sizeof(float) + 255) / 256 * 256;
}

int launch_linear_kn_decode(const LinearArgs& a) {
    if (!kn_decode_supported(a)) {
        set_error("[K,N] decode path needs M<=16, N%%16==0, INT4 groups that are a multiple of 16 and divide N, 16-byte aligned codes");
        return SGQ_ERR_UNSUPPORTED;
    }
    const size_t need = kn_decode_workspace_bytes(a.bits, a.M, a.K, a.N);
    if (!a.workspace || a.workspace_bytes < need || !aligned(a.workspace, 256)) {
        set_error("[K,N] decode path needs %zu bytes of 256-byte aligned workspace", need);
        return SGQ_ERR_WORKSPACE;
    }
    const KnPlan p = kn_plan(a.M, a.K, a.N);
    const int scale_mode = a.bits == 4 ? 0 : (a.scheme == SGQ_PER_ROW ? 1 : 2);
    float* part = static_cast<float*>(a.workspace);
    // batches larger than the pass width run as several passes over row blocks (weights streamed again)
    for (int64_t m0 = 0; m0 < a.M;) {
        const int64_t left = a.M - m0;
        const int mb = (p.mb == 4 && left >= 4) ? 4 : (left >= 2 && p.mb >= 2 ? 2 : 1);
        const float* x = a.x + m0 * a.K;
        float* y = a.y + m0 * a.ldy;
        int rc;
        if (a.bits == 4)
            rc = mb == 4 ? launch_pass<4, 4>(a, p, scale_mode, x, y, mb, part)
                         : (mb == 2 ? launch_pass<4, 2>(a, p, scale_mode, x, y, mb, part) : launch_pass<4, 1>(a, p, scale_mode, x, y, mb, part));
        else
            rc = mb == 4 ? launch_pass<8, 4>(a, p, scale_mode, x, y, mb, part)
                         : (mb == 2 ? launch_pass<8, 2>(a, p, scale_mode, x, y, mb, part) : launch_pass<8, 1>(a, p, scale_mode, x, y, mb, part));
        if (rc != SGQ_OK) return rc;
        m0 += mb;
    }
    return SGQ_OK;
}

}  // namespace sgq
