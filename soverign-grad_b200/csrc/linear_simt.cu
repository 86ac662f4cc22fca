// Tiled fp32 SIMT forward: y = x * deq(W) + bias for any M, K, N, either weight layout, either
// bit width and any INT4 group size.  Each output is ONE fused-multiply-add chain over k in
// ascending order with w = (float)code * scale rounded to fp32 first, and the bias is a
// separate fp32 add afterwards — the rounding of the reference's CPU forward
// (src/quantization.cpp:189-206 -> src/ops.cpp:378-455 with include/sovereigngrad/simd.hpp:152-221).
// This is the any-shape path; the decode and prefill kernels take over where they apply.
#include "sgq_common.cuh"

namespace sgq {
namespace {

struct WeightView {
    const void* wq;
    const float* scales;
    int64_t K, N;
    int64_t group;  // INT4
    int scheme;     // INT8
    int layout;
};

template <int BITS>
__device__ __forceinline__ float load_weight(const WeightView& w, int64_t k, int64_t n) {
    const int64_t flat = (w.layout == SGQ_LAYOUT_KN) ? k * w.N + n : n * w.K + k;
    if (BITS == 4) {
        const int c = load_code_int4(static_cast<const uint8_t*>(w.wq), flat);
        return __fmul_rn(static_cast<float>(c), w.scales[flat / w.group]);
    } else {
        const int c = static_cast<const int8_t*>(w.wq)[flat];
        const float s = (w.scheme == SGQ_PER_TENSOR) ? w.scales[0] : w.scales[(w.layout == SGQ_LAYOUT_KN) ? k : n];
        return __fmul_rn(static_cast<float>(c), s);
    }
}

// BM x BN outputs per CTA, BK k per step, 256 threads, TM x TN outputs per thread.
template <int BITS, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__(256) linear_simt_kernel(const float* __restrict__ x, int64_t M, WeightView w,
                                                          const float* __restrict__ bias, float* __restrict__ y,
                                                          int64_t ldy) {
    static_assert((BM / TM) * (BN / TN) == 256, "thread tiling must cover the CTA tile");
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    const int tid = threadIdx.x;
    const int tn = tid % (BN / TN), tm = tid / (BN / TN);
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
    const int64_t K = w.K, N = w.N;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < K; k0 += BK) {
        // x tile: consecutive threads walk k (contiguous in memory)
        for (int e = tid; e < BM * BK; e += 256) {
            const int kk = e % BK, mm = e / BK;
            const int64_t m = m0 + mm, k = k0 + kk;
            xs[kk][mm] = (m < M && k < K) ? x[m * K + k] : 0.0f;
        }
        // weight tile: consecutive threads walk the contiguous dimension of the stored tensor
        for (int e = tid; e < BN * BK; e += 256) {
            int kk, nn;
            if (w.layout == SGQ_LAYOUT_KN) { nn = e % BN; kk = e / BN; } else { kk = e % BK; nn = e / BK; }
            const int64_t n = n0 + nn, k = k0 + kk;
            ws[kk][nn] = (n < N && k < K) ? load_weight<BITS>(w, k, n) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][tm * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tn * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int64_t m = m0 + tm * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int64_t n = n0 + tn * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v = __fadd_rn(v, bias[n]);
            y[m * ldy + n] = v;
        }
    }
}

template <int BITS>
int launch(const LinearArgs& a) {
    WeightView w{a.wq, a.scales, a.K, a.N, a.group, a.scheme, a.layout};
    if (a.M <= 16) {
        constexpr int BM = 16, BN = 64, BK = 32;
        dim3 grid(static_cast<unsigned>(ceil_div(a.N, BN)), static_cast<unsigned>(ceil_div(a.M, BM)));
        linear_simt_kernel<BITS, BM, BN, BK, 2, 2><<<grid, 256, 0, a.stream>>>(a.x, a.M, w, a.bias, a.y, a.ldy);
    } else {
        constexpr int BM = 64, BN = 64, BK = 16;
        dim3 grid(static_cast<unsigned>(ceil_div(a.N, BN)), static_cast<unsigned>(ceil_div(a.M, BM)));
        linear_simt_kernel<BITS, BM, BN, BK, 4, 4><<<grid, 256, 0, a.stream>>>(a.x, a.M, w, a.bias, a.y, a.ldy);
    }
    SGQ_LAUNCH_CHECK("linear_simt_kernel");
    return SGQ_OK;
}

}  // namespace

int launch_linear_simt(const LinearArgs& a) {
    if (a.M == 0 || a.N == 0) return SGQ_OK;
    if (ceil_div(a.M, 16) > 65535) {
        set_error("SIMT path: M=%lld exceeds the grid limit", static_cast<long long>(a.M));
        return SGQ_ERR_UNSUPPORTED;
    }
    return a.bits == 4 ? launch<4>(a) : launch<8>(a);
}

}  // namespace sgq
