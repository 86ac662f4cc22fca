// fp32 operators between the quantized linears of a decoder block (include/sgq_decoder.h):
// residual add + RMSNorm, rotary embedding + KV-cache store, single-query attention over the
// cache, SiLU gate.  All are HBM/latency bound; none waits on another block, so there is no
// spin anywhere in this file.  The position in the cache is read from device memory so that a
// recorded CUDA graph of a decode step stays valid from step to step.
#include "sgq_common.cuh"
#include "gemv_prepare.cuh"
#include "sm100_ptx.cuh"

#include "../../include/sgq_decoder.h"

#include <cooperative_groups.h>
#include <math_constants.h>

namespace sgq {
namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One block per row.  Pass 1 adds the delta into the residual stream and accumulates the sum of
// squares; pass 2 re-reads the row (L1/L2) and scales it.  The reference sums the squares of a row
// sequentially in fp32 (src/ops.cpp:1546-1550); a tree sum differs from it by a few ulps.
// PREP: the normalised row is also converted to the decode kernel's prepared-activation format.
template <bool PREP>
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                                  const float* __restrict__ gamma, float eps, int64_t dim,
                                                                  float* out, int pmode, int nmain, int nlow, uint8_t* planes) {
    __shared__ float red[kNormThreads / 32];
    __shared__ float inv_rms_s;
    pdl_launch_dependents();
    pdl_wait();
    float* hr = h + blockIdx.x * dim;
    const float* dr = delta ? delta + blockIdx.x * dim : nullptr;
    float* orow = out + blockIdx.x * dim;
    float ss = 0.f;
    if ((dim & 3) == 0) {
        for (int64_t i = threadIdx.x * 4; i < dim; i += kNormThreads * 4) {
            float4 v = *reinterpret_cast<const float4*>(hr + i);
            if (dr) {
                const float4 d = *reinterpret_cast<const float4*>(dr + i);
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
                *reinterpret_cast<float4*>(hr + i) = v;
            }
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int64_t i = threadIdx.x; i < dim; i += kNormThreads) {
            float v = hr[i];
            if (dr) { v += dr[i]; hr[i] = v; }
            ss = fmaf(v, v, ss);
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < kNormThreads / 32 ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) inv_rms_s = 1.0f / sqrtf(t / static_cast<float>(dim) + eps);
    }
    __syncthreads();      // also orders this thread block's writes of h before the re-read below
    const float inv = inv_rms_s;
    if ((dim & 3) == 0) {
        for (int64_t i = threadIdx.x * 4; i < dim; i += kNormThreads * 4) {
            const float4 v = *reinterpret_cast<const float4*>(hr + i);
            const float4 g = *reinterpret_cast<const float4*>(gamma + i);
            float4 o;
            o.x = v.x * inv * g.x; o.y = v.y * inv * g.y; o.z = v.z * inv * g.z; o.w = v.w * inv * g.w;
            *reinterpret_cast<float4*>(orow + i) = o;
        }
    } else {
        for (int64_t i = threadIdx.x; i < dim; i += kNormThreads) orow[i] = hr[i] * inv * gamma[i];
    }
    if (PREP) {
        __syncthreads();                                           // publishes this block's stores of orow
        prepare_row_block<kNormThreads>(orow, blockIdx.x, gridDim.x, dim, pmode, nmain, nlow, planes);
    }
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = (threadIdx.x & 31) < THREADS / 32 ? red[threadIdx.x & 31] : 0.f;
    return warp_sum(t);
}

// The same operator for rows that fit in registers (dim % 256 == 0, dim <= 2048 * CH): the row is read
// once, normalised and, with PREP, converted to digit planes from registers — no pass re-reads memory.
// The decode steps of a model take this form (a few rows, launch- and latency-bound).
template <bool PREP, int CH>
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_row_kernel(float* __restrict__ h, const float* __restrict__ delta,
                                                                      const float* __restrict__ gamma, float eps, int64_t dim,
                                                                      float* __restrict__ out, int pmode, int nmain, int nlow,
                                                                      uint8_t* __restrict__ planes) {
    __shared__ float red[kNormThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const int chunks = static_cast<int>(dim / 8);
    float* hr = h + blockIdx.x * dim;
    const float* dr = delta ? delta + blockIdx.x * dim : nullptr;
    float* orow = out + blockIdx.x * dim;
    float v[CH][8];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < CH; ++r) {
        const int c = threadIdx.x + r * kNormThreads;
        if (c < chunks) {
            float4 a = *(reinterpret_cast<const float4*>(hr) + 2 * c), b = *(reinterpret_cast<const float4*>(hr) + 2 * c + 1);
            if (dr) {
                const float4 da = *(reinterpret_cast<const float4*>(dr) + 2 * c), db = *(reinterpret_cast<const float4*>(dr) + 2 * c + 1);
                a.x += da.x; a.y += da.y; a.z += da.z; a.w += da.w;
                b.x += db.x; b.y += db.y; b.z += db.z; b.w += db.w;
                *(reinterpret_cast<float4*>(hr) + 2 * c) = a;
                *(reinterpret_cast<float4*>(hr) + 2 * c + 1) = b;
            }
            v[r][0] = a.x; v[r][1] = a.y; v[r][2] = a.z; v[r][3] = a.w; v[r][4] = b.x; v[r][5] = b.y; v[r][6] = b.z; v[r][7] = b.w;
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[r][j], v[r][j], ss);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum<kNormThreads>(ss, red) / static_cast<float>(dim) + eps);
#pragma unroll
    for (int r = 0; r < CH; ++r) {
        const int c = threadIdx.x + r * kNormThreads;
        if (c < chunks) {
            const float4 ga = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c), gb = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * c + 1);
            const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[r][j] = v[r][j] * inv * g[j];
            *(reinterpret_cast<float4*>(orow) + 2 * c) = make_float4(v[r][0], v[r][1], v[r][2], v[r][3]);
            *(reinterpret_cast<float4*>(orow) + 2 * c + 1) = make_float4(v[r][4], v[r][5], v[r][6], v[r][7]);
        }
    }
    if (PREP) {
        const PreparedParts pp = prepared_parts(planes, static_cast<size_t>(dim / 32), nmain, nlow);
#pragma unroll
        for (int r = 0; r < CH; ++r) {
            const int c = threadIdx.x + r * kNormThreads;       // chunks % 32 == 0: whole warps
            if (c < chunks) convert_groups<kOrderNibble>(v[r], blockIdx.x, gridDim.x, static_cast<size_t>(c >> 5) * 8, pmode, nmain, nlow, 0.0625f, pp);
        }
    }
}

// One block per token; thread items are (head, d) pairs with d < head_dim / 2.
__global__ void __launch_bounds__(256) rope_kv_store_kernel(float* __restrict__ qkv, int t_new, int n_heads, int head_dim,
                                                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                            const int32_t* __restrict__ pos0, float* __restrict__ kc,
                                                            float* __restrict__ vc, int64_t max_seq) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t m = blockIdx.x;
    const int b = static_cast<int>(m / t_new), i = static_cast<int>(m % t_new);
    const int64_t pos = static_cast<int64_t>(*pos0) + i;
    if (pos < 0 || pos >= max_seq) return;                 // never write outside the cache
    const int half = head_dim >> 1;
    const int64_t dim = static_cast<int64_t>(n_heads) * head_dim;
    float* q = qkv + m * 3 * dim;
    const float* k = q + dim;
    const float* v = k + dim;
    const float* cr = cos_t + pos * half;
    const float* sr = sin_t + pos * half;
    for (int it = threadIdx.x; it < n_heads * half; it += blockDim.x) {
        const int hh = it / half, d = it - hh * half;
        const float c = cr[d], s = sr[d];
        const int o = hh * head_dim + d;
        const float q1 = q[o], q2 = q[o + half];
        q[o] = q1 * c - q2 * s;                             // src/ops.cpp:1737-1738
        q[o + half] = q2 * c + q1 * s;
        const float k1 = k[o], k2 = k[o + half];
        const int64_t co = ((static_cast<int64_t>(b) * n_heads + hh) * max_seq + pos) * head_dim + d;
        kc[co] = k1 * c - k2 * s;
        kc[co + half] = k2 * c + k1 * s;
        vc[co] = v[o];
        vc[co + half] = v[o + half];
    }
}

// Outputs of a column-sharded operator: the slice goes into every GPU's full-width buffer (plain peer stores),
// so no copy kernel is needed between the operator and the barrier.  n == 0: the local output only.
struct PeerPtrs {
    float* p[kMaxPeers];
    int n;
};

constexpr int kAttnWarps = 8;
constexpr int kKeysPerIter = 4;
constexpr int kAttnCtasPerSm = 2;      // 256 threads x <= 128 registers: two sets of key/value rows in flight per warp

// Rotary pair (d, d + HD/2) when a warp holds one head with VEC consecutive elements per lane:
// lane l < 16 holds x1 of the pairs whose x2 sits in lane l + 16.  src/ops.cpp:1737-1738.
template <int VEC>
__device__ __forceinline__ void rope_lanes(float (&v)[VEC], const float* cos_row, const float* sin_row, int lane) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
        const float c = cos_row[(lane & 15) * VEC + j], s = sin_row[(lane & 15) * VEC + j];
        v[j] = (lane < 16) ? v[j] * c - other * s : v[j] * c + other * s;
    }
}

// Decode attention of one new token per sequence, fused with its rotary embedding and KV-cache
// store.  grid (batch * n_heads, S) launched as clusters of S CTAs: the S CTAs of a cluster split
// the cache positions [0, pos) of one (sequence, head); the last one also takes the new token,
// whose rotated key and value come straight from the qkv row (and are appended to the cache for
// later steps).  Each warp walks its keys four at a time with K and V rows loaded together, keeps
// a running max / sum / weighted value (online softmax); warps are merged through shared memory
// and the CTAs of the cluster through distributed shared memory, rank 0 writing the output.
template <int HD, bool PEERS = false>
__global__ void __launch_bounds__(kAttnWarps * 32, kAttnCtasPerSm)
attn_decode_kernel(const float* __restrict__ qkv, int64_t qkv_stride, int n_heads, const float* __restrict__ cos_t,
                   const float* __restrict__ sin_t, float* __restrict__ kc, float* __restrict__ vc, int64_t max_seq,
                   const int32_t* __restrict__ pos0, float* __restrict__ out, int64_t out_stride, int batch, int pmode, int nmain,
                   int nlow, uint8_t* __restrict__ planes, PeerPtrs peers) {
    constexpr int VEC = HD / 32;
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps];
    __shared__ float sm_acc[kAttnWarps][HD];
    __shared__ float sm_part[HD + 2];                      // this CTA's (max, sum, weighted value), read by rank 0
    __shared__ __align__(16) float sm_out[HD];             // rank 0: the finished head, for the prepared form
    const int bh = blockIdx.x, split = blockIdx.y, S = gridDim.y;
    const int b = bh / n_heads, h = bh - b * n_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();                                            // qkv, the caches and *pos0 come from earlier kernels
    int64_t pos = static_cast<int64_t>(*pos0);
    const bool in_range = pos >= 0 && pos < max_seq;       // else: attend to the cache only, store nothing
    pos = pos < 0 ? 0 : (pos > max_seq ? max_seq : pos);
    const int64_t chunk = (pos + S - 1) / S;
    const int64_t t0 = split * chunk;
    const int64_t t1 = (t0 + chunk < pos) ? t0 + chunk : pos;
    const int64_t dim = static_cast<int64_t>(n_heads) * HD;

    const float* row = qkv + static_cast<int64_t>(b) * qkv_stride + h * HD + lane * VEC;
    const float* cos_row = cos_t + (in_range ? pos : 0) * (HD / 2);
    const float* sin_row = sin_t + (in_range ? pos : 0) * (HD / 2);
    float* kb = kc + static_cast<int64_t>(bh) * max_seq * HD + lane * VEC;
    float* vb = vc + static_cast<int64_t>(bh) * max_seq * HD + lane * VEC;

    float qv[VEC];                                         // the rotated, scaled query: filled below, behind the first loads
    float m = -CUDART_INF_F, l = 0.f, acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;

    // Two register sets of key / value rows: the loads of the next four keys are issued before the current four are
    // used, so a warp waits for memory once, not once per iteration.
    auto load_rows = [&](int64_t t, float (&kk)[kKeysPerIter][VEC], float (&vv)[kKeysPerIter][VEC]) {
#pragma unroll
        for (int i = 0; i < kKeysPerIter; ++i) {
            const int64_t tt = (t + i < t1) ? t + i : t1 - 1;          // clamped: the tail reloads a valid row
            if constexpr (VEC == 4) {
                const float4 a = __ldcs(reinterpret_cast<const float4*>(kb + tt * HD));
                const float4 c = __ldcs(reinterpret_cast<const float4*>(vb + tt * HD));
                kk[i][0] = a.x; kk[i][1] = a.y; kk[i][2] = a.z; kk[i][3] = a.w;
                vv[i][0] = c.x; vv[i][1] = c.y; vv[i][2] = c.z; vv[i][3] = c.w;
            } else {
                const float2 a = __ldcs(reinterpret_cast<const float2*>(kb + tt * HD));
                const float2 c = __ldcs(reinterpret_cast<const float2*>(vb + tt * HD));
                kk[i][0] = a.x; kk[i][1] = a.y;
                vv[i][0] = c.x; vv[i][1] = c.y;
            }
        }
    };
    auto use_rows = [&](int64_t t, const float (&kk)[kKeysPerIter][VEC], const float (&vv)[kKeysPerIter][VEC]) {
        float s[kKeysPerIter];
        float mx = m;
#pragma unroll
        for (int i = 0; i < kKeysPerIter; ++i) {
            float d = 0.f;
#pragma unroll
            for (int j = 0; j < VEC; ++j) d = fmaf(qv[j], kk[i][j], d);
            d = warp_sum(d);
            s[i] = (t + i < t1) ? d : -CUDART_INF_F;
            mx = fmaxf(mx, s[i]);
        }
        const float corr = expf(m - mx);                    // m = -inf on the first pass: exp(-inf) = 0
        l *= corr;
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] *= corr;
#pragma unroll
        for (int i = 0; i < kKeysPerIter; ++i) {
            const float p = expf(s[i] - mx);                // 0 for the clamped tail
            l += p;
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[j] = fmaf(p, vv[i][j], acc[j]);
        }
        m = mx;
    };
    {
        constexpr int64_t kStride = kAttnWarps * kKeysPerIter;
        float ka[kKeysPerIter][VEC], va[kKeysPerIter][VEC], kb2[kKeysPerIter][VEC], vb2[kKeysPerIter][VEC];
        int64_t t = t0 + warp * kKeysPerIter;
        // The first cache rows are asked for before anything else: they need the position only, and the query's
        // own loads and rotation (and the new token's, below) then run while those rows are on their way.
        if (t < t1) load_rows(t, ka, va);
#pragma unroll
        for (int j = 0; j < VEC; ++j) qv[j] = row[j];
        const bool appends = split == S - 1 && warp == 0;  // this warp takes the new token
        float kn[VEC], vn[VEC];
        if (appends) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) { kn[j] = row[dim + j]; vn[j] = row[2 * dim + j]; }
        }
        rope_lanes<VEC>(qv, cos_row, sin_row, lane);
        const float scale = rsqrtf(static_cast<float>(HD));
#pragma unroll
        for (int j = 0; j < VEC; ++j) qv[j] *= scale;
        if (appends) {
            // the new token: its key is rotated and both rows are appended to the cache; it is the first key of this
            // warp's running softmax (m = its score, l = 1, acc = its value)
            rope_lanes<VEC>(kn, cos_row, sin_row, lane);
            if (in_range) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) { kb[pos * HD + j] = kn[j]; vb[pos * HD + j] = vn[j]; }
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < VEC; ++j) d = fmaf(qv[j], kn[j], d);
                m = warp_sum(d);
                l = 1.f;
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[j] = vn[j];
            }
        }
        for (; t < t1; t += 2 * kStride) {
            const bool second = t + kStride < t1;
            if (second) load_rows(t + kStride, kb2, vb2);
            use_rows(t, ka, va);
            if (second) {
                if (t + 2 * kStride < t1) load_rows(t + 2 * kStride, ka, va);
                use_rows(t + kStride, kb2, vb2);
            }
        }
    }

    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < VEC; ++j) sm_acc[warp][lane * VEC + j] = acc[j];
    __syncthreads();

    // merge the warps: thread d < HD owns output element d
    if (threadIdx.x < HD) {
        float M = -CUDART_INF_F, L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm_m[w]);
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float wgt = (sm_m[w] == -CUDART_INF_F) ? 0.f : expf(sm_m[w] - M);
            L = fmaf(sm_l[w], wgt, L);
            A = fmaf(sm_acc[w][threadIdx.x], wgt, A);
        }
        sm_part[2 + threadIdx.x] = A;
        if (threadIdx.x == 0) { sm_part[0] = M; sm_part[1] = L; }
    }
    cluster.sync();                                        // every CTA's partial result is in its shared memory
    if (cluster.block_rank() == 0) {
        if (threadIdx.x < HD) {
            float MM = -CUDART_INF_F;
            for (int r = 0; r < S; ++r) MM = fmaxf(MM, cluster.map_shared_rank(sm_part, r)[0]);
            float LL = 0.f, AA = 0.f;
            for (int r = 0; r < S; ++r) {
                const float* rp = cluster.map_shared_rank(sm_part, r);
                const float ms = rp[0];
                const float wgt = (ms == -CUDART_INF_F) ? 0.f : expf(ms - MM);
                LL = fmaf(rp[1], wgt, LL);
                AA = fmaf(rp[2 + threadIdx.x], wgt, AA);
            }
            // LL > 0 whenever there is at least one key; an out-of-range position with an empty cache yields 0
            const float o = LL > 0.f ? AA / LL : 0.f;
            const int64_t at = static_cast<int64_t>(b) * out_stride + h * HD + threadIdx.x;
            if constexpr (PEERS) {
                for (int r = 0; r < peers.n; ++r) peers.p[r][at] = o;
            } else {
                out[at] = o;
            }
            sm_out[threadIdx.x] = o;
        }
        if (planes != nullptr) {
            // the same values as prepared activations of the [batch, n_heads * HD] matrix (gemv_prepare.cuh): a head is
            // HD / 32 whole groups of row b, so the linear behind the attention needs no conversion launch
            __syncthreads();
            if (warp == 0) {
                const bool in = lane < HD / 8;
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = in ? sm_out[lane * 8 + j] : 0.f;
                const PreparedParts pp = prepared_parts(planes, static_cast<size_t>(n_heads) * (HD / 32), nmain, nlow);
                convert_groups<kOrderNibble>(v, b, batch, static_cast<size_t>(h) * (HD / 32), pmode, nmain, nlow, 0.0625f, pp, in);
            }
        }
    }
    cluster.sync();                                        // keep shared memory alive until rank 0 has read it
}

__global__ void __launch_bounds__(256) silu_mul_kernel(const float* __restrict__ gu, int64_t rows, int64_t hidden,
                                                       float* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t n = rows * hidden;
    for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += gridDim.x * 256ll) {
        const int64_t r = i / hidden, c = i - r * hidden;
        const float g = gu[r * 2 * hidden + c], u = gu[r * 2 * hidden + hidden + c];
        out[i] = g / (1.0f + expf(-g)) * u;              // include/sovereigngrad/simd.hpp:103-108, then gate * up
    }
}

// The same with the output slice stored into every GPU's buffer: out_r[r * ld + c] for the local column c (the
// pointers already stand at this rank's column offset).
__global__ void __launch_bounds__(256) silu_mul_peers_kernel(const float* __restrict__ gu, int64_t rows, int64_t hidden, int64_t ld,
                                                             PeerPtrs peers) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t n = rows * hidden;
    for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < n; i += gridDim.x * 256ll) {
        const int64_t r = i / hidden, c = i - r * hidden;
        const float g = gu[r * 2 * hidden + c], u = gu[r * 2 * hidden + hidden + c];
        const float v = g / (1.0f + expf(-g)) * u;
        for (int q = 0; q < peers.n; ++q) peers.p[q][r * ld + c] = v;
    }
}

// One block per row; also converts the row to the decode kernel's prepared-activation format.
__global__ void __launch_bounds__(kNormThreads) silu_mul_prepare_kernel(const float* __restrict__ gu, int64_t hidden, float* out,
                                                                       int pmode, int nmain, int nlow, uint8_t* planes) {
    pdl_launch_dependents();
    pdl_wait();
    const float* g = gu + blockIdx.x * 2 * hidden;
    const float* u = g + hidden;
    float* orow = out + blockIdx.x * hidden;
    for (int64_t i = threadIdx.x * 4; i < hidden; i += kNormThreads * 4) {
        const float4 a = *reinterpret_cast<const float4*>(g + i);
        const float4 b = *reinterpret_cast<const float4*>(u + i);
        float4 o;
        o.x = a.x / (1.0f + expf(-a.x)) * b.x; o.y = a.y / (1.0f + expf(-a.y)) * b.y;
        o.z = a.z / (1.0f + expf(-a.z)) * b.z; o.w = a.w / (1.0f + expf(-a.w)) * b.w;
        *reinterpret_cast<float4*>(orow + i) = o;
    }
    __syncthreads();                                               // publishes this block's stores of orow
    prepare_row_block<kNormThreads>(orow, blockIdx.x, gridDim.x, hidden, pmode, nmain, nlow, planes);
}

// The one-pass form of the same (hidden % 256 == 0): grid (rows, hidden / 1024), a thread owns eight consecutive
// values, i.e. a quarter of a 32-k group, so nothing crosses a warp and a handful of rows still spreads over
// many SMs (one CTA per row took 5.7 us for 8 rows of 5632 in a decode step).
constexpr int kSiluThreads = 128;
__global__ void __launch_bounds__(kSiluThreads) silu_mul_prepare_row_kernel(const float* __restrict__ gu, int64_t hidden,
                                                                           float* __restrict__ out, int pmode, int nmain, int nlow,
                                                                           uint8_t* __restrict__ planes) {
    pdl_launch_dependents();
    pdl_wait();
    const int chunks = static_cast<int>(hidden / 8);
    const int c = blockIdx.y * kSiluThreads + threadIdx.x;
    if (c >= chunks) return;                                    // chunks % 32 == 0: whole warps
    const float* g = gu + blockIdx.x * 2 * hidden;
    const float* u = g + hidden;
    float* orow = out + blockIdx.x * hidden;
    const float4 ga = *(reinterpret_cast<const float4*>(g) + 2 * c), gb = *(reinterpret_cast<const float4*>(g) + 2 * c + 1);
    const float4 ua = *(reinterpret_cast<const float4*>(u) + 2 * c), ub = *(reinterpret_cast<const float4*>(u) + 2 * c + 1);
    const float gg[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
    const float uu[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gg[j] / (1.0f + expf(-gg[j])) * uu[j];
    *(reinterpret_cast<float4*>(orow) + 2 * c) = make_float4(v[0], v[1], v[2], v[3]);
    *(reinterpret_cast<float4*>(orow) + 2 * c + 1) = make_float4(v[4], v[5], v[6], v[7]);
    const PreparedParts pp = prepared_parts(planes, static_cast<size_t>(hidden / 32), nmain, nlow);
    convert_groups<kOrderNibble>(v, blockIdx.x, gridDim.x, static_cast<size_t>(c >> 5) * 8, pmode, nmain, nlow, 0.0625f, pp);
}

// Causal attention of a block of new tokens (the prompt pass): token i of a sequence, at position *pos0 + i,
// attends to the cache positions 0 .. *pos0 + i, which sgqd_rope_kv_store has filled (the new tokens included);
// q comes from the rotated qkv rows.  Online softmax over tiles of keys, as the reference's attention does
// (src/cuda_kernels.cu:1323-1394).  grid (ceil(t_new / 128), batch * heads), 256 threads.  Eight threads share
// a query row, each owning an eighth of the head dimension (16-byte chunk c of a row belongs to thread c % 8,
// so the eight threads read 128 consecutive bytes: no bank conflicts), and every thread carries FOUR queries, so
// that a key or value fetched from shared memory is used four times.  K and V tiles of 16 keys go through
// shared memory and are read by all 128 queries of the block.
constexpr int kPrefillTPQ = 8, kPrefillQPT = 4, kPrefillKeys = 16;
constexpr int kPrefillQ = 256 / kPrefillTPQ * kPrefillQPT;        // 128 queries per block
template <int HD>
__global__ void __launch_bounds__(256) attn_prefill_kernel(const float* __restrict__ qkv, int64_t qkv_stride, int t_new, int n_heads,
                                                           const float* __restrict__ kc, const float* __restrict__ vc,
                                                           int64_t max_seq, const int32_t* __restrict__ pos0,
                                                           float* __restrict__ out, int64_t out_stride) {
    constexpr int TPQ = kPrefillTPQ, QPT = kPrefillQPT, KT = kPrefillKeys;
    constexpr int NC = HD / (4 * TPQ);         // 16-byte chunks of a row per thread
    constexpr int LD = HD + 4;                 // padded row of a shared tile (keeps rows 16-byte aligned)
    __shared__ __align__(16) float ks[KT * LD];
    __shared__ __align__(16) float vs[KT * LD];
    pdl_launch_dependents();
    pdl_wait();
    const int bh = blockIdx.y, b = bh / n_heads, h = bh - b * n_heads;
    const int q0 = blockIdx.x * kPrefillQ;
    const int part = threadIdx.x % TPQ, qrow = threadIdx.x / TPQ;          // queries q0 + qrow + 32 u, u = 0..3
    int64_t p0 = static_cast<int64_t>(*pos0);
    p0 = p0 < 0 ? 0 : p0;
    const float scale = rsqrtf(static_cast<float>(HD));
    float q[QPT][NC * 4], o[QPT][NC * 4], m[QPT], l[QPT];
    bool live[QPT];
#pragma unroll
    for (int u = 0; u < QPT; ++u) {
        const int qi = q0 + qrow + 32 * u;
        live[u] = qi < t_new;
        m[u] = -CUDART_INF_F;
        l[u] = 0.f;
        const float* qr = qkv + (static_cast<int64_t>(b) * t_new + (live[u] ? qi : 0)) * qkv_stride + h * HD + part * 4;
#pragma unroll
        for (int c = 0; c < NC; ++c) {         // registers 4c .. 4c+3 = head dimensions 4 * (part + TPQ * c) .. + 3
            const float4 v = live[u] ? *reinterpret_cast<const float4*>(qr + 4 * TPQ * c) : make_float4(0.f, 0.f, 0.f, 0.f);
            q[u][4 * c] = v.x * scale; q[u][4 * c + 1] = v.y * scale; q[u][4 * c + 2] = v.z * scale; q[u][4 * c + 3] = v.w * scale;
            o[u][4 * c] = o[u][4 * c + 1] = o[u][4 * c + 2] = o[u][4 * c + 3] = 0.f;
        }
    }
    const int last_q = (q0 + kPrefillQ - 1 < t_new - 1) ? q0 + kPrefillQ - 1 : t_new - 1;
    int64_t nk = p0 + last_q + 1;              // keys this block needs
    nk = nk > max_seq ? max_seq : nk;
    const float* kb = kc + static_cast<int64_t>(bh) * max_seq * HD;
    const float* vb = vc + static_cast<int64_t>(bh) * max_seq * HD;
    for (int64_t j0 = 0; j0 < nk; j0 += KT) {
        __syncthreads();                       // the tile of the last round has been read by everyone
        for (int it = threadIdx.x; it < KT * (HD / 4); it += 256) {
            const int r = it / (HD / 4), c = (it - r * (HD / 4)) * 4;
            const int64_t j = (j0 + r < nk) ? j0 + r : nk - 1;                         // clamped: masked below
            *reinterpret_cast<float4*>(ks + r * LD + c) = __ldg(reinterpret_cast<const float4*>(kb + j * HD + c));
            *reinterpret_cast<float4*>(vs + r * LD + c) = __ldg(reinterpret_cast<const float4*>(vb + j * HD + c));
        }
        __syncthreads();
        float sc[QPT][KT];
#pragma unroll
        for (int jj = 0; jj < KT; ++jj) {
            float dot[QPT];
#pragma unroll
            for (int u = 0; u < QPT; ++u) dot[u] = 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float4 kv = *reinterpret_cast<const float4*>(ks + jj * LD + (part + TPQ * c) * 4);
#pragma unroll
                for (int u = 0; u < QPT; ++u)
                    dot[u] = fmaf(q[u][4 * c], kv.x, fmaf(q[u][4 * c + 1], kv.y, fmaf(q[u][4 * c + 2], kv.z, fmaf(q[u][4 * c + 3], kv.w, dot[u]))));
            }
#pragma unroll
            for (int u = 0; u < QPT; ++u) {
                float d = dot[u];
                d += __shfl_xor_sync(0xffffffffu, d, 1);
                d += __shfl_xor_sync(0xffffffffu, d, 2);
                d += __shfl_xor_sync(0xffffffffu, d, 4);
                const int64_t jmax = p0 + q0 + qrow + 32 * u;                           // last key of this query
                sc[u][jj] = (live[u] && j0 + jj <= jmax && j0 + jj < nk) ? d : -CUDART_INF_F;
            }
        }
#pragma unroll
        for (int u = 0; u < QPT; ++u) {
            float tmax = -CUDART_INF_F;
#pragma unroll
            for (int jj = 0; jj < KT; ++jj) tmax = fmaxf(tmax, sc[u][jj]);
            const float m_new = fmaxf(m[u], tmax);
            // a query whose every key so far is masked keeps m = -inf: its weights and its rescaling are zero
            const float alpha = (m_new == -CUDART_INF_F) ? 0.f : expf(m[u] - m_new);
            l[u] *= alpha;
#pragma unroll
            for (int d = 0; d < NC * 4; ++d) o[u][d] *= alpha;
#pragma unroll
            for (int jj = 0; jj < KT; ++jj) {
                sc[u][jj] = (m_new == -CUDART_INF_F) ? 0.f : expf(sc[u][jj] - m_new);   // the score becomes its weight; 0 for masked keys
                l[u] += sc[u][jj];
            }
            m[u] = m_new;
        }
#pragma unroll
        for (int jj = 0; jj < KT; ++jj) {
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const float4 vv = *reinterpret_cast<const float4*>(vs + jj * LD + (part + TPQ * c) * 4);
#pragma unroll
                for (int u = 0; u < QPT; ++u) {
                    o[u][4 * c] = fmaf(sc[u][jj], vv.x, o[u][4 * c]);
                    o[u][4 * c + 1] = fmaf(sc[u][jj], vv.y, o[u][4 * c + 1]);
                    o[u][4 * c + 2] = fmaf(sc[u][jj], vv.z, o[u][4 * c + 2]);
                    o[u][4 * c + 3] = fmaf(sc[u][jj], vv.w, o[u][4 * c + 3]);
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < QPT; ++u) {
        if (!live[u]) continue;
        const int qi = q0 + qrow + 32 * u;
        const float inv = l[u] > 0.f ? 1.0f / l[u] : 0.f;
        float* orow = out + (static_cast<int64_t>(b) * t_new + qi) * out_stride + h * HD + part * 4;
#pragma unroll
        for (int c = 0; c < NC; ++c)
            *reinterpret_cast<float4*>(orow + 4 * TPQ * c) =
                make_float4(o[u][4 * c] * inv, o[u][4 * c + 1] * inv, o[u][4 * c + 2] * inv, o[u][4 * c + 3] * inv);
    }
}

// The same causal attention on the tensor cores (head dimension 128), for prompt passes whose linears run on the
// bf16 tensor-core path anyway: q, k, v and the softmax weights are rounded to bf16, scores and outputs accumulate in
// fp32 (mma.sync m16n8k16), the softmax itself is fp32.  grid (ceil(t_new / 64), batch * heads), 128 threads: a
// warp owns 16 query rows, their q fragments live in registers; K and V tiles of 64 keys are converted to bf16 on the
// way into shared memory (rows padded to 272 bytes: ldmatrix reads are conflict free) and are shared by the four
// warps; the score accumulators become the A fragments of the second product without leaving registers.
constexpr int kTcQ = 64, kTcKeys = 64, kTcLd = 128 + 8;
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__global__ void __launch_bounds__(128) attn_prefill_tc_kernel(const float* __restrict__ qkv, int64_t qkv_stride, int t_new, int n_heads,
                                                              const float* __restrict__ kc, const float* __restrict__ vc,
                                                              int64_t max_seq, const int32_t* __restrict__ pos0,
                                                              float* __restrict__ out, int64_t out_stride) {
    constexpr int HD = 128;
    __shared__ __align__(16) uint16_t ks[kTcKeys * kTcLd];
    __shared__ __align__(16) uint16_t vs[kTcKeys * kTcLd];
    pdl_launch_dependents();
    pdl_wait();
    const int bh = blockIdx.y, b = bh / n_heads, h = bh - b * n_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int q0 = blockIdx.x * kTcQ;
    int64_t p0 = static_cast<int64_t>(*pos0);
    p0 = p0 < 0 ? 0 : p0;
    // 1/sqrt(HD) and log2(e) go into q: the softmax then works with exp2
    const float qscale = rsqrtf(static_cast<float>(HD)) * 1.4426950408889634f;
    const int row_lo = q0 + 16 * warp + g, row_hi = row_lo + 8;         // this lane's two query rows
    uint32_t qa[HD / 16][4];
    {
        const float* qlo = qkv + (static_cast<int64_t>(b) * t_new + (row_lo < t_new ? row_lo : 0)) * qkv_stride + h * HD;
        const float* qhi = qkv + (static_cast<int64_t>(b) * t_new + (row_hi < t_new ? row_hi : 0)) * qkv_stride + h * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const float2 a = *reinterpret_cast<const float2*>(qlo + 16 * kk + 2 * t), c = *reinterpret_cast<const float2*>(qlo + 16 * kk + 8 + 2 * t);
            const float2 e = *reinterpret_cast<const float2*>(qhi + 16 * kk + 2 * t), f = *reinterpret_cast<const float2*>(qhi + 16 * kk + 8 + 2 * t);
            qa[kk][0] = pack_bf16(a.x * qscale, a.y * qscale);
            qa[kk][1] = pack_bf16(e.x * qscale, e.y * qscale);
            qa[kk][2] = pack_bf16(c.x * qscale, c.y * qscale);
            qa[kk][3] = pack_bf16(f.x * qscale, f.y * qscale);
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_lo = -CUDART_INF_F, m_hi = -CUDART_INF_F, l_lo = 0.f, l_hi = 0.f;
    const int last_q = (q0 + kTcQ - 1 < t_new - 1) ? q0 + kTcQ - 1 : t_new - 1;
    int64_t nk = p0 + last_q + 1;                  // keys this block needs
    nk = nk > max_seq ? max_seq : nk;
    const float* kb = kc + static_cast<int64_t>(bh) * max_seq * HD;
    const float* vb = vc + static_cast<int64_t>(bh) * max_seq * HD;
    const int64_t lim_lo = p0 + row_lo, lim_hi = p0 + row_hi;           // last key each row may see
    const uint32_t ks_u = smem_u32(ks), vs_u = smem_u32(vs);
    for (int64_t j0 = 0; j0 < nk; j0 += kTcKeys) {
        __syncthreads();                           // the tiles of the last round have been read by everyone
        for (int it = threadIdx.x; it < kTcKeys * (HD / 4); it += 128) {
            const int r = it / (HD / 4), c = (it - r * (HD / 4)) * 4;
            const int64_t j = (j0 + r < nk) ? j0 + r : nk - 1;                         // clamped: masked below
            const float4 kv = __ldg(reinterpret_cast<const float4*>(kb + j * HD + c));
            const float4 vv = __ldg(reinterpret_cast<const float4*>(vb + j * HD + c));
            *reinterpret_cast<uint2*>(ks + r * kTcLd + c) = make_uint2(pack_bf16(kv.x, kv.y), pack_bf16(kv.z, kv.w));
            *reinterpret_cast<uint2*>(vs + r * kTcLd + c) = make_uint2(pack_bf16(vv.x, vv.y), pack_bf16(vv.z, vv.w));
        }
        __syncthreads();
        // scores of 16 rows x 64 keys: 8 key tiles of 8, 8 steps of 16 head dimensions each
        float sc[kTcKeys / 8][4];
#pragma unroll
        for (int j = 0; j < kTcKeys / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
        for (int j = 0; j < kTcKeys / 8; ++j) {
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk += 2) {
                // four 8x8 matrices: keys 8j.., head dimensions 16kk + {0, 8, 16, 24}..: (b0, b1) of steps kk and kk + 1
                uint32_t bfr[4];
                ldsm_x4(bfr, ks_u + ((8 * j + (lane & 7)) * kTcLd + 16 * kk + 8 * (lane >> 3)) * 2);
                mma_bf16_16816(sc[j], qa[kk], bfr[0], bfr[1]);
                mma_bf16_16816(sc[j], qa[kk + 1], bfr[2], bfr[3]);
            }
        }
        // mask (causal and end of range), row maxima over the quad that shares a row
        float t_lo = -CUDART_INF_F, t_hi = -CUDART_INF_F;
#pragma unroll
        for (int j = 0; j < kTcKeys / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int64_t key = j0 + 8 * j + 2 * t + e;
                const bool in = key < nk;
                if (!(in && key <= lim_lo && row_lo < t_new)) sc[j][e] = -CUDART_INF_F;
                if (!(in && key <= lim_hi && row_hi < t_new)) sc[j][2 + e] = -CUDART_INF_F;
                t_lo = fmaxf(t_lo, sc[j][e]);
                t_hi = fmaxf(t_hi, sc[j][2 + e]);
            }
        }
        t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 1)); t_lo = fmaxf(t_lo, __shfl_xor_sync(0xffffffffu, t_lo, 2));
        t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 1)); t_hi = fmaxf(t_hi, __shfl_xor_sync(0xffffffffu, t_hi, 2));
        const float n_lo = fmaxf(m_lo, t_lo), n_hi = fmaxf(m_hi, t_hi);
        // a row whose every key so far is masked keeps m = -inf: its weights and its rescaling are zero
        const float a_lo = (n_lo == -CUDART_INF_F) ? 0.f : exp2f(m_lo - n_lo), a_hi = (n_hi == -CUDART_INF_F) ? 0.f : exp2f(m_hi - n_hi);
        m_lo = n_lo; m_hi = n_hi;
        float s_lo = 0.f, s_hi = 0.f;
        uint32_t pa[kTcKeys / 16][4];               // the weights as A fragments: keys 16kk.. = score tiles 2kk, 2kk + 1
#pragma unroll
        for (int j = 0; j < kTcKeys / 8; ++j) {
            const float p0v = (n_lo == -CUDART_INF_F) ? 0.f : exp2f(sc[j][0] - n_lo), p1v = (n_lo == -CUDART_INF_F) ? 0.f : exp2f(sc[j][1] - n_lo);
            const float p2v = (n_hi == -CUDART_INF_F) ? 0.f : exp2f(sc[j][2] - n_hi), p3v = (n_hi == -CUDART_INF_F) ? 0.f : exp2f(sc[j][3] - n_hi);
            s_lo += p0v + p1v;
            s_hi += p2v + p3v;
            pa[j >> 1][(j & 1) * 2] = pack_bf16(p0v, p1v);
            pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2v, p3v);
        }
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1); s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1); s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
        l_lo = l_lo * a_lo + s_lo;
        l_hi = l_hi * a_hi + s_hi;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) { o[j][0] *= a_lo; o[j][1] *= a_lo; o[j][2] *= a_hi; o[j][3] *= a_hi; }
        // weighted values: 16 tiles of 8 head dimensions, 4 steps of 16 keys
#pragma unroll
        for (int kk = 0; kk < kTcKeys / 16; ++kk) {
#pragma unroll
            for (int j = 0; j < HD / 8; j += 2) {
                // transposed 8x8 matrices: keys 16kk + {0, 8}.., head dimensions 8j.. and 8(j+1)..: (b0, b1) of tiles j and j + 1
                uint32_t bfr[4];
                ldsm_x4_trans(bfr, vs_u + ((16 * kk + 8 * ((lane >> 3) & 1) + (lane & 7)) * kTcLd + 8 * (j + (lane >> 4))) * 2);
                mma_bf16_16816(o[j], pa[kk], bfr[0], bfr[1]);
                mma_bf16_16816(o[j + 1], pa[kk], bfr[2], bfr[3]);
            }
        }
    }
    const float i_lo = l_lo > 0.f ? 1.0f / l_lo : 0.f, i_hi = l_hi > 0.f ? 1.0f / l_hi : 0.f;
    if (row_lo < t_new) {
        float* orow = out + (static_cast<int64_t>(b) * t_new + row_lo) * out_stride + h * HD + 2 * t;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) *reinterpret_cast<float2*>(orow + 8 * j) = make_float2(o[j][0] * i_lo, o[j][1] * i_lo);
    }
    if (row_hi < t_new) {
        float* orow = out + (static_cast<int64_t>(b) * t_new + row_hi) * out_stride + h * HD + 2 * t;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) *reinterpret_cast<float2*>(orow + 8 * j) = make_float2(o[j][2] * i_hi, o[j][3] * i_hi);
    }
}

// Embedding lookup: one block per index.  An index outside [0, vocab) yields a row of zeros, as the
// reference's lookup does (src/ops.cpp:2643-2649); nothing is ever read outside the table.
__global__ void __launch_bounds__(256) embedding_kernel(const float* __restrict__ table, int64_t vocab, int64_t dim,
                                                        const int64_t* __restrict__ ids, float* __restrict__ out, int vec) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t id = ids[blockIdx.x];
    const bool ok = id >= 0 && id < vocab;
    float* o = out + blockIdx.x * dim;
    const float* src = table + (ok ? id : 0) * dim;
    if (vec) {
        for (int64_t i = threadIdx.x * 4; i < dim; i += 1024)
            *reinterpret_cast<float4*>(o + i) = ok ? __ldg(reinterpret_cast<const float4*>(src + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        for (int64_t i = threadIdx.x; i < dim; i += 256) o[i] = ok ? __ldg(src + i) : 0.f;
    }
}

// First index of the strict maximum of every row (the reference's greedy choice keeps the first of equal
// candidates: `if (p > best)`, include/sovereigngrad/models.hpp:291-298).  NaN never wins a comparison; a
// row without any comparable value yields 0.
constexpr int kArgmaxThreads = 512;
__global__ void __launch_bounds__(kArgmaxThreads) argmax_rows_kernel(const float* __restrict__ x, int64_t n, int64_t ld,
                                                                    int64_t* __restrict__ out) {
    __shared__ float sv[kArgmaxThreads / 32];
    __shared__ long long si[kArgmaxThreads / 32];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = x + blockIdx.x * ld;
    float best = -CUDART_INF_F;
    long long idx = -1;                                   // -1: nothing seen yet (a -inf entry must still be able to win)
    for (int64_t i = threadIdx.x; i < n; i += kArgmaxThreads) {
        const float v = row[i];
        if (v > best || (idx < 0 && v == best)) { best = v; idx = i; }
    }
    auto better = [](float v, long long i, float bv, long long bi) {
        return i >= 0 && (bi < 0 || v > bv || (v == bv && i < bi));
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const long long oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < kArgmaxThreads / 32 ? sv[threadIdx.x] : -CUDART_INF_F;
        idx = threadIdx.x < kArgmaxThreads / 32 ? si[threadIdx.x] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const long long oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (better(ov, oi, best, idx)) { best = ov; idx = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = idx < 0 ? 0 : idx;
    }
}

int attn_splits(int64_t batch, int64_t n_heads, int64_t max_seq) {
    // as many splits as keep every CTA resident at once (one wave), at least 32 keys each, at most
    // the portable cluster size
    const int64_t bh = batch * n_heads > 0 ? batch * n_heads : 1;
    int64_t s = (static_cast<int64_t>(kAttnCtasPerSm) * sm_count()) / bh;
    const int64_t cap = ceil_div(max_seq, 32);
    if (s > cap) s = cap;
    if (s > 8) s = 8;
    if (s < 1) s = 1;
    return static_cast<int>(s);
}

template <int HD>
int launch_attn(const float* qkv, int64_t qkv_stride, int64_t batch, int n_heads, const float* cos_t, const float* sin_t, float* kc,
                float* vc, int64_t max_seq, const int32_t* pos0, float* out, int64_t out_stride, const PreparedLayout& L,
                uint8_t* planes, cudaStream_t s, const PeerPtrs& peers = PeerPtrs{}) {
    const int S = attn_splits(batch, n_heads, max_seq);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(batch * n_heads), static_cast<unsigned>(S), 1);
    cfg.blockDim = dim3(kAttnWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(S);
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = stream_overlap_enabled() ? 2 : 1;
    if (peers.n > 0) {
        SGQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, true>, qkv, qkv_stride, n_heads, cos_t, sin_t, kc, vc, max_seq, pos0,
                                        out, out_stride, static_cast<int>(batch), L.mode, L.nmain, L.nlow, planes, peers));
        return SGQ_OK;
    }
    // (no preference for the largest shared-memory split here: this kernel fills the register file, so no dependent
    // kernel can join its SMs anyway, and its streaming loads want the L1 they get by default)
    SGQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, false>, qkv, qkv_stride, n_heads, cos_t, sin_t, kc, vc, max_seq, pos0,
                                    out, out_stride, static_cast<int>(batch), L.mode, L.nmain, L.nlow, planes, peers));
    return SGQ_OK;
}

}  // namespace
}  // namespace sgq

using namespace sgq;

extern "C" {

namespace {
// prepared_out is optional; when given, (rows, width) must have a prepared form and the buffer must hold it
int check_prepared(void* prepared_out, size_t prepared_bytes, int64_t rows, int64_t width, PreparedLayout* L) {
    if (!prepared_out) return SGQ_OK;
    const size_t need = gemv_prepared_bytes(rows, width);
    if (need == 0) return bad(SGQ_ERR_UNSUPPORTED, "no prepared-activation form for this (rows, width): rows <= 16, width % 256 == 0");
    if (prepared_bytes < need || !aligned(prepared_out, 256)) return bad(SGQ_ERR_WORKSPACE, "prepared buffer too small or not 256-byte aligned");
    *L = prepared_layout(rows, width);
    return SGQ_OK;
}
}  // namespace

int sgqd_add_rmsnorm(float* h, const float* delta, const float* gamma, float eps, int64_t rows, int64_t dim, float* out,
                     void* prepared_out, size_t prepared_bytes, void* stream) {
    if (rows < 0 || dim < 0 || rows > 0x7fffffff) return bad(SGQ_ERR_BAD_SHAPE, "bad rows/dim");
    if (rows == 0 || dim == 0) return SGQ_OK;
    if (!h || !gamma || !out) return bad(SGQ_ERR_NULL_POINTER, "h, gamma or out is NULL");
    if (out == h) return bad(SGQ_ERR_BAD_ARGUMENT, "out may not alias h");
    if ((dim & 3) == 0 && !(aligned(h, 16) && aligned(out, 16) && aligned(gamma, 16) && (!delta || aligned(delta, 16))))
        return bad(SGQ_ERR_ALIGNMENT, "rows must be 16-byte aligned");
    PreparedLayout L = {};
    int rc = check_prepared(prepared_out, prepared_bytes, rows, dim, &L);
    if (rc != SGQ_OK) return rc;
    rc = check_device();
    if (rc != SGQ_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool ov = stream_overlap_enabled();
    const bool in_regs = (dim % 256) == 0 && dim <= 8192 && aligned(h, 16) && aligned(out, 16) && aligned(gamma, 16) &&
                         (!delta || aligned(delta, 16));
    if (in_regs) {
        uint8_t* pl = static_cast<uint8_t*>(prepared_out);
        const dim3 grid(static_cast<unsigned>(rows)), block(kNormThreads);
#define SGQ_NORM_ROW(PREPV, CHV) \
    SGQ_CUDA_TRY(launch_kernel(add_rmsnorm_row_kernel<PREPV, CHV>, grid, block, 0, s, ov, h, delta, gamma, eps, dim, out, L.mode, L.nmain, L.nlow, pl))
        if (dim <= 2048) { if (pl) SGQ_NORM_ROW(true, 1); else SGQ_NORM_ROW(false, 1); }
        else if (dim <= 4096) { if (pl) SGQ_NORM_ROW(true, 2); else SGQ_NORM_ROW(false, 2); }
        else { if (pl) SGQ_NORM_ROW(true, 4); else SGQ_NORM_ROW(false, 4); }
#undef SGQ_NORM_ROW
        return SGQ_OK;
    }
    if (prepared_out)
        SGQ_CUDA_TRY(launch_kernel(add_rmsnorm_kernel<true>, dim3(static_cast<unsigned>(rows)), dim3(kNormThreads), 0, s, ov, h, delta,
                                   gamma, eps, dim, out, L.mode, L.nmain, L.nlow, static_cast<uint8_t*>(prepared_out)));
    else
        SGQ_CUDA_TRY(launch_kernel(add_rmsnorm_kernel<false>, dim3(static_cast<unsigned>(rows)), dim3(kNormThreads), 0, s, ov, h, delta,
                                   gamma, eps, dim, out, 0, 1, 1, static_cast<uint8_t*>(nullptr)));
    return SGQ_OK;
}

int sgqd_rope_kv_store(float* qkv, int64_t batch, int64_t t_new, int64_t n_heads, int64_t head_dim, const float* cos_table,
                       const float* sin_table, const int32_t* pos0, float* k_cache, float* v_cache, int64_t max_seq,
                       void* stream) {
    if (batch < 0 || t_new < 0 || n_heads <= 0 || head_dim <= 0 || max_seq <= 0 || batch * t_new > 0x7fffffff)
        return bad(SGQ_ERR_BAD_SHAPE, "bad decoder shape");
    if (head_dim % 8) return bad(SGQ_ERR_BAD_SHAPE, "head_dim must be a multiple of 8");
    if (batch * t_new == 0) return SGQ_OK;
    if (!qkv || !cos_table || !sin_table || !pos0 || !k_cache || !v_cache) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    SGQ_CUDA_TRY(launch_kernel(rope_kv_store_kernel, dim3(static_cast<unsigned>(batch * t_new)), dim3(256), 0,
                               static_cast<cudaStream_t>(stream), stream_overlap_enabled(), qkv, static_cast<int>(t_new),
                               static_cast<int>(n_heads), static_cast<int>(head_dim), cos_table, sin_table, pos0, k_cache, v_cache,
                               max_seq));
    return SGQ_OK;
}

int sgqd_attn_decode(float* qkv, int64_t qkv_stride, int64_t batch, int64_t n_heads, int64_t head_dim, const float* cos_table,
                     const float* sin_table, float* k_cache, float* v_cache, int64_t max_seq, const int32_t* pos0, float* out,
                     int64_t out_stride, void* prepared_out, size_t prepared_bytes, void* stream) {
    if (batch < 0 || n_heads <= 0 || max_seq <= 0 || batch * n_heads > 0x7fffffff) return bad(SGQ_ERR_BAD_SHAPE, "bad decoder shape");
    if (head_dim != 64 && head_dim != 128) return bad(SGQ_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
    if (qkv_stride < 3 * n_heads * head_dim || out_stride < n_heads * head_dim) return bad(SGQ_ERR_BAD_SHAPE, "row stride too small");
    if (batch == 0) return SGQ_OK;
    if (!qkv || !cos_table || !sin_table || !k_cache || !v_cache || !pos0 || !out) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    if (!aligned(qkv, 16) || !aligned(k_cache, 16) || !aligned(v_cache, 16) || (qkv_stride & 3))
        return bad(SGQ_ERR_ALIGNMENT, "qkv rows and caches must be 16-byte aligned");
    PreparedLayout L = {};
    int rc = check_prepared(prepared_out, prepared_bytes, batch, n_heads * head_dim, &L);
    if (rc != SGQ_OK) return rc;
    rc = check_device();
    if (rc != SGQ_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* pl = static_cast<uint8_t*>(prepared_out);
    if (head_dim == 128)
        return launch_attn<128>(qkv, qkv_stride, batch, static_cast<int>(n_heads), cos_table, sin_table, k_cache, v_cache, max_seq, pos0,
                                out, out_stride, L, pl, s);
    return launch_attn<64>(qkv, qkv_stride, batch, static_cast<int>(n_heads), cos_table, sin_table, k_cache, v_cache, max_seq, pos0, out,
                           out_stride, L, pl, s);
}

int sgqd_attn_decode_allgather(float* qkv, int64_t qkv_stride, int64_t batch, int64_t n_heads, int64_t head_dim,
                               const float* cos_table, const float* sin_table, float* k_cache, float* v_cache, int64_t max_seq,
                               const int32_t* pos0, float* const* out_ranks, int world, int64_t out_stride, int64_t col_offset,
                               void* stream) {
    if (batch < 0 || n_heads <= 0 || max_seq <= 0 || batch * n_heads > 0x7fffffff) return bad(SGQ_ERR_BAD_SHAPE, "bad decoder shape");
    if (head_dim != 64 && head_dim != 128) return bad(SGQ_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
    if (world < 1 || world > kMaxPeers) return bad(SGQ_ERR_BAD_ARGUMENT, "world must be 1..8");
    if (qkv_stride < 3 * n_heads * head_dim || col_offset < 0 || out_stride < col_offset + n_heads * head_dim)
        return bad(SGQ_ERR_BAD_SHAPE, "row stride too small");
    if (batch == 0) return SGQ_OK;
    if (!qkv || !cos_table || !sin_table || !k_cache || !v_cache || !pos0 || !out_ranks) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    if (!aligned(qkv, 16) || !aligned(k_cache, 16) || !aligned(v_cache, 16) || (qkv_stride & 3))
        return bad(SGQ_ERR_ALIGNMENT, "qkv rows and caches must be 16-byte aligned");
    PeerPtrs peers = {};
    for (int r = 0; r < world; ++r) {
        if (!out_ranks[r]) return bad(SGQ_ERR_NULL_POINTER, "an output pointer is NULL");
        peers.p[r] = out_ranks[r] + col_offset;
    }
    peers.n = world;
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    const PreparedLayout L = {};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (head_dim == 128)
        return launch_attn<128>(qkv, qkv_stride, batch, static_cast<int>(n_heads), cos_table, sin_table, k_cache, v_cache, max_seq, pos0,
                                peers.p[0], out_stride, L, nullptr, s, peers);
    return launch_attn<64>(qkv, qkv_stride, batch, static_cast<int>(n_heads), cos_table, sin_table, k_cache, v_cache, max_seq, pos0,
                           peers.p[0], out_stride, L, nullptr, s, peers);
}

int sgqd_silu_mul_allgather(const float* gate_up, int64_t rows, int64_t hidden, float* const* out_ranks, int world, int64_t ld,
                            int64_t col_offset, void* stream) {
    if (rows < 0 || hidden < 0 || col_offset < 0 || ld < col_offset + hidden) return bad(SGQ_ERR_BAD_SHAPE, "bad slice shape");
    if (world < 1 || world > kMaxPeers) return bad(SGQ_ERR_BAD_ARGUMENT, "world must be 1..8");
    if (rows * hidden == 0) return SGQ_OK;
    if (!gate_up || !out_ranks) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    PeerPtrs peers = {};
    for (int r = 0; r < world; ++r) {
        if (!out_ranks[r]) return bad(SGQ_ERR_NULL_POINTER, "an output pointer is NULL");
        peers.p[r] = out_ranks[r] + col_offset;
    }
    peers.n = world;
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    int64_t blocks = ceil_div(rows * hidden, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    SGQ_CUDA_TRY(launch_kernel(silu_mul_peers_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                               stream_overlap_enabled(), gate_up, rows, hidden, ld, peers));
    return SGQ_OK;
}

int sgqd_attn_prefill(const float* qkv, int64_t qkv_stride, int64_t batch, int64_t t_new, int64_t n_heads, int64_t head_dim,
                      const float* k_cache, const float* v_cache, int64_t max_seq, const int32_t* pos0, float* out, int64_t out_stride,
                      void* stream) {
    if (batch < 0 || t_new < 0 || n_heads <= 0 || max_seq <= 0 || batch * n_heads > 65535 || t_new > 0x3fffffff)
        return bad(SGQ_ERR_BAD_SHAPE, "bad decoder shape");
    if (head_dim != 64 && head_dim != 128) return bad(SGQ_ERR_UNSUPPORTED, "head_dim must be 64 or 128");
    if (qkv_stride < 3 * n_heads * head_dim || out_stride < n_heads * head_dim) return bad(SGQ_ERR_BAD_SHAPE, "row stride too small");
    if (batch * t_new == 0) return SGQ_OK;
    if (!qkv || !k_cache || !v_cache || !pos0 || !out) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    if (!aligned(qkv, 16) || !aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(out, 16) || (qkv_stride & 3) || (out_stride & 3))
        return bad(SGQ_ERR_ALIGNMENT, "rows and caches must be 16-byte aligned");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    const dim3 grid(static_cast<unsigned>(ceil_div(t_new, kPrefillQ)), static_cast<unsigned>(batch * n_heads));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (head_dim == 128)
        SGQ_CUDA_TRY(launch_kernel(attn_prefill_kernel<128>, grid, dim3(256), 0, s, stream_overlap_enabled(), qkv, qkv_stride,
                                   static_cast<int>(t_new), static_cast<int>(n_heads), k_cache, v_cache, max_seq, pos0, out, out_stride));
    else
        SGQ_CUDA_TRY(launch_kernel(attn_prefill_kernel<64>, grid, dim3(256), 0, s, stream_overlap_enabled(), qkv, qkv_stride,
                                   static_cast<int>(t_new), static_cast<int>(n_heads), k_cache, v_cache, max_seq, pos0, out, out_stride));
    return SGQ_OK;
}

int sgqd_attn_prefill_bf16(const float* qkv, int64_t qkv_stride, int64_t batch, int64_t t_new, int64_t n_heads, int64_t head_dim,
                           const float* k_cache, const float* v_cache, int64_t max_seq, const int32_t* pos0, float* out,
                           int64_t out_stride, void* stream) {
    if (batch < 0 || t_new < 0 || n_heads <= 0 || max_seq <= 0 || batch * n_heads > 65535 || t_new > 0x3fffffff)
        return bad(SGQ_ERR_BAD_SHAPE, "bad decoder shape");
    if (head_dim != 128) return bad(SGQ_ERR_UNSUPPORTED, "head_dim must be 128");
    if (qkv_stride < 3 * n_heads * head_dim || out_stride < n_heads * head_dim) return bad(SGQ_ERR_BAD_SHAPE, "row stride too small");
    if (batch * t_new == 0) return SGQ_OK;
    if (!qkv || !k_cache || !v_cache || !pos0 || !out) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    if (!aligned(qkv, 16) || !aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(out, 16) || (qkv_stride & 3) || (out_stride & 3))
        return bad(SGQ_ERR_ALIGNMENT, "rows and caches must be 16-byte aligned");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    const dim3 grid(static_cast<unsigned>(ceil_div(t_new, kTcQ)), static_cast<unsigned>(batch * n_heads));
    SGQ_CUDA_TRY(launch_kernel(attn_prefill_tc_kernel, grid, dim3(128), 0, static_cast<cudaStream_t>(stream), stream_overlap_enabled(), qkv,
                               qkv_stride, static_cast<int>(t_new), static_cast<int>(n_heads), k_cache, v_cache, max_seq, pos0, out,
                               out_stride));
    return SGQ_OK;
}

int sgqd_embedding(const float* table, int64_t vocab, int64_t dim, const int64_t* ids, int64_t rows, float* out, void* stream) {
    if (vocab < 0 || dim < 0 || rows < 0 || rows > 0x7fffffff) return bad(SGQ_ERR_BAD_SHAPE, "bad embedding shape");
    if (rows * dim == 0) return SGQ_OK;
    if (!table || !ids || !out) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    const int vec = ((dim & 3) == 0 && aligned(table, 16) && aligned(out, 16)) ? 1 : 0;
    SGQ_CUDA_TRY(launch_kernel(embedding_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                               stream_overlap_enabled(), table, vocab, dim, ids, out, vec));
    return SGQ_OK;
}

int sgqd_argmax_rows(const float* x, int64_t rows, int64_t n, int64_t ld, int64_t* out, void* stream) {
    if (rows < 0 || n < 0 || ld < n || rows > 0x7fffffff) return bad(SGQ_ERR_BAD_SHAPE, "bad argmax shape");
    if (rows == 0) return SGQ_OK;
    if (!out || (n > 0 && !x)) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    int rc = check_device();
    if (rc != SGQ_OK) return rc;
    SGQ_CUDA_TRY(launch_kernel(argmax_rows_kernel, dim3(static_cast<unsigned>(rows)), dim3(kArgmaxThreads), 0,
                               static_cast<cudaStream_t>(stream), stream_overlap_enabled(), x, n, ld, out));
    return SGQ_OK;
}

int sgqd_silu_mul(const float* gate_up, int64_t rows, int64_t hidden, float* out, void* prepared_out, size_t prepared_bytes,
                  void* stream) {
    if (rows < 0 || hidden < 0) return bad(SGQ_ERR_BAD_SHAPE, "negative dimension");
    if (rows * hidden == 0) return SGQ_OK;
    if (!gate_up || !out) return bad(SGQ_ERR_NULL_POINTER, "NULL argument");
    PreparedLayout L = {};
    int rc = check_prepared(prepared_out, prepared_bytes, rows, hidden, &L);
    if (rc != SGQ_OK) return rc;
    if (prepared_out && !(aligned(gate_up, 16) && aligned(out, 16))) return bad(SGQ_ERR_ALIGNMENT, "rows must be 16-byte aligned");
    rc = check_device();
    if (rc != SGQ_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (prepared_out && (hidden % 256) == 0 && hidden / 8 <= 65535LL * kSiluThreads) {
        SGQ_CUDA_TRY(launch_kernel(silu_mul_prepare_row_kernel,
                                   dim3(static_cast<unsigned>(rows), static_cast<unsigned>(ceil_div(hidden / 8, kSiluThreads))), dim3(kSiluThreads), 0, s,
                                   stream_overlap_enabled(), gate_up, hidden, out, L.mode, L.nmain, L.nlow,
                                   static_cast<uint8_t*>(prepared_out)));
        return SGQ_OK;
    }
    if (prepared_out) {
        SGQ_CUDA_TRY(launch_kernel(silu_mul_prepare_kernel, dim3(static_cast<unsigned>(rows)), dim3(kNormThreads), 0, s,
                                   stream_overlap_enabled(), gate_up, hidden, out, L.mode, L.nmain, L.nlow,
                                   static_cast<uint8_t*>(prepared_out)));
        return SGQ_OK;
    }
    int64_t blocks = ceil_div(rows * hidden, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    SGQ_CUDA_TRY(launch_kernel(silu_mul_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, s, stream_overlap_enabled(), gate_up,
                               rows, hidden, out));
    return SGQ_OK;
}

}  // extern "C"
