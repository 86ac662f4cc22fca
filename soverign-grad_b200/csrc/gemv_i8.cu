// Decode-shape forward (M <= 16) for INT8 weights stored [N,K], one scale per tensor or per row:
//   y = x * (codes * scale)^T + bias.
//
// HBM-bound: every weight byte is read exactly once (algorithmic bytes N*K + M*K*4 + M*N*4).
//
// Same skeleton as the INT4 decode kernel (gemv.cu): one persistent CTA per SM, a TMA producer
// thread, 8 consumer warps.  What INT8 changes:
//   * a step is 128 k of a 16-row tile (one 128-byte swizzled row per weight row), a stage is 8
//     steps; the bytes go to the tensor core as they are (mma.sync m16n8k32 s8 x s8 -> s32), with
//     no unpacking and no offset;
//   * there is no per-group weight scale, and the activations are scaled per 128 k (gemv_prepare.cuh
//     with blocks of four groups: 24-bit fixed point below the block's absmax, the low digit in column
//     sets of its own that are skipped where it cannot matter): the exact sums of a step's four groups
//     add up in one int32 accumulator, are multiplied by the step's activation scale and added up in
//     fp32; the weight scale is applied once per output;
//   * the main activation digit planes, their scales and the low-digit flags (laid out for the
//     natural k order of an int8 B fragment) are written once by a conversion kernel and stream
//     through the same pipeline stages as the weights, 32 groups at a time, from L2.  They are
//     never resident as a whole, so K is not limited by shared memory (K = 8192 at M = 16 runs);
//     low digits are fetched from the prepared buffer itself, for flagged groups only;
//   * tile epilogue: every warp leaves its fp32 partial sums in one of two shared-memory slots,
//     one named barrier, then thread (m, row) adds the eight partials in warp order (fixed order:
//     the same bits every run), recombines the digits, applies the weight scale and the bias.
//
// y[m,n] = (sum_j 256^j * sum_b sx[m,b] * S_j[b,m,n]) * scale[n] + bias[n],  S_j exact integers per 128-k block b.
#include "sgq_common.cuh"
#include "gemv_prepare.cuh"
#include "sm100_ptx.cuh"

#include <cuda.h>

namespace sgq {

__device__ uint32_t g_status_gemv_i8 = 0;

cudaError_t read_status_gemv_i8(uint32_t* v, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(v, g_status_gemv_i8, sizeof(uint32_t));
    if (e == cudaSuccess && clear && *v != 0) {
        const uint32_t zero = 0;
        e = cudaMemcpyToSymbol(g_status_gemv_i8, &zero, sizeof(zero));
    }
    return e;
}

namespace {

constexpr int kRows = 16;                       // weight rows per tile (mma M)
constexpr int kStepK = 128;                     // k per step: one 128-byte swizzle row per weight row
constexpr int kSteps = 8;                       // steps per stage = consumer warps
constexpr int kStageK = kStepK * kSteps;        // 1024
constexpr int kStageW = kSteps * kRows * 128;   // 16384 bytes of weights per stage
constexpr int kGroupsPerStage = kStageK / 32;   // 32 digit groups per stage
constexpr int kWarps = kSteps;
constexpr int kConsumerThreads = kWarps * 32;
constexpr int kThreads = kConsumerThreads + 32; // + producer warp
constexpr int kMaxM = 16;
constexpr int kMaxStages = 8;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kPrepThreads = 256;

__device__ __forceinline__ void report(uint32_t code, uint32_t detail) {
    atomicCAS(&g_status_gemv_i8, 0u, (code << 24) | (detail & 0xFFFFFFu));
}

// D(16x8,s32) = A(16x32,s8,row) * B(32x8,s8,col) + magic
__device__ __forceinline__ void mma_s8s8_16832_magic(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(kMagicBits));
}

// N consecutive floats (16-byte aligned for N = 4, 8-byte for N = 2) with the widest load that fits.
template <int N>
__device__ __forceinline__ void load_scales(float (&v)[N], const float* p) {
    if constexpr (N == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else if constexpr (N == 2) {
        const float2 q = *reinterpret_cast<const float2*>(p);
        v[0] = q.x; v[1] = q.y;
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = p[i];
    }
}

// Four 8x8 matrices of 16-byte rows: lane l supplies the address of row (l & 7) of matrix (l >> 3);
// lane (g, t) receives word t of row g of every matrix.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}

// D += A * B: the groups of a 128-k step add up in the same int32 accumulator (four groups of at most 32 * 127 * 127
// stay inside the range in which the fp32 view of the magic start value is exact)
__device__ __forceinline__ void mma_s8s8_16832_acc(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// total += (exact int32 sums of one 128-k step, as 12582912.0f + sum in fp32 bits) * (activation scales of columns 2t, 2t+1)
__device__ __forceinline__ void scale_step(float (&total)[4], const int (&d)[4], float2 sx) {
    total[0] = __fmaf_rn(sx.x, __fsub_rn(__int_as_float(d[0]), kMagicF), total[0]);
    total[1] = __fmaf_rn(sx.y, __fsub_rn(__int_as_float(d[1]), kMagicF), total[1]);
    total[2] = __fmaf_rn(sx.x, __fsub_rn(__int_as_float(d[2]), kMagicF), total[2]);
    total[3] = __fmaf_rn(sx.y, __fsub_rn(__int_as_float(d[3]), kMagicF), total[3]);
}

// Digit planes and group scales for the int8 kernel (gemv_prepare.cuh, natural k order): one CTA per
// row, one pass.  K is a multiple of 128: in the last warp-wide call of a row the lanes beyond the end
// pass zeros and store nothing.
__global__ void __launch_bounds__(kPrepThreads) prepare_x_i8_kernel(const float* __restrict__ x, int64_t K, int mode, int nmain,
                                                                   int nlow, uint8_t* __restrict__ planes) {
    pdl_launch_dependents();
    pdl_wait();                                        // x comes from the kernel before this one
    const int m = blockIdx.x, M = gridDim.x;
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<int64_t>(m) * K);
    const int chunks = static_cast<int>(K / 8);
    const int padded = (chunks + 31) & ~31;
    const PreparedParts pp = prepared_parts(planes, static_cast<size_t>(K / 32), nmain, nlow);
    for (int c = threadIdx.x; c < padded; c += kPrepThreads) {
        const bool in = c < chunks;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (in) {
            const float4 a = __ldg(xr + 2 * c), b = __ldg(xr + 2 * c + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
        convert_groups<kOrderNatural, 4>(v, m, M, static_cast<size_t>(c >> 5) * 8, mode, nmain, nlow, 1.0f, pp, in);
    }
}

struct Smem {
    uint32_t stage_bytes, partial_off, misc_off, total;
};

__host__ __device__ inline Smem smem_layout(int nstages, int nmain, int nlow) {
    Smem s;
    s.stage_bytes = kStageW + kGroupsPerStage * ((256u + 32u) * nmain + (nlow ? 16u : 0u));   // weights, main digits and scales, flags
    s.stage_bytes = (s.stage_bytes + 1023u) & ~1023u;      // the swizzled weight box of every stage starts on a 1024-byte boundary
    s.partial_off = nstages * s.stage_bytes;
    s.misc_off = s.partial_off + 2u * kWarps * (512u * nmain + 16u);      // two slots of per-warp fp32 partial sums (padded)
    s.total = s.misc_off + 2u * kMaxStages * 8u + 16u;
    return s;
}

template <int NM, int NL, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemv_int8_nk_kernel(const __grid_constant__ CUtensorMap map_w, const uint8_t* __restrict__ planes, const float* __restrict__ wscales,
                    int scale_per_row, const float* __restrict__ bias, float* __restrict__ y, int M, int64_t K, int64_t N, int64_t ldy,
                    int nstages) {
    constexpr int kDigitsOut = NL > 0 ? 2 : 3;
    extern __shared__ uint8_t smem_raw[];
    // aligned by pointer arithmetic on the shared array itself: a round trip through an integer would make the
    // compiler lose the address space and emit generic loads for every shared-memory access below
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const Smem L = smem_layout(nstages, NM, NL);
    float* partial = reinterpret_cast<float*>(smem + L.partial_off);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.misc_off);
    uint64_t* empty = full + kMaxStages;
    constexpr int kPStride = 128 * NM + 4;          // floats per warp in a partial-sum slot

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t ntiles = (N + kRows - 1) / kRows;
    const int spt = static_cast<int>((K + kStepK - 1) / kStepK);     // steps per tile
    const int groups_total = static_cast<int>(K / 32);

    pdl_launch_dependents();
    if (threadIdx.x == kConsumerThreads) tma_prefetch_descriptor(&map_w);
    if (threadIdx.x == 0) {
        for (int i = 0; i < nstages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kWarps);
        }
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    __syncthreads();
    pdl_wait();                                     // the planes are the output of the conversion kernel

    if (warp == kWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            fence_proxy_async_all();                // the planes were written through the generic proxy
            uint32_t seq = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                for (int c0 = 0; c0 < spt; c0 += kSteps, ++seq) {
                    const int st = seq % nstages;
                    const uint32_t ph = (seq / nstages) & 1u;
                    if (!mbar_wait(&empty[st], ph ^ 1u)) {
                        report(kDevErrEmptyWait, seq);
                        ok = false;
                        break;
                    }
                    const int g0 = c0 * 4;                                              // first digit group of the stage
                    const int ng = (groups_total - g0 < kGroupsPerStage) ? groups_total - g0 : kGroupsPerStage;
                    const uint32_t pbytes = static_cast<uint32_t>(ng) * 256u * NM;                    // main digit planes of the stage
                    const uint32_t sbytes = static_cast<uint32_t>(ng) * 32u * NM;                     // their group scales
                    const uint32_t fbytes = NL ? static_cast<uint32_t>(ng) * 16u : 0u;                // and the low-digit flags
                    // steps past K/128 are out of range in the third dimension: zero-filled, still counted
                    mbar_arrive_expect_tx(&full[st], kStageW + pbytes + sbytes + fbytes);
                    uint8_t* sw = smem + st * L.stage_bytes;
                    tma_load_3d(sw, &map_w, &full[st], 0, static_cast<int32_t>(tile * kRows), c0);
                    const size_t G = static_cast<size_t>(groups_total);
                    bulk_copy_g2s(sw + kStageW, planes + static_cast<size_t>(g0) * 256u * NM, pbytes, &full[st]);
                    bulk_copy_g2s(sw + kStageW + kGroupsPerStage * 256u * NM, planes + G * 256u * (NM + NL) + static_cast<size_t>(g0) * 32u * NM,
                                  sbytes, &full[st]);
                    if (NL)
                        bulk_copy_g2s(sw + kStageW + kGroupsPerStage * (256u + 32u) * NM,
                                      planes + G * (256u + 32u) * (NM + NL) + static_cast<size_t>(g0) * 16u, fbytes, &full[st]);
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int g = lane >> 2, t = lane & 3;
    // ldmatrix row address of this lane inside a step box for group i (bytes 32 i .. 32 i + 31 of every row):
    // matrix (lane >> 3) = (rows 0-7 | rows 8-15) x (16-byte chunk 2i | 2i+1); 128-byte swizzle: chunk ^ (row & 7)
    uint32_t lm_off[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        lm_off[i] = ((lane & 7) + 8 * ((lane >> 3) & 1)) * 128 + (((2 * i + (lane >> 4)) ^ (lane & 7)) << 4);
    const uint32_t smem_u = smem_u32(smem);
    // epilogue role of this thread: output (row er of the tile, batch row em)
    const int em = threadIdx.x >> 4, er = threadIdx.x & 15;
    const float sw_all = scale_per_row ? 1.0f : __ldg(wscales);
    // low digit planes and scales: read from the prepared buffer, for flagged groups only
    const uint8_t* low_digits = planes + static_cast<size_t>(groups_total) * 256u * NM;
    const float* low_scales = reinterpret_cast<const float*>(planes + static_cast<size_t>(groups_total) * (256u * (NM + NL) + 32u * NM));

    bool alive = true;
    uint32_t seq = 0, tcount = 0;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
        float total[NM + NL][4];
#pragma unroll
        for (int s = 0; s < NM + NL; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) total[s][i] = 0.0f;

        for (int c0 = 0; c0 < spt; c0 += kSteps, ++seq) {
            const int st = seq % nstages;
            const uint32_t ph = (seq / nstages) & 1u;
            if (alive && !mbar_wait(&full[st], ph)) {
                report(kDevErrFullWait, seq);
                alive = false;
            }
            const int step = c0 + warp;
            if (alive && step < spt) {
                const uint32_t wbox = smem_u + st * L.stage_bytes + warp * (kRows * 128);
                const uint8_t* xg = smem + st * L.stage_bytes + kStageW + (warp * 4) * (256 * NM);
                const float* sg = reinterpret_cast<const float*>(smem + st * L.stage_bytes + kStageW + kGroupsPerStage * 256 * NM) +
                                  ((warp * 4) * 4 + t) * (2 * NM);                        // this lane's group scales
                const uint8_t* fg = smem + st * L.stage_bytes + kStageW + kGroupsPerStage * (256 + 32) * NM + (warp * 4) * 16;
                const size_t grp0 = static_cast<size_t>(step) * 4;                        // first 32-k group of this step
                uint32_t a[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) ldmatrix_x4(a[i], wbox + lm_off[i]);    // rows g / g+8, k = 32i + 4t.. and 32i + 16 + 4t..
                // The four 32-k groups of the step share their activation scales (gemv_prepare.cuh, blocks of four)
                // and the weights have no group scale: their exact sums add up in int32, one scaling per step.
                int d[NM][4];
#pragma unroll
                for (int s2 = 0; s2 < NM; ++s2)
#pragma unroll
                    for (int c = 0; c < 4; ++c) d[s2][c] = kMagicBits;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint8_t* xgi = xg + i * (256 * NM);
#pragma unroll
                    for (int s2 = 0; s2 < NM; ++s2) {
                        if ((s2 & 1) == 0 && s2 + 1 < NM) {          // two main sets side by side: one 128-bit load per lane
                            const uint4 q = *reinterpret_cast<const uint4*>(xgi + (s2 >> 1) * 512 + lane * 16);
                            mma_s8s8_16832_acc(d[s2], a[i], q.x, q.y);
                            mma_s8s8_16832_acc(d[s2 + 1], a[i], q.z, q.w);
                        } else if ((s2 & 1) == 0) {
                            const uint2 q = *reinterpret_cast<const uint2*>(xgi + plane_offset(0, NM, s2, lane));
                            mma_s8s8_16832_acc(d[s2], a[i], q.x, q.y);
                        }
                    }
                }
#pragma unroll
                for (int s2 = 0; s2 < NM; ++s2) scale_step(total[s2], d[s2], *reinterpret_cast<const float2*>(sg + 2 * s2));
                // low digits: only where a row of the set flagged this step (rare: one value dominating its 128)
#pragma unroll
                for (int l = 0; l < NL; ++l) {
                    const uint2 fl = *reinterpret_cast<const uint2*>(fg + l * 8);
                    if ((fl.x | fl.y) != 0u) {                       // the same for every lane of the warp
                        int dl[4] = {kMagicBits, kMagicBits, kMagicBits, kMagicBits};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint2 q = __ldg(reinterpret_cast<const uint2*>(low_digits + plane_offset(grp0 + i, NL, l, lane)));
                            mma_s8s8_16832_acc(dl, a[i], q.x, q.y);
                        }
                        scale_step(total[NM + l], dl, __ldg(reinterpret_cast<const float2*>(low_scales + (grp0 * 4 + t) * NL * 2 + l * 2)));
                    }
                }
            }
            // everything loaded from the stage has been consumed once the accumulators are final
            uint32_t fold = 0;
#pragma unroll
            for (int s = 0; s < NM + NL; ++s) fold ^= __float_as_uint(total[s][0]) ^ __float_as_uint(total[s][3]);
            const uint32_t landed = loads_landed(fold);
            if (lane == 0) mbar_arrive_after(&empty[st], landed);
        }

        // ---- tile epilogue: partial sums -> shared memory, one barrier, one output per thread ----
        // Low-digit sums join the accumulator of digit 1 of their batch row (the main scales carry the factor
        // 256 between the digits).  Low set l holds row 8l + 2t + e in column 2t + e of lane t; that row's
        // digit-1 accumulator is column 2t' of main set (8l + 2t + e) / 4 in lane t' = 2 (t & 1) + e.
#pragma unroll
        for (int s = 0; s < NM && NL > 0; ++s) {
            const int l = s >> 1;
            const int src = (lane & ~3) | (2 * (s & 1) + (t >> 1));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float v0 = __shfl_sync(0xffffffffu, total[NM + (l < NL ? l : 0)][0 + 2 * h], src);
                const float v1 = __shfl_sync(0xffffffffu, total[NM + (l < NL ? l : 0)][1 + 2 * h], src);
                total[s][2 * h] += (t & 1) ? v1 : v0;
            }
        }
        float* pslot = partial + (tcount & 1u) * (kWarps * kPStride);
#pragma unroll
        for (int s = 0; s < NM; ++s)
            *reinterpret_cast<float4*>(pslot + warp * kPStride + (s * 32 + lane) * 4) =
                make_float4(total[s][0], total[s][1], total[s][2], total[s][3]);
        named_barrier_sync(1, kConsumerThreads);
        if (em < M) {
            float v = 0.0f, weight = 1.0f;
#pragma unroll
            for (int j = 3 - kDigitsOut; j < 3; ++j, weight *= 256.0f) {
                int set, cc;
                digit_slot(MODE, em, j, &set, &cc);
                const float* src = pslot + (set * 32 + (er & 7) * 4 + (cc >> 1)) * 4 + (er >> 3) * 2 + (cc & 1);
                float sum = src[0];
#pragma unroll
                for (int w = 1; w < kWarps; ++w) sum += src[w * kPStride];          // warp order: the same bits every run
                v = __fmaf_rn(weight, sum, v);
            }
            const int64_t n = tile * kRows + er;
            if (n < N && alive) {
                v = __fmul_rn(v, scale_per_row ? __ldg(wscales + n) : sw_all);
                if (bias) v = __fadd_rn(v, bias[n]);
                y[static_cast<int64_t>(em) * ldy + n] = v;
            }
        }
        // no second barrier: the next tile writes the other slot, and nobody reaches the tile after
        // that before every thread has passed the next barrier, i.e. finished reading this slot
    }
}

struct Plan {
    PreparedLayout L;
    int nstages;
    uint32_t smem;
    size_t planes_bytes;
};

bool make_plan(int64_t M, int64_t K, Plan* p) {
    p->L = prepared_layout(M, K);
    p->planes_bytes = p->L.bytes;
    for (int st = kMaxStages; st >= 2; --st) {
        const Smem S = smem_layout(st, p->L.nmain, p->L.nlow);
        if (S.total + 1024 <= static_cast<uint32_t>(kSmemLimit)) {
            p->nstages = st;
            p->smem = S.total + 1024;
            return true;
        }
    }
    return false;
}

template <int NM, int NL, int MODE>
int launch_variant(const LinearArgs& a, const Plan& p, const CUtensorMap& map_w, int grid) {
    static SmemOptIn optin;
    auto kernel = gemv_int8_nk_kernel<NM, NL, MODE>;
    SGQ_CUDA_TRY(optin.ensure(kernel, kSmemLimit));
    const bool overlap = stream_overlap_enabled();
    SGQ_CUDA_TRY(launch_kernel(prepare_x_i8_kernel, dim3(static_cast<unsigned>(a.M)), dim3(kPrepThreads), 0, a.stream, overlap, a.x, a.K,
                               p.L.mode, p.L.nmain, p.L.nlow, static_cast<uint8_t*>(a.workspace)));
    SGQ_CUDA_TRY(launch_kernel(kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), p.smem, a.stream, overlap, map_w,
                               static_cast<const uint8_t*>(a.workspace), a.scales, a.scheme == SGQ_PER_ROW ? 1 : 0, a.bias, a.y,
                               static_cast<int>(a.M), a.K, a.N, a.ldy, p.nstages));
    return SGQ_OK;
}

}  // namespace

bool gemv_i8_supported(const LinearArgs& a) {
    Plan p;
    return a.bits == 8 && a.layout == SGQ_LAYOUT_NK && a.M >= 1 && a.M <= kMaxM && a.K >= 128 && (a.K % 128) == 0 && a.K < (1LL << 17) &&
           a.N >= 1 && a.N < (1LL << 31) && aligned(a.wq, 16) && aligned(a.x, 16) && make_plan(a.M, a.K, &p);
}

size_t gemv_i8_workspace_bytes(int64_t M, int64_t K) {
    Plan p;
    if (M < 1 || M > kMaxM || K < 128 || (K % 128) != 0 || K >= (1LL << 17) || !make_plan(M, K, &p)) return 0;
    return (p.planes_bytes + 255) / 256 * 256;
}

int launch_linear_gemv_i8(const LinearArgs& a) {
    Plan p;
    if (!gemv_i8_supported(a) || !make_plan(a.M, a.K, &p)) {
        set_error("INT8 decode path needs weights stored [N,K], M<=16, K%%128==0, K<131072, 16-byte aligned x and codes");
        return SGQ_ERR_UNSUPPORTED;
    }
    const size_t need = gemv_i8_workspace_bytes(a.M, a.K);
    if (!a.workspace || a.workspace_bytes < need || !aligned(a.workspace, 256)) {
        set_error("INT8 decode path needs %zu bytes of 256-byte aligned workspace", need);
        return SGQ_ERR_WORKSPACE;
    }
    CUtensorMap map_w;
    const uint64_t steps = static_cast<uint64_t>(a.K / kStepK);
    const uint64_t dims[3] = {128, static_cast<uint64_t>(a.N), steps};
    const uint64_t strides[2] = {static_cast<uint64_t>(a.K), 128};
    const uint32_t box[3] = {128, kRows, kSteps};
    if (!make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    const int64_t ntiles = ceil_div(a.N, kRows);
    const int grid = static_cast<int>(ntiles < sm_count() ? ntiles : sm_count());
    if (p.L.mode == 0) return launch_variant<1, 0, 0>(a, p, map_w, grid);
    if (p.L.mode == 1) return launch_variant<1, 0, 1>(a, p, map_w, grid);
    switch (p.L.nmain) {                 // three rows or more: ceil(M / 4) main sets, ceil(M / 8) low sets
        case 1: return launch_variant<1, 1, 2>(a, p, map_w, grid);
        case 2: return launch_variant<2, 1, 2>(a, p, map_w, grid);
        case 3: return launch_variant<3, 2, 2>(a, p, map_w, grid);
        default: return launch_variant<4, 2, 2>(a, p, map_w, grid);
    }
}

}  // namespace sgq
