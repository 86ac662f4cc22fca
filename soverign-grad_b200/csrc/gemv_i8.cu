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
//   * there is no per-group scale, so the int32 accumulators run over the WHOLE of K (exact:
//     |sum| <= K * 127 * 128 < 2^31 for K < 2^17) and are converted to fp32 once per output;
//   * the activation digit planes (same fixed-point digits as gemv_prepare.cuh, laid out for the
//     natural k order of an int8 B fragment) are written once by a conversion kernel and stream
//     through the same pipeline stages as the weights, 32 groups at a time, from L2.  They are
//     never resident as a whole, so K is not limited by shared memory (K = 8192 at M = 16 runs);
//   * tile epilogue: every warp leaves its int32 partial sums in one of two shared-memory slots,
//     one named barrier, then thread (m, row) adds the eight partials (integers: any order gives
//     the same bits), recombines the digits, applies 2^-p, the weight scale and the bias.
//
// y[m,n] = ((sum_j 256^j * S_j[m,n]) * 2^-p_m) * scale[n] + bias[n],  S_j exact integers.
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

// D(16x8,s32) = A(16x32,s8,row) * B(32x8,s8,col) + C
__device__ __forceinline__ void mma_s8s8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Digit planes for the int8 kernel: [group K/32][set][col 8][t 4] x 8 bytes, the 8 bytes of (col, t)
// being the digits of k = 32*group + 4t + {0,1,2,3} (b0) and 32*group + 16 + 4t + {0,1,2,3} (b1);
// column col = m * ndigits + j.  Followed by 16 fp32: 2^-p of every row.
__global__ void __launch_bounds__(kPrepThreads) prepare_x_i8_kernel(const float* __restrict__ x, int64_t K, int ndigits, int nsets,
                                                                   uint8_t* __restrict__ planes) {
    __shared__ float red[kPrepThreads / 32];
    pdl_launch_dependents();
    pdl_wait();                                        // x comes from the kernel before this one
    const int m = blockIdx.x, lane = threadIdx.x & 31;
    const float* xr = x + static_cast<int64_t>(m) * K;
    const int chunks = static_cast<int>(K / 8);
    float mx = 0.0f;
    for (int c = threadIdx.x; c < chunks; c += kPrepThreads) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(xr) + 2 * c);
        const float4 b = __ldg(reinterpret_cast<const float4*>(xr) + 2 * c + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        mx = fmaxf(mx, absmax8(v));
    }
    mx = warp_max(mx);
    if (lane == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    float all = red[lane < kPrepThreads / 32 ? lane : 0];
    all = warp_max(all);
    float P, invP;
    row_scale(__float_as_uint(all), ndigits == 3 ? 22 : 14, &P, &invP);
    const size_t groups = static_cast<size_t>(K / 32);
    if (threadIdx.x == 0) reinterpret_cast<float*>(planes + groups * nsets * 256)[m] = invP;
    for (int c = threadIdx.x; c < chunks; c += kPrepThreads) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(xr) + 2 * c);          // second read: L1/L2
        const float4 b = __ldg(reinterpret_cast<const float4*>(xr) + 2 * c + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t db[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) db[j] = digit_bytes(__float2int_rn(v[j] * P));
        const int group = c >> 2, q = c & 3;           // chunk q of its group: k = 8q .. 8q+7
        const int t0 = 2 * (q & 1), half = q >> 1;     // k < 16 -> b0, else b1; words of t0 and t0 + 1
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            if (j < ndigits) {
                const int col = m * ndigits + j, set = col >> 3, cc = col & 7;
                uint8_t* base = planes + (static_cast<size_t>(group) * nsets + set) * 256 + (cc * 4 + t0) * 8 + half * 4;
                *reinterpret_cast<uint32_t*>(base) = gather_byte(db[0], db[1], db[2], db[3], j);
                *reinterpret_cast<uint32_t*>(base + 8) = gather_byte(db[4], db[5], db[6], db[7], j);
            }
        }
    }
}

struct Smem {
    uint32_t stage_bytes, partial_off, misc_off, total;
};

__host__ __device__ inline Smem smem_layout(int nstages, int nsets) {
    Smem s;
    s.stage_bytes = kStageW + kGroupsPerStage * 256u * nsets;
    s.partial_off = nstages * s.stage_bytes;
    s.misc_off = s.partial_off + 2u * kWarps * (512u * nsets + 16u);      // two slots of per-warp int32 partial sums (padded)
    s.total = s.misc_off + 2u * kMaxStages * 8u + 16u;
    return s;
}

template <int NSETS>
__global__ void __launch_bounds__(kThreads, 1)
gemv_int8_nk_kernel(const __grid_constant__ CUtensorMap map_w, const uint8_t* __restrict__ planes, const float* __restrict__ wscales,
                    int scale_per_row, const float* __restrict__ bias, float* __restrict__ y, int M, int ndigits, int64_t K, int64_t N,
                    int64_t ldy, int nstages) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const Smem L = smem_layout(nstages, NSETS);
    int* partial = reinterpret_cast<int*>(smem + L.partial_off);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.misc_off);
    uint64_t* empty = full + kMaxStages;
    constexpr int kPStride = 128 * NSETS + 4;       // ints per warp in a partial-sum slot

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
                    const uint32_t pbytes = static_cast<uint32_t>(ng) * 256u * NSETS;
                    // steps past K/128 are out of range in the third dimension: zero-filled, still counted
                    mbar_arrive_expect_tx(&full[st], kStageW + pbytes);
                    uint8_t* sw = smem + st * L.stage_bytes;
                    tma_load_3d(sw, &map_w, &full[st], 0, static_cast<int32_t>(tile * kRows), c0);
                    bulk_copy_g2s(sw + kStageW, planes + static_cast<size_t>(g0) * 256u * NSETS, pbytes, &full[st]);
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int g = lane >> 2, t = lane & 3;
    uint32_t woff[4][2];                            // this lane's word in chunks 2i and 2i+1 of rows g and g+8 (swizzle: chunk ^ row)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        woff[i][0] = g * 128 + (((2 * i) ^ g) << 4) + t * 4;
        woff[i][1] = g * 128 + (((2 * i + 1) ^ g) << 4) + t * 4;
    }
    const float* inv_p = reinterpret_cast<const float*>(planes + static_cast<size_t>(groups_total) * 256u * NSETS);
    // epilogue role of this thread: output (row er of the tile, batch row em)
    const int em = threadIdx.x >> 4, er = threadIdx.x & 15;
    float my_inv_p = 0.f;
    if (em < M) my_inv_p = __ldg(inv_p + em);
    const float sw_all = scale_per_row ? 1.0f : __ldg(wscales);

    bool alive = true;
    uint32_t seq = 0, tcount = 0;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
        int acc[NSETS][4];
#pragma unroll
        for (int s = 0; s < NSETS; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][i] = 0;

        for (int c0 = 0; c0 < spt; c0 += kSteps, ++seq) {
            const int st = seq % nstages;
            const uint32_t ph = (seq / nstages) & 1u;
            if (alive && !mbar_wait(&full[st], ph)) {
                report(kDevErrFullWait, seq);
                alive = false;
            }
            const int step = c0 + warp;
            if (alive && step < spt) {
                const uint8_t* wbox = smem + st * L.stage_bytes + warp * (kRows * 128);
                const uint8_t* xg = smem + st * L.stage_bytes + kStageW + (warp * 4) * (256 * NSETS) + lane * 8;
                uint32_t a[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    a[i][0] = *reinterpret_cast<const uint32_t*>(wbox + woff[i][0]);             // row g,   k = 32i + 4t..
                    a[i][1] = *reinterpret_cast<const uint32_t*>(wbox + 1024 + woff[i][0]);      // row g+8
                    a[i][2] = *reinterpret_cast<const uint32_t*>(wbox + woff[i][1]);             // row g,   k = 32i + 16 + 4t..
                    a[i][3] = *reinterpret_cast<const uint32_t*>(wbox + 1024 + woff[i][1]);      // row g+8
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int s = 0; s < NSETS; ++s) {
                        const uint2 xb = *reinterpret_cast<const uint2*>(xg + i * (256 * NSETS) + s * 256);
                        mma_s8s8_16832(acc[s], a[i], xb.x, xb.y);
                    }
                }
            }
            // everything loaded from the stage has been consumed once the accumulators are final
            uint32_t fold = 0;
#pragma unroll
            for (int s = 0; s < NSETS; ++s) fold ^= static_cast<uint32_t>(acc[s][0] ^ acc[s][3]);
            const uint32_t landed = loads_landed(fold);
            if (lane == 0) mbar_arrive_after(&empty[st], landed);
        }

        // ---- tile epilogue: partial sums -> shared memory, one barrier, one output per thread ----
        int* pslot = partial + (tcount & 1u) * (kWarps * kPStride);
#pragma unroll
        for (int s = 0; s < NSETS; ++s)
            *reinterpret_cast<int4*>(pslot + warp * kPStride + (s * 32 + lane) * 4) = make_int4(acc[s][0], acc[s][1], acc[s][2], acc[s][3]);
        named_barrier_sync(1, kConsumerThreads);
        if (em < M) {
            float v = 0.0f, weight = 1.0f;
            for (int j = 0; j < ndigits; ++j, weight *= 256.0f) {
                const int col = em * ndigits + j, set = col >> 3, cc = col & 7;
                const int* src = pslot + (set * 32 + (er & 7) * 4 + (cc >> 1)) * 4 + (er >> 3) * 2 + (cc & 1);
                int sum = 0;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) sum += src[w * kPStride];
                v = __fmaf_rn(weight, static_cast<float>(sum), v);
            }
            const int64_t n = tile * kRows + er;
            if (n < N && alive) {
                v = __fmul_rn(__fmul_rn(v, my_inv_p), scale_per_row ? __ldg(wscales + n) : sw_all);
                if (bias) v = __fadd_rn(v, bias[n]);
                y[static_cast<int64_t>(em) * ldy + n] = v;
            }
        }
        // no second barrier: the next tile writes the other slot, and nobody reaches the tile after
        // that before every thread has passed the next barrier, i.e. finished reading this slot
    }
}

struct Plan {
    int ndigits, nsets, nstages;
    uint32_t smem;
    size_t planes_bytes;
};

bool make_plan(int64_t M, int64_t K, Plan* p) {
    const PreparedLayout L = prepared_layout(M, K);
    p->ndigits = L.ndigits;
    p->nsets = L.nsets;
    p->planes_bytes = static_cast<size_t>(K / 32) * p->nsets * 256 + kMaxM * 4;
    for (int st = kMaxStages; st >= 2; --st) {
        const Smem S = smem_layout(st, p->nsets);
        if (S.total + 1024 <= static_cast<uint32_t>(kSmemLimit)) {
            p->nstages = st;
            p->smem = S.total + 1024;
            return true;
        }
    }
    return false;
}

template <int NSETS>
int launch_variant(const LinearArgs& a, const Plan& p, const CUtensorMap& map_w, int grid) {
    static SmemOptIn optin;
    auto kernel = gemv_int8_nk_kernel<NSETS>;
    SGQ_CUDA_TRY(optin.ensure(kernel, kSmemLimit));
    const bool overlap = stream_overlap_enabled();
    SGQ_CUDA_TRY(launch_kernel(prepare_x_i8_kernel, dim3(static_cast<unsigned>(a.M)), dim3(kPrepThreads), 0, a.stream, overlap, a.x, a.K,
                               p.ndigits, p.nsets, static_cast<uint8_t*>(a.workspace)));
    SGQ_CUDA_TRY(launch_kernel(kernel, dim3(static_cast<unsigned>(grid)), dim3(kThreads), p.smem, a.stream, overlap, map_w,
                               static_cast<const uint8_t*>(a.workspace), a.scales, a.scheme == SGQ_PER_ROW ? 1 : 0, a.bias, a.y,
                               static_cast<int>(a.M), p.ndigits, a.K, a.N, a.ldy, p.nstages));
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
    switch (p.nsets) {
        case 1: return launch_variant<1>(a, p, map_w, grid);
        case 2: return launch_variant<2>(a, p, map_w, grid);
        case 3: return launch_variant<3>(a, p, map_w, grid);
        default: return launch_variant<4>(a, p, map_w, grid);
    }
}

}  // namespace sgq
