// Decode-shape forward (M <= 8) for INT4 g=32 weights stored [N,K]:  y = x * deq(W)^T + bias.
//
// HBM-bound: every packed byte and every scale is read exactly once.
//   bytes per weight row-block = 16 rows * (K/2 + K/32*4);  x (M*K*4) and y are negligible.
//
// Structure (one persistent CTA per SM, 8 consumer warps + 1 producer warp):
//   * the producer thread streams [16 rows x 128 B] boxes of packed weights (128-byte swizzle,
//     so the per-row word reads below are bank-conflict free) and [16 rows x 32] boxes of fp32
//     scales through TMA into a ring of stages guarded by full/empty mbarriers;
//   * x is converted once per CTA to split bf16 (hi + lo, 16 significant bits) and kept in
//     shared memory in the order the B fragments want it;
//   * a consumer warp owns one 256-k box of a stage: nibbles become exact bf16 integers in
//     registers with one LOP3 per pair (0x4300 | (nibble ^ 8) = 136 + code, minus 136), the
//     16x8 products of 16 rows with the hi/lo columns of up to 4 (8) batch rows come from
//     mma.sync m16n8k16 with fp32 accumulators, and the group scale is applied in fp32 to each
//     32-k group sum: y = sum_g scale[n,g] * (sum_{k in g} code[n,k] * x[k]);
//   * the 8 warps' partial sums of a 16-row tile are added in warp order through shared memory
//     (fixed order -> run-to-run deterministic), hi+lo are joined, bias is added, y is stored.
//
// The accumulation differs from the reference's single fp32 chain only in rounding (products
// with 16-bit x are exact, group sums are fp32): max error ~1e-5 relative, inside the 1e-3 bound.
#include <cuda_bf16.h>

#include "sgq_common.cuh"
#include "sm100_ptx.cuh"

namespace sgq {

__device__ uint32_t g_status_gemv = 0;  // see sm100_ptx.cuh: (code << 24) | detail

cudaError_t read_status_gemv(uint32_t* v, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(v, g_status_gemv, sizeof(uint32_t));
    if (e == cudaSuccess && clear && *v != 0) {
        const uint32_t zero = 0;
        e = cudaMemcpyToSymbol(g_status_gemv, &zero, sizeof(zero));
    }
    return e;
}

namespace {

constexpr int kRows = 16;                  // rows of W per tile (mma M)
constexpr int kStepK = 256;                // k per box
constexpr int kConsumerWarps = 8;          // one box each per stage
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kWBoxBytes = kRows * 128;    // 2048
constexpr int kSBoxBytes = kRows * 128;    // 16 rows x 32 fp32 = 4 steps worth of scales
constexpr int kStageW = kConsumerWarps * kWBoxBytes;          // 16384
constexpr int kStageS = 2 * kSBoxBytes;                       // 4096
constexpr int kStageBytes = kStageW + kStageS;                // 20480
constexpr int kMaxStages = 8;
constexpr int kSmemLimit = 227 * 1024;

struct Smem {
    // offsets from a 1024-byte aligned base
    uint32_t stages_off, x_off, partial_off, bars_off, total;
};

__host__ __device__ inline Smem smem_layout(int nstages, int64_t K, int nsets) {
    Smem s;
    s.stages_off = 0;
    s.x_off = nstages * kStageBytes;
    const uint32_t ksteps32 = static_cast<uint32_t>((K + kStepK - 1) / kStepK) * (kStepK / 32);  // groups, padded
    s.partial_off = s.x_off + ksteps32 * 512u * nsets;
    s.bars_off = s.partial_off + 2u * kConsumerWarps * 512u * nsets;  // double-buffered partials
    s.total = s.bars_off + 2u * kMaxStages * 8u + 16u;
    return s;
}

__device__ __forceinline__ void report(uint32_t code, uint32_t detail) {
    atomicCAS(&g_status_gemv, 0u, (code << 24) | (detail & 0xFFFFFFu));
}

// split x into bf16 hi + bf16 lo (x ~= hi + lo, 16 significant bits)
__device__ __forceinline__ void split_bf16(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    const float r = v - __bfloat162float(hi);
    lo = (fabsf(v) <= 3.0e38f) ? __float2bfloat16_rn(r) : __float2bfloat16_rn(0.0f);
}

__device__ __forceinline__ uint32_t pack_bf16(__nv_bfloat16 a, __nv_bfloat16 b) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(a)) | (static_cast<uint32_t>(__bfloat16_as_ushort(b)) << 16);
}

// 8 nibbles of one row-word -> four bf16x2 registers holding the exact codes
//   p[j] = (code of nibble j, code of nibble j+4)
__device__ __forceinline__ void nibbles_to_bf16(uint32_t w, uint32_t (&p)[4]) {
    const uint32_t kMagic = 0x43084308u;   // bf16 136.0 in both halves; ^8 folds the sign bias in
    const uint32_t k136 = 0x43084308u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t v = ((w >> (4 * j)) & 0x000F000Fu) ^ kMagic;   // 136 + code, exact in bf16
        uint32_t r;
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(k136));
        p[j] = r;
    }
}

template <int NSETS>
__global__ void __launch_bounds__(kThreads, 1)
gemv_int4_nk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                    const float* __restrict__ x, const float* __restrict__ bias, float* __restrict__ y, int M,
                    int64_t K, int64_t N, int64_t ldy, int nstages) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const Smem L = smem_layout(nstages, K, NSETS);
    uint8_t* stages = smem + L.stages_off;
    uint8_t* xs = smem + L.x_off;
    float* partial = reinterpret_cast<float*>(smem + L.partial_off);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars_off);
    uint64_t* empty = full + kMaxStages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t ntiles = (N + kRows - 1) / kRows;
    const int spt = static_cast<int>((K + kStepK - 1) / kStepK);   // steps (boxes) per tile
    const int sgroups = static_cast<int>(K / 32);                  // scale columns

    if (threadIdx.x == 0) {
        for (int i = 0; i < nstages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kConsumerWarps);
        }
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            tma_prefetch_descriptor(&map_w);
            tma_prefetch_descriptor(&map_s);
            uint32_t seq = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                for (int c0 = 0; c0 < spt; c0 += kConsumerWarps, ++seq) {
                    const int st = seq % nstages;
                    const uint32_t ph = (seq / nstages) & 1u;
                    if (!mbar_wait(&empty[st], ph ^ 1u)) {
                        report(kDevErrEmptyWait, seq);
                        ok = false;
                        break;
                    }
                    const int cnt = (spt - c0 < kConsumerWarps) ? spt - c0 : kConsumerWarps;
                    const int sboxes = (c0 * 8 + 32 < sgroups) ? 2 : 1;
                    mbar_arrive_expect_tx(&full[st], cnt * kWBoxBytes + sboxes * kSBoxBytes);
                    uint8_t* sw = stages + st * kStageBytes;
                    for (int b = 0; b < cnt; ++b)
                        tma_load_2d(sw + b * kWBoxBytes, &map_w, &full[st], (c0 + b) * 128, static_cast<int32_t>(tile * kRows));
                    for (int b = 0; b < sboxes; ++b)
                        tma_load_2d(sw + kStageW + b * kSBoxBytes, &map_s, &full[st], c0 * 8 + b * 32,
                                    static_cast<int32_t>(tile * kRows));
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // x -> split bf16, fragment order: [group s][set][col n (8)][t (4)] x 16 bytes, the 8 values
    // of (s, t) being k = 32s + 8t + {0,4,1,5,2,6,3,7}.
    {
        const int64_t chunks = static_cast<int64_t>(spt) * (kStepK / 8);   // 8-float chunks per row (padded)
        const int mrows = NSETS * 4;                                       // batch rows covered
        for (int64_t it = threadIdx.x; it < chunks * mrows; it += kConsumerThreads) {
            const int m = static_cast<int>(it / chunks);
            const int64_t c = it % chunks;                                 // chunk = (s, t)
            float v[8];
            if (m < M && (c + 1) * 8 <= K) {
                const float4 a = *reinterpret_cast<const float4*>(x + static_cast<int64_t>(m) * K + c * 8);
                const float4 b = *reinterpret_cast<const float4*>(x + static_cast<int64_t>(m) * K + c * 8 + 4);
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.0f;
            }
            __nv_bfloat16 hi[8], lo[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) split_bf16(v[j], hi[j], lo[j]);
            const uint4 H = make_uint4(pack_bf16(hi[0], hi[4]), pack_bf16(hi[1], hi[5]), pack_bf16(hi[2], hi[6]),
                                       pack_bf16(hi[3], hi[7]));
            const uint4 Lo = make_uint4(pack_bf16(lo[0], lo[4]), pack_bf16(lo[1], lo[5]), pack_bf16(lo[2], lo[6]),
                                        pack_bf16(lo[3], lo[7]));
            const int64_t s = c >> 2;
            const int t = static_cast<int>(c & 3);
            uint8_t* base = xs + s * (512 * NSETS);
            if (NSETS == 1) {
                // columns 0..3 = hi of batch rows 0..3, columns 4..7 = lo
                *reinterpret_cast<uint4*>(base + (m * 4 + t) * 16) = H;
                *reinterpret_cast<uint4*>(base + ((m + 4) * 4 + t) * 16) = Lo;
            } else {
                // set 0 = hi of batch rows 0..7, set 1 = lo
                *reinterpret_cast<uint4*>(base + (m * 4 + t) * 16) = H;
                *reinterpret_cast<uint4*>(base + 512 + (m * 4 + t) * 16) = Lo;
            }
        }
    }
    named_barrier_sync(1, kConsumerThreads);

    const int g = lane >> 2, t = lane & 3;
    uint32_t seq = 0;
    int tile_parity = 0;
    bool alive = true;   // false after a wait ran out: skip the math but keep every barrier balanced
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, tile_parity ^= 1) {
        float total[NSETS][4];
#pragma unroll
        for (int s = 0; s < NSETS; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) total[s][i] = 0.0f;

        for (int c0 = 0; c0 < spt; c0 += kConsumerWarps, ++seq) {
            const int st = seq % nstages;
            const uint32_t ph = (seq / nstages) & 1u;
            if (alive && !mbar_wait(&full[st], ph)) {
                report(kDevErrFullWait, seq);
                alive = false;
            }
            const int step = c0 + warp;
            if (alive && step < spt) {
                const uint8_t* wbox = stages + st * kStageBytes + warp * kWBoxBytes;
                const uint8_t* sbox = stages + st * kStageBytes + kStageW + (warp >> 2) * kSBoxBytes;
                // the 8 scales of this step for rows g and g+8: 16-byte chunks (warp&3)*2 and +1,
                // swizzled by the row (chunk ^ (row & 7)); rows g+8 live in the second 1 KiB atom.
                float sc_lo[8], sc_hi[8];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int chunk = ((warp & 3) * 2 + h) ^ g;
                    const float4 a = *reinterpret_cast<const float4*>(sbox + g * 128 + chunk * 16);
                    const float4 b = *reinterpret_cast<const float4*>(sbox + 1024 + g * 128 + chunk * 16);
                    sc_lo[4 * h + 0] = a.x; sc_lo[4 * h + 1] = a.y; sc_lo[4 * h + 2] = a.z; sc_lo[4 * h + 3] = a.w;
                    sc_hi[4 * h + 0] = b.x; sc_hi[4 * h + 1] = b.y; sc_hi[4 * h + 2] = b.z; sc_hi[4 * h + 3] = b.w;
                }
                const uint8_t* xstep = xs + static_cast<int64_t>(step) * 8 * (512 * NSETS) + lane * 16;
#pragma unroll
                for (int s8 = 0; s8 < 8; ++s8) {
                    const int chunk = (s8 ^ g) * 16 + t * 4;
                    const uint32_t w_lo = *reinterpret_cast<const uint32_t*>(wbox + g * 128 + chunk);
                    const uint32_t w_hi = *reinterpret_cast<const uint32_t*>(wbox + 1024 + g * 128 + chunk);
                    uint32_t pl[4], phh[4];
                    nibbles_to_bf16(w_lo, pl);
                    nibbles_to_bf16(w_hi, phh);
                    const uint32_t a1[4] = {pl[0], phh[0], pl[1], phh[1]};
                    const uint32_t a2[4] = {pl[2], phh[2], pl[3], phh[3]};
#pragma unroll
                    for (int s = 0; s < NSETS; ++s) {
                        const uint4 xb = *reinterpret_cast<const uint4*>(xstep + s8 * (512 * NSETS) + s * 512);
                        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        float d[4];
                        mma_bf16_16816(d, a1, xb.x, xb.y, zero);
                        mma_bf16_16816(d, a2, xb.z, xb.w, d);
                        total[s][0] = __fmaf_rn(sc_lo[s8], d[0], total[s][0]);
                        total[s][1] = __fmaf_rn(sc_lo[s8], d[1], total[s][1]);
                        total[s][2] = __fmaf_rn(sc_hi[s8], d[2], total[s][2]);
                        total[s][3] = __fmaf_rn(sc_hi[s8], d[3], total[s][3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }

        // ---- tile epilogue: fixed-order sum over the 8 warps, join hi+lo, bias, store ----
        float* pbuf = partial + tile_parity * (kConsumerWarps * 128 * NSETS);
#pragma unroll
        for (int s = 0; s < NSETS; ++s)
            *reinterpret_cast<float4*>(pbuf + ((warp * NSETS + s) * 32 + lane) * 4) =
                make_float4(total[s][0], total[s][1], total[s][2], total[s][3]);
        named_barrier_sync(1, kConsumerThreads);
        {
            // thread -> (row r of the tile, batch row m)
            const int r = threadIdx.x >> 3, m = threadIdx.x & 7;
            if (r < kRows && m < M) {
                const int gg = r & 7, half = r >> 3;
                float v;
                if (NSETS == 1) {
                    // hi in column m, lo in column m+4
                    const int l_hi = gg * 4 + (m >> 1), l_lo = gg * 4 + ((m + 4) >> 1);
                    const int idx = half * 2 + (m & 1);
                    float vh = 0.0f, vl = 0.0f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) {
                        vh += pbuf[(w * 32 + l_hi) * 4 + idx];
                        vl += pbuf[(w * 32 + l_lo) * 4 + idx];
                    }
                    v = vh + vl;
                } else {
                    const int l = gg * 4 + (m >> 1);
                    const int idx = half * 2 + (m & 1);
                    float vh = 0.0f, vl = 0.0f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) {
                        vh += pbuf[((w * 2 + 0) * 32 + l) * 4 + idx];
                        vl += pbuf[((w * 2 + 1) * 32 + l) * 4 + idx];
                    }
                    v = vh + vl;
                }
                const int64_t n = tile * kRows + r;
                if (n < N) {
                    if (bias) v += bias[n];
                    y[static_cast<int64_t>(m) * ldy + n] = v;
                }
            }
        }
    }
}

struct Plan {
    int nsets;
    int nstages;
    uint32_t smem;
};

bool make_plan(int64_t M, int64_t K, Plan* p) {
    p->nsets = (M <= 4) ? 1 : 2;
    for (int st = kMaxStages; st >= 2; --st) {
        const Smem L = smem_layout(st, K, p->nsets);
        if (L.total + 1024 <= static_cast<uint32_t>(kSmemLimit)) {
            p->nstages = st;
            p->smem = L.total + 1024;
            return true;
        }
    }
    return false;
}

}  // namespace

bool gemv_supported(const LinearArgs& a) {
    Plan p;
    return a.bits == 4 && a.layout == SGQ_LAYOUT_NK && a.group == 32 && a.M >= 1 && a.M <= 8 && a.K >= 128 &&
           (a.K % 128) == 0 && a.N >= 1 && a.N < (1LL << 31) && a.K < (1LL << 31) && aligned(a.wq, 16) &&
           aligned(a.scales, 16) && aligned(a.x, 16) && make_plan(a.M, a.K, &p);
}

size_t gemv_workspace_bytes(int, int64_t, int64_t, int64_t, int) { return 0; }

int launch_linear_gemv(const LinearArgs& a) {
    Plan p;
    if (!gemv_supported(a) || !make_plan(a.M, a.K, &p)) {
        set_error("decode path needs INT4 g=32, layout NK, M<=8, K%%128==0, 16-byte aligned x/packed/scales");
        return SGQ_ERR_UNSUPPORTED;
    }
    CUtensorMap map_w, map_s;
    if (!make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, static_cast<uint64_t>(a.K / 2),
                            static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 2), 128, kRows,
                            CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    if (!make_tensor_map_2d(&map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.scales, static_cast<uint64_t>(a.K / 32),
                            static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 32) * 4, 32, kRows,
                            CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    const int64_t ntiles = ceil_div(a.N, kRows);
    const int grid = static_cast<int>(ntiles < sm_count() ? ntiles : sm_count());
    static SmemOptIn optin1, optin2;
    if (p.nsets == 1) {
        SGQ_CUDA_TRY(optin1.ensure(gemv_int4_nk_kernel<1>, kSmemLimit));
        gemv_int4_nk_kernel<1><<<grid, kThreads, p.smem, a.stream>>>(map_w, map_s, a.x, a.bias, a.y,
                                                                      static_cast<int>(a.M), a.K, a.N, a.ldy, p.nstages);
    } else {
        SGQ_CUDA_TRY(optin2.ensure(gemv_int4_nk_kernel<2>, kSmemLimit));
        gemv_int4_nk_kernel<2><<<grid, kThreads, p.smem, a.stream>>>(map_w, map_s, a.x, a.bias, a.y,
                                                                      static_cast<int>(a.M), a.K, a.N, a.ldy, p.nstages);
    }
    SGQ_LAUNCH_CHECK("gemv_int4_nk_kernel");
    return SGQ_OK;
}

}  // namespace sgq
