// Prefill-shape forward on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// weights stored [N,K]:  y[M,N] = x[M,K] * deq(W)^T + bias.
//
// Two modes share one persistent, warp-specialised kernel (one CTA per SM, 128 x 256 output
// tile, two TMEM accumulators of 256 columns so the epilogue of tile i overlaps the main loop
// of tile i+1):
//   kI8   kind::i8 — INT8 weight codes and per-row quantized INT8 activations go from HBM to
//         shared memory by TMA untouched (128-byte swizzle), int32 accumulation is exact, the
//         epilogue applies sx[m] * sw[n].  k-block = 128.
//   kBF16 kind::f16 (bf16 x bf16 -> fp32) — activations are pre-converted to bf16; packed INT4
//         weights arrive by TMA as raw nibbles and dequant warps expand them in shared memory
//         to bf16 (exact integer from one LOP3 per pair, times the bf16-rounded group scale)
//         directly in the swizzled K-major layout the MMA reads.  k-block = 64 (two groups).
//         Two groups of 8 dequant warps take alternate k-blocks, so two k-blocks are being
//         expanded while a third is being multiplied.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer (one thread), 2..5 = epilogue (TMEM lane
// quarter = warp % 4), 6..21 = dequant (kBF16 only; two groups of 8).  All waits are bounded; a wait that runs
// out records a code in the device status word and the role winds down to the common exit.
#include <cuda_bf16.h>

#include "sgq_common.cuh"
#include "sm100_ptx.cuh"

namespace sgq {

__device__ uint32_t g_status_gemm = 0;

cudaError_t read_status_gemm(uint32_t* v, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(v, g_status_gemm, sizeof(uint32_t));
    if (e == cudaSuccess && clear && *v != 0) {
        const uint32_t zero = 0;
        e = cudaMemcpyToSymbol(g_status_gemm, &zero, sizeof(zero));
    }
    return e;
}

namespace {

enum Mode { kI8 = 0, kBF16 = 1 };

constexpr int BM = 128, BN = 256;
constexpr int kABytes = BM * 128;     // 128 rows x 128 B
constexpr int kBBytes = BN * 128;     // 256 rows x 128 B
constexpr int kRawBytes = BN * 32;    // 256 rows x 64 nibbles
constexpr int kDequantWarps = 8;      // per group: one thread per row of the 256-row weight tile
constexpr int kDequantGroups = 2;     // groups take alternate k-blocks
constexpr int kEpilogueWarp0 = 2;
constexpr int kDequantWarp0 = 6;
constexpr int kTmemCols = 512;

template <int MODE>
struct Cfg {
    static constexpr int kStages = MODE == kI8 ? 4 : 3;
    static constexpr int kBlockK = MODE == kI8 ? 128 : 64;          // elements per k-block
    static constexpr int kUmmaK = MODE == kI8 ? 32 : 16;            // elements per instruction (32 bytes)
    static constexpr int kWarps = MODE == kI8 ? 6 : 6 + kDequantWarps * kDequantGroups;
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kStageBytes = kABytes + kBBytes + (MODE == kBF16 ? kRawBytes : 0);
    static constexpr int kBarOffset = kStages * kStageBytes;
    static constexpr int kSmemBytes = kBarOffset + 256 + 1024;      // barriers + alignment slack
};

struct Params {
    const float* bias;      // [N] or null
    float* y;               // [M, ldy]
    int64_t ldy;
    int64_t M, N, K;
    // kI8
    const float* sx;        // [M] activation scales
    const float* sw;        // weight scales: [1] or [N]
    int sw_per_row;
    int32_t* acc_out;       // optional [M,N]
    // kBF16
    const float* wscales;   // [N, K/32]
};

__device__ __forceinline__ void report(uint32_t code, uint32_t detail) {
    atomicCAS(&g_status_gemm, 0u, (code << 24) | (detail & 0xFFFFFFu));
}

template <int MODE>
__global__ void __launch_bounds__(Cfg<MODE>::kThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, Params p) {
    using C = Cfg<MODE>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBarOffset);
    uint64_t* full = bars;                         // [kStages] operands of a k-block are in shared memory
    uint64_t* empty = bars + C::kStages;           // [kStages] the MMAs reading the stage have completed
    uint64_t* raw_full = bars + 2 * C::kStages;    // [kStages] packed nibbles landed (kBF16)
    uint64_t* raw_empty = bars + 3 * C::kStages;   // [kStages] packed nibbles consumed (kBF16)
    uint64_t* tmem_full = bars + 4 * C::kStages;   // [2] accumulator complete
    uint64_t* tmem_empty = tmem_full + 2;          // [2] accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
    const int64_t tiles = m_tiles * n_tiles;
    const int kblocks = static_cast<int>((p.K + C::kBlockK - 1) / C::kBlockK);

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::kStages; ++i) {
            mbar_init(&full[i], MODE == kI8 ? 1 : 1 + kDequantWarps);
            mbar_init(&empty[i], 1);
            mbar_init(&raw_full[i], 1);
            mbar_init(&raw_empty[i], kDequantWarps);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&tmem_full[i], 1);
            mbar_init(&tmem_empty[i], 4);
        }
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == kEpilogueWarp0) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            tma_prefetch_descriptor(&map_a);
            tma_prefetch_descriptor(&map_b);
            uint32_t it = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                const int32_t m0 = static_cast<int32_t>((tile % m_tiles) * BM);
                const int32_t n0 = static_cast<int32_t>((tile / m_tiles) * BN);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1u;
                    uint8_t* st = smem + s * C::kStageBytes;
                    if (!mbar_wait(&empty[s], ph ^ 1u)) { report(kDevErrEmptyWait, it); alive = false; break; }
                    if (MODE == kI8) {
                        mbar_arrive_expect_tx(&full[s], kABytes + kBBytes);
                        tma_load_2d(st, &map_a, &full[s], kb * C::kBlockK, m0);
                        tma_load_2d(st + kABytes, &map_b, &full[s], kb * C::kBlockK, n0);
                    } else {
                        mbar_arrive_expect_tx(&full[s], kABytes);
                        tma_load_2d(st, &map_a, &full[s], kb * C::kBlockK, m0);
                        if (!mbar_wait(&raw_empty[s], ph ^ 1u)) { report(kDevErrEmptyWait, 0x800000u | it); alive = false; break; }
                        mbar_arrive_expect_tx(&raw_full[s], kRawBytes);
                        tma_load_2d(st + kABytes + kBBytes, &map_b, &raw_full[s], kb * (C::kBlockK / 2), n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0) {
            const uint32_t idesc = (MODE == kI8) ? umma_idesc(2u, 1u, BM, BN) : umma_idesc(1u, 1u, BM, BN);
            uint32_t it = 0, tcount = 0;
            bool alive = true;
            for (int64_t tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++tcount) {
                const uint32_t buf = tcount & 1u, aph = (tcount >> 1) & 1u;
                if (!mbar_wait(&tmem_empty[buf], aph ^ 1u)) { report(kDevErrMmaWait, tcount); alive = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1u;
                    if (!mbar_wait(&full[s], ph)) { report(kDevErrFullWait, it); alive = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes);
                    const uint64_t adesc = umma_desc_sw128(a_addr);
                    const uint64_t bdesc = umma_desc_sw128(a_addr + kABytes);
#pragma unroll
                    for (int k = 0; k < C::kBlockK / C::kUmmaK; ++k) {
                        // +32 bytes per instruction inside the 128-byte swizzle row: +2 in the address field
                        if (MODE == kI8)
                            tcgen05_mma_i8(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        else
                            tcgen05_mma_f16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tcgen05_commit(&empty[s]);
                }
                if (alive) tcgen05_commit(&tmem_full[buf]);
            }
        }
    } else if (warp < kDequantWarp0) {
        // ------------------------------- epilogue -----------------------------------
        const int quarter = warp & 3;
        uint32_t tcount = 0;
        bool alive = true;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.y) & 15) == 0) && ((p.ldy & 3) == 0);
        for (int64_t tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ++tcount) {
            const int64_t m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const uint32_t buf = tcount & 1u, aph = (tcount >> 1) & 1u;
            if (!mbar_wait(&tmem_full[buf], aph)) { report(kDevErrMmaWait, 0x800000u | tcount); alive = false; break; }
            tcgen05_fence_after();
            const int64_t m = m0 + quarter * 32 + lane;
            float sxm = 1.0f;
            if (MODE == kI8 && m < p.M) sxm = p.sx[m];
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + buf * BN + c * 32 + (static_cast<uint32_t>(quarter * 32) << 16), v);
                tmem_ld_wait();
                const int64_t nb = n0 + c * 32;
                if (m < p.M && nb < p.N) {
                    float o[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int64_t n = nb + j;
                        if (MODE == kI8) {
                            const float sw = (n < p.N) ? (p.sw_per_row ? p.sw[n] : p.sw[0]) : 0.0f;
                            o[j] = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int32_t>(v[j])), sxm), sw);
                        } else {
                            o[j] = __uint_as_float(v[j]);
                        }
                        if (p.bias && n < p.N) o[j] = __fadd_rn(o[j], p.bias[n]);
                    }
                    float* dst = p.y + m * p.ldy + nb;
                    if (vec_ok && nb + 32 <= p.N) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            reinterpret_cast<float4*>(dst)[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (nb + j < p.N) dst[j] = o[j];
                    }
                    if (MODE == kI8 && p.acc_out) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (nb + j < p.N) p.acc_out[m * p.N + nb + j] = static_cast<int32_t>(v[j]);
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        }
    } else if (MODE == kBF16) {
        // ------------------------------- dequant ------------------------------------
        // thread r owns row r of the 256-row weight tile: 32 packed bytes in, 128 bytes of bf16 out
        const int r = (threadIdx.x - kDequantWarp0 * 32) % (kDequantWarps * 32);
        const uint32_t my_group = (threadIdx.x - kDequantWarp0 * 32) / (kDequantWarps * 32);
        const int64_t sgroups = p.K / 32;
        uint32_t it = 0;
        bool alive = true;
        for (int64_t tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
            const int64_t n = (tile / m_tiles) * BN + r;
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                if ((it % kDequantGroups) != my_group) continue;
                const int s = it % C::kStages;
                const uint32_t ph = (it / C::kStages) & 1u;
                float2 sc = make_float2(0.0f, 0.0f);
                if (n < p.N) sc = *reinterpret_cast<const float2*>(p.wscales + n * sgroups + 2 * kb);
                if (!mbar_wait(&raw_full[s], ph)) { report(kDevErrFullWait, 0x800000u | it); alive = false; break; }
                if (!mbar_wait(&empty[s], ph ^ 1u)) { report(kDevErrEmptyWait, 0x400000u | it); alive = false; break; }
                uint8_t* st = smem + s * C::kStageBytes;
                const uint4* raw = reinterpret_cast<const uint4*>(st + kABytes + kBBytes + r * 32);
                const uint4 w0 = raw[0], w1 = raw[1];
                const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                const __nv_bfloat16 s0 = __float2bfloat16_rn(sc.x), s1 = __float2bfloat16_rn(sc.y);
                const uint32_t s0x2 = static_cast<uint32_t>(__bfloat16_as_ushort(s0)) * 0x00010001u;
                const uint32_t s1x2 = static_cast<uint32_t>(__bfloat16_as_ushort(s1)) * 0x00010001u;
                uint8_t* brow = st + kABytes + r * 128;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const uint32_t sx2 = (w < 4) ? s0x2 : s1x2;
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t v = ((words[w] >> (4 * j)) & 0x000F000Fu) ^ 0x43084308u;  // 136 + code
                        uint32_t c;
                        asm("sub.bf16x2 %0, %1, %2;" : "=r"(c) : "r"(v), "r"(0x43084308u));
                        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(o[j]) : "r"(c), "r"(sx2));
                    }
                    // chunk w of the row goes to chunk (w ^ (r & 7)): the 128-byte swizzle the MMA expects
                    *reinterpret_cast<uint4*>(brow + ((w ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full[s]);
                    mbar_arrive(&raw_empty[s]);
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == kEpilogueWarp0) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// x fp32 [M,K] -> bf16 [M,K]; inside every aligned group of 8 the order is k+{0,4,1,5,2,6,3,7},
// the order in which the dequant warps emit the 8 nibbles of a packed word.
__global__ void __launch_bounds__(256) convert_x_bf16_kernel(const float* __restrict__ x, uint4* __restrict__ out,
                                                             int64_t chunks) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
    for (; i < chunks; i += stride) {
        const float4 a = reinterpret_cast<const float4*>(x)[2 * i];
        const float4 b = reinterpret_cast<const float4*>(x)[2 * i + 1];
        auto pk = [](float lo, float hi) {
            return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
                   (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
        };
        out[i] = make_uint4(pk(a.x, b.x), pk(a.y, b.y), pk(a.z, b.z), pk(a.w, b.w));
    }
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <int MODE>
int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, cudaStream_t stream) {
    using C = Cfg<MODE>;
    const int64_t tiles = ceil_div(p.M, BM) * ceil_div(p.N, BN);
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    static SmemOptIn optin;   // one per MODE instantiation
    SGQ_CUDA_TRY(optin.ensure(linear_tc_kernel<MODE>, C::kSmemBytes));
    linear_tc_kernel<MODE><<<grid, C::kThreads, C::kSmemBytes, stream>>>(ma, mb, p);
    SGQ_LAUNCH_CHECK("linear_tc_kernel");
    return SGQ_OK;
}

}  // namespace

bool tc_bf16_supported(int bits, int64_t M, int64_t K, int64_t N, int layout, int64_t group) {
    return bits == 4 && layout == SGQ_LAYOUT_NK && group == 32 && M >= 1 && N >= 1 && K >= 64 && (K % 64) == 0 &&
           M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31);
}

size_t tc_bf16_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout) {
    (void)bits; (void)N; (void)layout;
    return round_up(static_cast<size_t>(M) * static_cast<size_t>(K) * 2, 256);
}

int launch_linear_tc_bf16(const LinearArgs& a) {
    if (!tc_bf16_supported(a.bits, a.M, a.K, a.N, a.layout, a.group)) {
        set_error("bf16 tensor-core path needs INT4 g=32 weights stored [N,K] and K%%64==0");
        return SGQ_ERR_UNSUPPORTED;
    }
    if (!aligned(a.x, 16) || !aligned(a.wq, 16) || !aligned(a.scales, 8)) {
        set_error("bf16 tensor-core path needs 16-byte aligned x and packed weights, 8-byte aligned scales");
        return SGQ_ERR_ALIGNMENT;
    }
    const size_t need = tc_bf16_workspace_bytes(a.bits, a.M, a.K, a.N, a.layout);
    if (!a.workspace || a.workspace_bytes < need) {
        set_error("bf16 tensor-core path needs %zu workspace bytes, got %zu", need, a.workspace ? a.workspace_bytes : 0);
        return SGQ_ERR_WORKSPACE;
    }
    const int64_t chunks = a.M * a.K / 8;
    int64_t blocks = ceil_div(chunks, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    convert_x_bf16_kernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, a.stream>>>(
        a.x, static_cast<uint4*>(a.workspace), chunks);
    SGQ_LAUNCH_CHECK("convert_x_bf16_kernel");

    CUtensorMap ma, mb;
    if (!make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.workspace, static_cast<uint64_t>(a.K),
                            static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.K) * 2, 64, BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    if (!make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, static_cast<uint64_t>(a.K / 2),
                            static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 2), 32, BN, CU_TENSOR_MAP_SWIZZLE_NONE))
        return SGQ_ERR_CUDA;
    Params p{};
    p.bias = a.bias; p.y = a.y; p.ldy = a.ldy; p.M = a.M; p.N = a.N; p.K = a.K;
    p.wscales = a.scales;
    return launch_tc<kBF16>(ma, mb, p, a.stream);
}

bool tc_i8_supported(int64_t M, int64_t K, int64_t N) {
    return M >= 1 && N >= 1 && K >= 16 && (K % 16) == 0 && M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31);
}

size_t tc_i8_workspace_bytes(int64_t M, int64_t K, int64_t N) {
    (void)N;
    return round_up(static_cast<size_t>(M) * static_cast<size_t>(K), 256) + round_up(static_cast<size_t>(M) * 4, 256);
}

int launch_linear_w8a8(const LinearArgs& a, int8_t* xq_out, float* sx_out, int32_t* acc_out) {
    if (!tc_i8_supported(a.M, a.K, a.N)) {
        set_error("kind::i8 path needs K%%16==0");
        return SGQ_ERR_UNSUPPORTED;
    }
    int8_t* xq = xq_out;
    float* sx = sx_out;
    uint8_t* ws = static_cast<uint8_t*>(a.workspace);
    size_t off = 0;
    if (!xq) {
        const size_t need = round_up(static_cast<size_t>(a.M) * a.K, 256);
        if (!ws || a.workspace_bytes < off + need) { set_error("kind::i8 path: workspace too small"); return SGQ_ERR_WORKSPACE; }
        xq = reinterpret_cast<int8_t*>(ws + off);
        off += need;
    }
    if (!sx) {
        const size_t need = round_up(static_cast<size_t>(a.M) * 4, 256);
        if (!ws || a.workspace_bytes < off + need) { set_error("kind::i8 path: workspace too small"); return SGQ_ERR_WORKSPACE; }
        sx = reinterpret_cast<float*>(ws + off);
        off += need;
    }
    if (!aligned(xq, 16) || !aligned(a.wq, 16)) {
        set_error("kind::i8 path needs 16-byte aligned code buffers");
        return SGQ_ERR_ALIGNMENT;
    }
    // activations: the reference's per-row rule (src/quantization.cpp:42-75) applied to x
    int rc = launch_quantize_int8(a.x, a.M, a.K, SGQ_PER_ROW, xq, sx, a.stream);
    if (rc != SGQ_OK) return rc;
    CUtensorMap ma, mb;
    if (!make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, xq, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.M),
                            static_cast<uint64_t>(a.K), 128, BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    if (!make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N),
                            static_cast<uint64_t>(a.K), 128, BN, CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    Params p{};
    p.bias = a.bias; p.y = a.y; p.ldy = a.ldy; p.M = a.M; p.N = a.N; p.K = a.K;
    p.sx = sx; p.sw = a.scales; p.sw_per_row = (a.scheme == SGQ_PER_ROW) ? 1 : 0; p.acc_out = acc_out;
    return launch_tc<kI8>(ma, mb, p, a.stream);
}

}  // namespace sgq
