// Decode-shape forward (M <= 16) for INT4 g=32 weights stored [N,K]:  y = x * deq(W)^T + bias.
//
// HBM-bound: every packed byte and every scale is read exactly once.
//   algorithmic bytes = N*K/2 (nibbles) + N*K/32*4 (scales) + M*K*4 (x) + M*N*4 (y).
//
// One persistent CTA per SM: 8 or 16 consumer warps + 1 TMA producer warp + 1 reducer warp.
//   * The producer thread issues two TMA copies per stage: a 3-D box [8 steps][16 rows][128 B]
//     of packed weights (128-byte swizzle: the per-row word reads below are bank-conflict free)
//     and a box [8 steps][16 rows][8] of fp32 scales, into a ring of stages guarded by
//     full/empty mbarriers.  A step is 256 k of a 16-row tile.
//   * Integer inner product.  Each activation row is turned once per CTA into fixed point
//     relative to the power of two above its absmax (22 bits for M <= 2, 14 bits above: eight digit columns = one MMA then cover M = 4), split
//     into balanced base-256 digits (int8).  The 4-bit codes become bytes with two LOP3s per
//     eight codes ((w & 0x0F0F0F0F) ^ 0x08080808 = code + 8, exact), and a 32-k group of 16
//     weight rows times up to 8 digit columns is ONE mma.sync m16n8k32 (u8 x s8 -> s32, exact).
//     The +8 offset is cancelled exactly by starting the accumulator at -8 * sum(digits).
//   * The exact group sums are converted to fp32, multiplied by the group's fp32 scale and
//     accumulated in fp32:  y[m,n] = 2^-p_m * sum_j 256^j * sum_g scale[n,g] * S[n,g,m,j].
//   * A consumer warp that finishes its share of a tile drops its partial sums into a small
//     ring in shared memory and moves on; a dedicated reducer warp adds the partials in warp
//     order (fixed order -> run-to-run deterministic), recombines digits, adds bias, stores y.
//     Consumer warps never wait for one another, only for data and for ring slots.
//
// Error against the reference's single fp32 chain: the fixed-point step is 2^-22 (2^-14) of the
// row's power-of-two bound per activation, everything up to the group sums is exact, the rest
// is fp32 rounding: ~1e-6 (M <= 2) / ~4e-5 (M > 2) relative for Gaussian rows, inside 1e-3.
// Activations must be finite.
#include "sgq_common.cuh"
#include "gemv_prepare.cuh"
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

#ifdef SGQ_TIMELINE
// Debug build only: per-warp timestamps (globaltimer, ns) of the kernel's phases.
__device__ unsigned long long* g_timeline = nullptr;
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define SGQ_MARK(slot)                                                                                     \
    do {                                                                                                   \
        if (g_timeline && (threadIdx.x & 31) == 0)                                                         \
            g_timeline[(blockIdx.x * 32 + (threadIdx.x >> 5)) * 16 + (slot)] = now_ns();                   \
    } while (0)
extern "C" __attribute__((visibility("default"))) int sgq_debug_set_timeline(unsigned long long* buf) {
    return static_cast<int>(cudaMemcpyToSymbol(g_timeline, &buf, sizeof(buf)));
}
#else
#define SGQ_MARK(slot) do { } while (0)
#endif

namespace {

constexpr int kRows = 16;                  // rows of W per tile (mma M)
constexpr int kStepK = 256;                // k per step (one 128-byte swizzle row per weight row)
constexpr int kStepsPerStage = 8;
constexpr int kWStepBytes = kRows * 128;   // 2048
constexpr int kSStepBytes = kRows * 32;    // 16 rows x 8 fp32
constexpr int kStageW = kStepsPerStage * kWStepBytes;   // 16384
constexpr int kStageS = kStepsPerStage * kSStepBytes;   // 4096
constexpr int kStageBytes = kStageW + kStageS;          // 20480
constexpr int kMaxStages = 8;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kMaxM = 16;
constexpr int kPSlots = 2;                 // ring of per-tile partial-sum buffers

struct Smem {
    uint32_t stages_off, x_off, corr_off, partial_off, misc_off, total;   // from a 1024-byte aligned base
};

// groups = K/32; x digits: 256 B per (group, set); corrections: 32 B per (group, set)
__host__ __device__ inline Smem smem_layout(int nstages, int64_t K, int nsets, int nwarps) {
    Smem s;
    const uint32_t groups = static_cast<uint32_t>(K / 32);
    s.stages_off = 0;
    s.x_off = nstages * kStageBytes;
    s.corr_off = s.x_off + groups * 256u * nsets;
    s.partial_off = s.corr_off + groups * 32u * nsets;
    s.misc_off = s.partial_off + kPSlots * nwarps * (512u * nsets + 16u);   // padded per-warp partial sums
    s.total = s.misc_off + (2u * kMaxStages + 2u * kPSlots + 1u) * 8u + kMaxM * 8u + 16u;
    return s;
}

__device__ __forceinline__ void report(uint32_t code, uint32_t detail) {
    atomicCAS(&g_status_gemv, 0u, (code << 24) | (detail & 0xFFFFFFu));
}

// D(16x8,s32) = A(16x32,u8,row) * B(32x8,s8,col) + C
__device__ __forceinline__ void mma_u8s8_16832(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                               int c0, int c1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c0), "r"(c1));
}

// Activation planes for batches too large to convert inside every CTA: one CTA per batch row,
// written once to global scratch in exactly the shared-memory layout the main kernel uses:
//   [digit planes: groups*nsets*256 B][corrections: groups*nsets*32 B][inv_p: 16 fp32]
constexpr int kPrepThreads = 512;
constexpr int kPrepMaxChunks = 8;   // per thread: K <= 8 * 512 * 8 = 32768
__global__ void __launch_bounds__(kPrepThreads) gemv_prepare_x_kernel(const float* __restrict__ x, int M, int64_t K,
                                                                     int ndigits, int nsets, uint8_t* __restrict__ planes) {
    __shared__ float red[kPrepThreads / 32];
    pdl_launch_dependents();
    pdl_wait();                                        // x comes from the kernel before this one
    const int m = blockIdx.x, lane = threadIdx.x & 31;
    const int chunks = static_cast<int>(K / 8);
    const size_t groups = static_cast<size_t>(K / 32);
    uint8_t* xs = planes;
    uint8_t* corr = planes + groups * nsets * 256;
    float* inv_p = reinterpret_cast<float*>(corr + groups * nsets * 32);
    float v[kPrepMaxChunks][8];
    float mx = 0.0f;
#pragma unroll
    for (int r = 0; r < kPrepMaxChunks; ++r) {
        const int c = threadIdx.x + r * kPrepThreads;
        if (c < chunks) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(x + static_cast<int64_t>(m) * K) + 2 * c);
            const float4 b = __ldg(reinterpret_cast<const float4*>(x + static_cast<int64_t>(m) * K) + 2 * c + 1);
            v[r][0] = a.x; v[r][1] = a.y; v[r][2] = a.z; v[r][3] = a.w; v[r][4] = b.x; v[r][5] = b.y; v[r][6] = b.z; v[r][7] = b.w;
            mx = fmaxf(mx, absmax8(v[r]));
        }
    }
    mx = warp_max(mx);
    if (lane == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    float all = red[lane < kPrepThreads / 32 ? lane : 0];
    all = warp_max(all);
    float P, invP;
    row_scale(__float_as_uint(all), ndigits == 3 ? 22 : 14, &P, &invP);
    if (threadIdx.x == 0) inv_p[m] = invP;
#pragma unroll
    for (int r = 0; r < kPrepMaxChunks; ++r) {
        const int c = threadIdx.x + r * kPrepThreads;
        if (c < chunks) digits_item(v[r], P, m, c, ndigits, nsets, xs, corr);   // chunks % 32 == 0: whole warps
    }
}

// Consumer organisation (template parameter WPB):
//   1: 8 warps, one per 256-k step, every warp works on every stage (the compact two-CTAs-per-SM form);
//   2: 16 warps, two per step (half a step each), every warp works on every stage;
//   3: 16 warps in two sets of 8, one warp per step, the sets take ALTERNATE stages — two stages are
//      in work at any time, so the latency bubbles of one set (barrier waits, the hand-off to the
//      reducer at the end of a tile) are covered by the other.
__host__ __device__ constexpr int consumer_warps(int wpb) { return wpb == 1 ? 8 : 16; }

// NSETS: sets of 8 digit columns; WPB: see above;
// PRE: the activation planes were prepared by gemv_prepare_x_kernel and are copied in by TMA.
template <int NSETS, int WPB, bool PRE>
__global__ void __launch_bounds__((consumer_warps(WPB) + 2) * 32, WPB == 1 ? 2 : 1)
gemv_int4_nk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                    const float* __restrict__ x, const uint8_t* __restrict__ planes, const float* __restrict__ bias,
                    float* __restrict__ y, int M, int ndigits, int64_t K, int64_t N, int64_t ldy, int nstages, int early_weights,
                    const __grid_constant__ PeerOut peers) {
    constexpr int kWarps = consumer_warps(WPB);
    constexpr int kConsumerThreads = kWarps * 32;
    constexpr int kWarpsPerStep = WPB == 2 ? 2 : 1;
    constexpr int kGroupsPerWarp = 8 / kWarpsPerStep;
    constexpr int kStageSets = WPB == 3 ? 2 : 1;       // sets of warps that take alternate stages

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const Smem L = smem_layout(nstages, K, NSETS, kWarps);
    uint8_t* stages = smem + L.stages_off;
    uint8_t* xs = smem + L.x_off;
    uint8_t* corr = smem + L.corr_off;
    float* partial = reinterpret_cast<float*>(smem + L.partial_off);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.misc_off);
    uint64_t* empty = full + kMaxStages;
    uint64_t* pfull = empty + kMaxStages;      // [kPSlots] every consumer warp has left its partial sums
    uint64_t* pempty = pfull + kPSlots;        // [kPSlots] the reducer is done with the slot
    uint64_t* xfull = pempty + kPSlots;        // [1] prepared activation planes have landed (PRE)
    uint32_t* rowmax_bits = reinterpret_cast<uint32_t*>(xfull + 1);            // [16]
    float* inv_p = reinterpret_cast<float*>(rowmax_bits + kMaxM);              // [16]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t ntiles = (N + kRows - 1) / kRows;
    const int spt = static_cast<int>(K / kStepK);   // steps per tile (K % 256 == 0)

    SGQ_MARK(0);
    pdl_launch_dependents();            // the next kernel may begin its prologue; it waits for this grid before touching data
    if (threadIdx.x == kWarps * 32) {   // the producer thread: start fetching both descriptors now
        tma_prefetch_descriptor(&map_w);
        tma_prefetch_descriptor(&map_s);
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < nstages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kWarps / kStageSets);
        }
        for (int i = 0; i < kPSlots; ++i) {
            mbar_init(&pfull[i], kWarps);
            mbar_init(&pempty[i], 1);
        }
        mbar_init(xfull, 1);
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (threadIdx.x < kMaxM) rowmax_bits[threadIdx.x] = 0;
    __syncthreads();
    // Everything above touches no global data.  From here on every thread except the producer
    // first waits for the kernels this launch depends on (they wrote x / the planes, and may still
    // be reading y); the producer decides for itself below, because weights are not their output.
    if (warp != kWarps) pdl_wait();
    SGQ_MARK(12);
    // The first kPre items of every consumer thread are requested before anything else, so that
    // their global-memory latency overlaps the producer's first TMA issues.
    constexpr int kPre = PRE ? 1 : 4;
    const int chunks = static_cast<int>(K / 8);   // 8-float chunks per activation row
    const int items = chunks * M;
    float4 pre_a[kPre], pre_b[kPre];
#pragma unroll
    for (int r = 0; r < kPre; ++r) {
        const int it = threadIdx.x + r * kConsumerThreads;
        if (!PRE && warp < kWarps && it < items) {
            pre_a[r] = __ldg(reinterpret_cast<const float4*>(x) + 2 * static_cast<int64_t>(it));
            pre_b[r] = __ldg(reinterpret_cast<const float4*>(x) + 2 * static_cast<int64_t>(it) + 1);
        } else {
            pre_a[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            pre_b[r] = pre_a[r];
        }
    }

    if (warp == kWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            // Weights and scales are parameters, not the output of the kernel before this one: with
            // early_weights the first ring of stages is requested before the dependency wait, so the
            // weight stream overlaps the tail of that kernel.  The activation planes are its output
            // and are copied only after the wait.
            bool synced = false;
            auto dependency_sync = [&]() {
                if (synced) return;
                synced = true;
                pdl_wait();
                SGQ_MARK(4);
                if (PRE) {
                    fence_proxy_async_all();        // the planes were written through the generic proxy
                    // digit planes + corrections, contiguous in both places, in pieces of <= 32 KiB
                    const uint32_t bytes = L.partial_off - L.x_off;
                    mbar_arrive_expect_tx(xfull, bytes);
                    for (uint32_t off = 0; off < bytes; off += 32768u)
                        bulk_copy_g2s(xs + off, planes + off, (bytes - off < 32768u) ? bytes - off : 32768u, xfull);
                }
            };
            if (!early_weights) dependency_sync();
            uint32_t seq = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                for (int c0 = 0; c0 < spt; c0 += kStepsPerStage, ++seq) {
                    if (seq == static_cast<uint32_t>(nstages)) dependency_sync();   // the ring is full: nothing more to request early
                    const int st = seq % nstages;
                    const uint32_t ph = (seq / nstages) & 1u;
                    if (!mbar_wait(&empty[st], ph ^ 1u)) {
                        report(kDevErrEmptyWait, seq);
                        ok = false;
                        break;
                    }
                    // steps past K/256 are out of range in the third dimension: zero-filled, still counted
                    mbar_arrive_expect_tx(&full[st], kStageBytes);
                    uint8_t* sw = stages + st * kStageBytes;
                    tma_load_3d(sw, &map_w, &full[st], 0, static_cast<int32_t>(tile * kRows), c0);
                    tma_load_3d(sw + kStageW, &map_s, &full[st], 0, static_cast<int32_t>(tile * kRows), c0);
                    if (seq == 0) SGQ_MARK(1);
                    if (seq == 6) SGQ_MARK(2);
                }
            }
            dependency_sync();
            SGQ_MARK(3);
        }
        return;
    }

    constexpr int kPStride = 128 * NSETS + 4;   // floats per warp in a partial-sum slot (padded against bank conflicts)
    if (warp == kWarps + 1) {
        // ---------------- reducer ----------------
        // lane -> output pairs (tile row r, batch row m); per digit column the kWarps partial sums
        // are added in warp order, then digits are recombined: y = 2^-p * sum_j 256^j v_j + bias.
        uint32_t tcount = 0;
        const int pairs = kRows * M;
        for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
            const int slot = tcount % kPSlots;
            const uint32_t pph = (tcount / kPSlots) & 1u;
            if (!mbar_wait(&pfull[slot], pph)) {
                report(kDevErrFullWait, 0x800000u | tcount);
                break;
            }
            if (tcount < 6) SGQ_MARK(2 * tcount);
            float* pbuf = partial + slot * (kWarps * kPStride);
            // Step 1: add the warps' partial sums fragment-wise, in warp order (fixed order -> the same
            // bits every run): lane L owns the float4 every consumer lane L wrote, so these are
            // conflict-free 128-bit reads.  The sum goes back into warp 0's part of the slot.
#pragma unroll
            for (int s = 0; s < NSETS; ++s) {
                float4 sum = *reinterpret_cast<const float4*>(pbuf + (s * 32 + lane) * 4);
#pragma unroll
                for (int w = 1; w < kWarps; ++w) {
                    const float4 v = *reinterpret_cast<const float4*>(pbuf + w * kPStride + (s * 32 + lane) * 4);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                *reinterpret_cast<float4*>(pbuf + (s * 32 + lane) * 4) = sum;
            }
            __syncwarp();
            // Step 2: one value per (output, digit): recombine the digits, scale, add bias, store.
            for (int p = lane; p < pairs; p += 32) {
                const int r = p & 15, m = p >> 4;
                const int gg = r & 7, hi = r >> 3;
                float acc = 0.0f, weight = 1.0f;
                for (int j = 0; j < ndigits; ++j, weight *= 256.0f) {
                    const int col = m * ndigits + j, set = col >> 3, cc = col & 7;
                    const float v = pbuf[(set * 32 + gg * 4 + (cc >> 1)) * 4 + hi * 2 + (cc & 1)];
                    acc = __fmaf_rn(weight, v, acc);
                }
                const int64_t n = tile * kRows + r;
                if (n < N) {
                    float v = acc * (PRE ? __ldg(reinterpret_cast<const float*>(planes + (L.partial_off - L.x_off)) + m)
                                         : inv_p[m]);
                    if (bias) v += bias[n];
                    if (peers.n == 0) {
                        y[static_cast<int64_t>(m) * ldy + n] = v;
                    } else {
                        // fused all-gather: the slice goes into every GPU's full-width output (plain peer stores)
                        for (int r2 = 0; r2 < peers.n; ++r2) peers.p[r2][static_cast<int64_t>(m) * ldy + n] = v;
                    }
                }
            }
            __syncwarp();
            if (tcount < 6) SGQ_MARK(2 * tcount + 1);
            if (lane == 0) mbar_arrive(&pempty[slot]);
        }
        if (peers.n > 0 && peers.sig[0] != nullptr) {
            // Barrier fused into the tail: this CTA's slices are out; the last CTA of the launch to get
            // here tells every rank and waits for every rank, so the kernel ends when all outputs are whole.
            __syncwarp();
            __threadfence_system();
            unsigned int* counter = reinterpret_cast<unsigned int*>(peers.state + 1);
            unsigned int ticket = 0;
            if (lane == 0) ticket = atomicAdd(counter, 1u);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            if (ticket == gridDim.x - 1) {
                if (lane == 0) *counter = 0;          // re-armed for the next launch, which counts only at its own end
                int late = 0;
                if (!peer_signal_and_wait(peers.sig, peers.rank, peers.n, peers.state, lane, &late) && lane == 0)
                    report(kDevErrPeerWait, 0x10000u);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    bool alive = true;   // false after a wait ran out: skip the math but keep every barrier balanced
    if (PRE) {
        if (!mbar_wait(xfull, 0)) {
            report(kDevErrFullWait, 0x400000u);
            alive = false;
        }
    } else {
        // Activations -> int8 digits, inside the CTA (small batches: every item was requested at the top).
        auto unpack = [](const float4& a, const float4& b, float (&v)[8]) {
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        };
        auto load_item = [&](int it, float (&v)[8]) {
            unpack(__ldg(reinterpret_cast<const float4*>(x) + 2 * static_cast<int64_t>(it)),
                   __ldg(reinterpret_cast<const float4*>(x) + 2 * static_cast<int64_t>(it) + 1), v);
        };
        // pass 1: absmax per row (the bit pattern of |x| orders like the value).  items % 32 == 0 and
        // chunks % 4 == 0, so whole warps are in or out and 4 neighbouring lanes share a row.
        auto absmax_item = [&](int it, const float (&v)[8]) {
            float mx = absmax8(v);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            if ((lane & 3) == 0) atomicMax(&rowmax_bits[it / chunks], __float_as_uint(mx));
        };
#pragma unroll
        for (int r = 0; r < kPre; ++r) {
            const int it = threadIdx.x + r * kConsumerThreads;
            if (it < items) {
                float v[8];
                unpack(pre_a[r], pre_b[r], v);
                absmax_item(it, v);
            }
        }
        for (int it = threadIdx.x + kPre * kConsumerThreads; it < items; it += kConsumerThreads) {
            float v[8];
            load_item(it, v);
            absmax_item(it, v);
        }
        // Columns >= M*ndigits of the digit planes stay uninitialised: they only feed accumulator
        // columns that nobody reads (integer MMA: no NaN can spread).
        named_barrier_sync(1, kConsumerThreads);
        const int frac_bits = (ndigits == 3) ? 22 : 14;
        // pass 2: fixed point + digits.  Four neighbouring lanes own the four t-chunks of one group.
        auto convert_item = [&](int it, const float (&v)[8]) {
            const int m = it / chunks, c = it - m * chunks;
            float P, invP;
            row_scale(rowmax_bits[m], frac_bits, &P, &invP);
            if (c == 0) inv_p[m] = invP;
            digits_item(v, P, m, c, ndigits, NSETS, xs, corr);
        };
#pragma unroll
        for (int r = 0; r < kPre; ++r) {
            const int it = threadIdx.x + r * kConsumerThreads;
            if (it < items) {
                float v[8];
                unpack(pre_a[r], pre_b[r], v);
                convert_item(it, v);
            }
        }
        for (int it = threadIdx.x + kPre * kConsumerThreads; it < items; it += kConsumerThreads) {
            float v[8];
            load_item(it, v);
            convert_item(it, v);
        }
    }
    SGQ_MARK(1);
    named_barrier_sync(1, kConsumerThreads);
    SGQ_MARK(2);

    const int g = lane >> 2, t = lane & 3;
    const int step_in_stage = (warp / kWarpsPerStep) & 7;          // which 256-k step of a stage this warp works on
    const int g0 = (warp % kWarpsPerStep) * kGroupsPerWarp;        // first of its groups inside the step
    const uint32_t my_set = (kStageSets == 2) ? static_cast<uint32_t>(warp >> 3) : 0u;
    // byte offset of this lane's word inside a step box, for each of its groups (swizzle: chunk ^ row)
    uint32_t woff[kGroupsPerWarp];
#pragma unroll
    for (int i = 0; i < kGroupsPerWarp; ++i) woff[i] = g * 128 + (((g0 + i) ^ g) << 4) + t * 4;

    uint32_t seq = 0, tcount = 0;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
        float total[NSETS][4];
#pragma unroll
        for (int s = 0; s < NSETS; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) total[s][i] = 0.0f;

        for (int c0 = 0; c0 < spt; c0 += kStepsPerStage, ++seq) {
            if (kStageSets == 2 && (seq & 1u) != my_set) continue;       // the other set's stage
            const int st = seq % nstages;
            const uint32_t ph = (seq / nstages) & 1u;
            if (alive && !mbar_wait(&full[st], ph)) {
                report(kDevErrFullWait, seq);
                alive = false;
            }
            if (seq < 5) SGQ_MARK(3 + 2 * seq);
            const int step = c0 + step_in_stage;
            if (alive && step < spt) {
                const uint8_t* wbox = stages + st * kStageBytes + step_in_stage * kWStepBytes;
                const uint8_t* sbox = stages + st * kStageBytes + kStageW + step_in_stage * kSStepBytes;
                float sc_lo[kGroupsPerWarp], sc_hi[kGroupsPerWarp];   // scales of rows g and g+8
#pragma unroll
                for (int h = 0; h < kGroupsPerWarp / 4; ++h) {
                    const float4 a = *reinterpret_cast<const float4*>(sbox + g * 32 + (g0 / 4 + h) * 16);
                    const float4 b = *reinterpret_cast<const float4*>(sbox + (g + 8) * 32 + (g0 / 4 + h) * 16);
                    sc_lo[4 * h + 0] = a.x; sc_lo[4 * h + 1] = a.y; sc_lo[4 * h + 2] = a.z; sc_lo[4 * h + 3] = a.w;
                    sc_hi[4 * h + 0] = b.x; sc_hi[4 * h + 1] = b.y; sc_hi[4 * h + 2] = b.z; sc_hi[4 * h + 3] = b.w;
                }
                const size_t group0 = static_cast<size_t>(step) * 8 + g0;
                const uint8_t* xg = xs + group0 * (256 * NSETS) + lane * 8;
                const uint8_t* cg = corr + group0 * (32 * NSETS) + t * 8;
                uint32_t wl[kGroupsPerWarp], wh[kGroupsPerWarp];
#pragma unroll
                for (int i = 0; i < kGroupsPerWarp; ++i) {
                    wl[i] = *reinterpret_cast<const uint32_t*>(wbox + woff[i]);
                    wh[i] = *reinterpret_cast<const uint32_t*>(wbox + 1024 + woff[i]);
                }
#pragma unroll
                for (int i = 0; i < kGroupsPerWarp; ++i) {
                    const uint32_t w_lo = wl[i], w_hi = wh[i];
                    uint32_t a[4];
                    a[0] = (w_lo & 0x0F0F0F0Fu) ^ 0x08080808u;          // row g,   k = 8t + {0,2,4,6}: code + 8
                    a[1] = (w_hi & 0x0F0F0F0Fu) ^ 0x08080808u;          // row g+8
                    a[2] = ((w_lo >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;   // row g,   k = 8t + {1,3,5,7}
                    a[3] = ((w_hi >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;   // row g+8
#pragma unroll
                    for (int s = 0; s < NSETS; ++s) {
                        const uint2 xb = *reinterpret_cast<const uint2*>(xg + i * (256 * NSETS) + s * 256);
                        const int2 cc = *reinterpret_cast<const int2*>(cg + i * (32 * NSETS) + s * 32);
                        int d[4];
                        mma_u8s8_16832(d, a, xb.x, xb.y, cc.x, cc.y);
                        // d holds 12582912.0f + (exact group sum) as fp32 bits: one subtraction instead of a conversion
                        total[s][0] = __fmaf_rn(sc_lo[i], __fsub_rn(__int_as_float(d[0]), kGroupSumBiasF), total[s][0]);
                        total[s][1] = __fmaf_rn(sc_lo[i], __fsub_rn(__int_as_float(d[1]), kGroupSumBiasF), total[s][1]);
                        total[s][2] = __fmaf_rn(sc_hi[i], __fsub_rn(__int_as_float(d[2]), kGroupSumBiasF), total[s][2]);
                        total[s][3] = __fmaf_rn(sc_hi[i], __fsub_rn(__int_as_float(d[3]), kGroupSumBiasF), total[s][3]);
                    }
                }
            }
            // everything loaded from the stage has been consumed once the accumulators are final
            uint32_t fold = 0;
#pragma unroll
            for (int s = 0; s < NSETS; ++s) fold ^= __float_as_uint(total[s][0]) ^ __float_as_uint(total[s][2]);
            const uint32_t landed = loads_landed(fold);
            if (seq < 5) SGQ_MARK(4 + 2 * seq);
            if (lane == 0) mbar_arrive_after(&empty[st], landed);
        }
        if (tile == blockIdx.x) SGQ_MARK(13);

        // ---- hand the tile's partial sums to the reducer warp ----
        {
            const int slot = tcount % kPSlots;
            const uint32_t pph = (tcount / kPSlots) & 1u;
            if (alive && !mbar_wait(&pempty[slot], pph ^ 1u)) {
                report(kDevErrEmptyWait, 0x800000u | tcount);
                alive = false;
            }
            float* pbuf = partial + slot * (kWarps * kPStride) + warp * kPStride;
#pragma unroll
            for (int s = 0; s < NSETS; ++s)
                *reinterpret_cast<float4*>(pbuf + (s * 32 + lane) * 4) =
                    make_float4(total[s][0], total[s][1], total[s][2], total[s][3]);
            __syncwarp();
            if (lane == 0) mbar_arrive(&pfull[slot]);
        }
        if (tile == blockIdx.x) SGQ_MARK(14);
    }
    SGQ_MARK(15);
}

struct Plan {
    int ndigits, nsets, wpb, nstages;
    bool pre;          // activation planes prepared by a separate launch into the workspace
    uint32_t smem;
    size_t planes_bytes;
};

// In-CTA conversion is used while every consumer thread can hold all its items in registers
// (4 items of 8 activations per thread); larger batches are converted once by a pre-kernel.
//
// compact: a CTA that leaves room for a second one on the same SM (half the shared memory, 10
// warps).  With overlapped launches the CTA of the NEXT kernel then sits beside the one still
// running and streams its first weight stages in the meantime, so the pipeline fill, the launch
// latency and the tail of consecutive decode forwards hide behind each other.
constexpr int kCompactSmem = 112 * 1024;
bool make_plan(int64_t M, int64_t K, bool have_workspace, Plan* p, bool compact = false) {
    p->ndigits = prepared_layout(M, K).ndigits;
    p->nsets = static_cast<int>((M * p->ndigits + 7) / 8);
    p->planes_bytes = static_cast<size_t>(K / 32) * p->nsets * 288 + kMaxM * 4;
    const int limit = compact ? kCompactSmem : kSmemLimit;
    // two warps per step while at least 3 stages still fit, else one (smaller partial-sum buffers)
    for (int wpb = compact ? 1 : 3; wpb >= 1; --wpb) {
        for (int st = kMaxStages; st >= (wpb == 3 ? 4 : (wpb == 2 ? 3 : 2)); --st) {
            const Smem L = smem_layout(st, K, p->nsets, consumer_warps(wpb));
            if (L.total + 1024 <= static_cast<uint32_t>(limit)) {
                p->wpb = wpb;
                p->nstages = st;
                p->smem = L.total + 1024;
                p->pre = have_workspace && (M * (K / 8) > 4 * consumer_warps(wpb) * 32) && K <= 8LL * kPrepMaxChunks * kPrepThreads;
                return true;
            }
        }
    }
    return false;
}

// Rows of the batch one launch can take: the largest m <= M whose activation planes fit in shared
// memory next to the pipeline stages (0: not even one row fits).  Larger batches run as several
// launches over row blocks; each streams the weights again, which is still far better than the
// any-shape kernel.
int64_t rows_per_launch(int64_t M, int64_t K) {
    Plan p;
    for (int64_t m = M; m >= 1; --m)
        if (make_plan(m, K, false, &p)) return m;
    return 0;
}

template <int NSETS, int WPB, bool PRE>
int launch_variant(const LinearArgs& a, const Plan& p, const CUtensorMap& map_w, const CUtensorMap& map_s, int grid,
                   bool planes_ready) {
    static SmemOptIn optin;
    auto kernel = gemv_int4_nk_kernel<NSETS, WPB, PRE>;
    SGQ_CUDA_TRY(optin.ensure(kernel, kSmemLimit));
    const uint8_t* planes = static_cast<const uint8_t*>(a.workspace);
    const bool overlap = stream_overlap_enabled();
    if (PRE && !planes_ready) {
        SGQ_CUDA_TRY(launch_kernel(gemv_prepare_x_kernel, dim3(static_cast<unsigned>(a.M)), dim3(kPrepThreads), 0, a.stream, overlap,
                                   a.x, static_cast<int>(a.M), a.K, p.ndigits, p.nsets, static_cast<uint8_t*>(a.workspace)));
    }
    SGQ_CUDA_TRY(launch_kernel(kernel, dim3(static_cast<unsigned>(grid)), dim3((consumer_warps(WPB) + 2) * 32), p.smem, a.stream,
                               overlap, map_w, map_s, a.x, planes, a.bias, a.y, static_cast<int>(a.M), p.ndigits, a.K, a.N, a.ldy,
                               p.nstages, overlap ? 1 : 0, a.peers));
    return SGQ_OK;
}

template <int NSETS>
int launch_nsets(const LinearArgs& a, const Plan& p, const CUtensorMap& map_w, const CUtensorMap& map_s, int grid,
                 bool planes_ready) {
    if (p.pre)
        return p.wpb == 3 ? launch_variant<NSETS, 3, true>(a, p, map_w, map_s, grid, planes_ready)
             : p.wpb == 2 ? launch_variant<NSETS, 2, true>(a, p, map_w, map_s, grid, planes_ready)
                          : launch_variant<NSETS, 1, true>(a, p, map_w, map_s, grid, planes_ready);
    return p.wpb == 3 ? launch_variant<NSETS, 3, false>(a, p, map_w, map_s, grid, false)
         : p.wpb == 2 ? launch_variant<NSETS, 2, false>(a, p, map_w, map_s, grid, false)
                      : launch_variant<NSETS, 1, false>(a, p, map_w, map_s, grid, false);
}

}  // namespace

bool gemv_supported(const LinearArgs& a) {
    Plan p;
    return a.bits == 4 && a.layout == SGQ_LAYOUT_NK && a.group == 32 && a.M >= 1 && a.M <= kMaxM && a.K >= 256 &&
           (a.K % 256) == 0 && a.N >= 1 && a.N < (1LL << 31) && a.K < (1LL << 24) && aligned(a.wq, 16) &&
           aligned(a.scales, 16) && aligned(a.x, 16) && rows_per_launch(a.M, a.K) >= 1;
}

// Scratch for the prepared activation planes (batches converted by the pre-kernel); 0 when the
// conversion happens inside the CTAs.
size_t gemv_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout) {
    (void)N;
    Plan p;
    if (bits != 4 || layout != SGQ_LAYOUT_NK || M < 1 || M > kMaxM || K < 256 || (K % 256) != 0) return 0;
    const int64_t rows = rows_per_launch(M, K);
    if (rows < 1) return 0;
    if (rows < M) M = rows;                          // the row blocks of a split batch reuse one scratch
    if (!make_plan(M, K, true, &p)) return 0;
    Plan c;
    const bool compact_pre = make_plan(M, K, true, &c, true) && c.pre;    // what an overlapped launch would want
    if (!p.pre && !compact_pre) return 0;
    return (p.planes_bytes + 255) / 256 * 256;
}

namespace {
int launch_gemv_impl(const LinearArgs& a, bool planes_ready);
}

int launch_linear_gemv(const LinearArgs& a) { return launch_gemv_impl(a, false); }

// a.workspace holds activations already converted to the prepared format (a.x is not read).
int launch_linear_gemv_prepared(const LinearArgs& a) { return launch_gemv_impl(a, true); }

size_t gemv_prepared_bytes(int64_t M, int64_t K) {
    Plan p;
    if (M < 1 || M > kMaxM || K < 256 || (K % 256) != 0 || K >= (1LL << 24) || !make_plan(M, K, true, &p)) return 0;
    return (p.planes_bytes + 255) / 256 * 256;
}

int launch_prepare_x(const float* x, int64_t M, int64_t K, void* prepared, cudaStream_t s) {
    const PreparedLayout L = prepared_layout(M, K);
    if (K > 8LL * kPrepMaxChunks * kPrepThreads) {
        set_error("K too large for the conversion kernel");
        return SGQ_ERR_UNSUPPORTED;
    }
    SGQ_CUDA_TRY(launch_kernel(gemv_prepare_x_kernel, dim3(static_cast<unsigned>(M)), dim3(kPrepThreads), 0, s,
                               stream_overlap_enabled(), x, static_cast<int>(M), K, L.ndigits, L.nsets,
                               static_cast<uint8_t*>(prepared)));
    return SGQ_OK;
}

namespace {
int launch_gemv_impl(const LinearArgs& a, bool planes_ready) {
    Plan p;
    if (!planes_ready && a.bits == 4 && a.M >= 1 && a.M <= kMaxM && a.K >= 256 && (a.K % 256) == 0) {
        const int64_t rows = rows_per_launch(a.M, a.K);
        if (rows >= 1 && rows < a.M) {               // planes of the whole batch do not fit: row blocks
            for (int64_t m0 = 0; m0 < a.M; m0 += rows) {
                LinearArgs sub = a;
                sub.M = (a.M - m0 < rows) ? a.M - m0 : rows;
                sub.x = a.x + m0 * a.K;
                sub.y = a.y + m0 * a.ldy;
                for (int r = 0; r < sub.peers.n; ++r) sub.peers.p[r] = a.peers.p[r] + m0 * a.ldy;
                if (m0 + sub.M < a.M) sub.peers.sig[0] = nullptr;     // a fused barrier belongs to the last block only
                const int rc = launch_gemv_impl(sub, false);
                if (rc != SGQ_OK) return rc;
            }
            return SGQ_OK;
        }
    }
    const size_t want = planes_ready ? gemv_prepared_bytes(a.M, a.K) : gemv_workspace_bytes(a.bits, a.M, a.K, a.N, a.layout);
    const bool have_ws = a.workspace != nullptr && want > 0 && a.workspace_bytes >= want;
    LinearArgs probe = a;
    if (planes_ready) probe.x = static_cast<const float*>(a.workspace);      // x is not read: only its alignment rule is waived
    const bool compact = stream_overlap_compact();
    if (!gemv_supported(probe) || !((compact && make_plan(a.M, a.K, have_ws, &p, true)) || make_plan(a.M, a.K, have_ws, &p)) ||
        (planes_ready && !have_ws)) {
        set_error("decode path needs INT4 g=32, layout NK, M<=16, K%%256==0, x digits fitting in shared memory, "
                  "16-byte aligned x/packed/scales");
        return SGQ_ERR_UNSUPPORTED;
    }
    if (planes_ready) p.pre = true;
    // packed weights as (128 B, N rows, K/256 steps); scales as (8 fp32, N rows, K/256 steps)
    CUtensorMap map_w, map_s;
    const uint64_t steps = static_cast<uint64_t>(a.K / kStepK);
    {
        const uint64_t dims[3] = {128, static_cast<uint64_t>(a.N), steps};
        const uint64_t strides[2] = {static_cast<uint64_t>(a.K / 2), 128};
        const uint32_t box[3] = {128, kRows, kStepsPerStage};
        if (!make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return SGQ_ERR_CUDA;
    }
    {
        const uint64_t dims[3] = {8, static_cast<uint64_t>(a.N), steps};
        const uint64_t strides[2] = {static_cast<uint64_t>(a.K / 32) * 4, 32};
        const uint32_t box[3] = {8, kRows, kStepsPerStage};
        if (!make_tensor_map(&map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.scales, 3, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_NONE))
            return SGQ_ERR_CUDA;
    }
    const int64_t ntiles = ceil_div(a.N, kRows);
    const int grid = static_cast<int>(ntiles < sm_count() ? ntiles : sm_count());
    switch (p.nsets) {
        case 1: return launch_nsets<1>(a, p, map_w, map_s, grid, planes_ready);
        case 2: return launch_nsets<2>(a, p, map_w, map_s, grid, planes_ready);
        case 3: return launch_nsets<3>(a, p, map_w, map_s, grid, planes_ready);
        default: return launch_nsets<4>(a, p, map_w, map_s, grid, planes_ready);
    }
}
}  // namespace

// ---- entry point without any allocation ---------------------------------------------------
// Some callers of the decode forward cannot obtain device memory at call time: code running
// under a fixed memory budget that was handed out at start-up, a plugin loaded into a host that
// owns every allocation, or a serving loop that must not touch the allocator (and its locks)
// between tokens.  For them the activation planes live in this file-scope array instead of a
// caller workspace.  Every GPU that loads the library reserves these bytes until the process
// exits.  The size bounds the batches this entry point accepts: (K/32) * ceil(M*digits/8) * 288
// + 64 bytes, e.g. K = 8192 with M = 16.
constexpr size_t kStaticPlanesBytes = 320 * 1024;
static __device__ __align__(256) unsigned char g_static_planes[kStaticPlanesBytes];

namespace {
// Device address of g_static_planes, looked up once per device.  In host code the array's name
// is only a handle for the runtime, not a device pointer, so kernels must be given this address.
int static_planes_address(void** out) {
    static void* cached[64] = {};
    int dev = 0;
    SGQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        set_error("device ordinal %d out of range", dev);
        return SGQ_ERR_DEVICE;
    }
    void* p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        SGQ_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_planes));   // with `dev` current: this device's copy
        __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);
    }
    *out = p;
    return SGQ_OK;
}
}  // namespace

int launch_linear_gemv_static(LinearArgs a) {
    // the limit is stated for the whole batch, whether or not it then runs as several row blocks
    size_t need = gemv_workspace_bytes(a.bits, a.M, a.K, a.N, a.layout);
    if (a.M >= 1 && a.M <= kMaxM && a.K >= 256 && (a.K % 256) == 0 && rows_per_launch(a.M, a.K) < a.M) {
        const size_t whole = (prepared_layout(a.M, a.K).bytes + 255) / 256 * 256;
        if (whole > need) need = whole;
    }
    if (need > kStaticPlanesBytes) {
        set_error("this batch needs %zu bytes of activation scratch; the built-in scratch holds %zu "
                  "(use sgq_linear_int4 with a caller workspace)", need, kStaticPlanesBytes);
        return SGQ_ERR_WORKSPACE;
    }
    void* planes = nullptr;
    int rc = static_planes_address(&planes);
    if (rc != SGQ_OK) return rc;
    a.workspace = need ? planes : nullptr;
    a.workspace_bytes = need ? kStaticPlanesBytes : 0;
    return launch_linear_gemv(a);
}

}  // namespace sgq
