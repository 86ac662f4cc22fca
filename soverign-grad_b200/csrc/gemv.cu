// Decode-shape forward (M <= 16) for INT4 g=32 weights stored [N,K]:  y = x * deq(W)^T + bias.
//
// HBM-bound: every packed byte and every scale is read exactly once.
//   algorithmic bytes = N*K/2 (nibbles) + N*K/32*4 (scales) + M*K*4 (x) + M*N*4 (y).
//
// One persistent CTA per SM (two smaller ones in the compact form): consumer warps + 1 TMA
// producer warp + 1 reducer warp.
//   * The producer thread issues three TMA copies per stage: a 3-D box [8 steps][16 rows][128 B]
//     of packed weights (128-byte swizzle: the ldmatrix reads below are bank-conflict free) and two
//     2-D boxes [16 rows][32 fp32] of scales (128-byte rows again: a 32-byte-wide box would cost the
//     copy engine four times as many requests), into a ring of stages guarded by full/empty
//     mbarriers.  A step is 256 k of a 16-row tile.
//   * Integer inner product.  The activations arrive as group-scaled int8 digit planes
//     (gemv_prepare.cuh: 24-bit fixed point per 32-k group; in batches of three rows or more the
//     low digit sits in column sets of its own that are skipped, group by group, where it cannot
//     matter).  A word of eight 4-bit codes becomes two words of signed bytes holding
//     16 * code with one shift and two masks ((w << 4) & 0xF0F0F0F0 and w & 0xF0F0F0F0: a nibble in
//     the high half of a byte IS the two's-complement value times 16), and a 32-k group of 16
//     weight rows times 8 digit columns is ONE mma.sync m16n8k32 (s8 x s8 -> s32, exact).
//   * The exact group sums are turned into fp32 by the magic-number start value of the
//     accumulator, multiplied by the product of the group's fp32 weight scale and the group's
//     activation scale, and accumulated in fp32:
//       y[m,n] = sum_j 256^j * sum_g (scale[n,g] * sx[m,g]) * (16 S[n,g,m,j]),  sx carrying the 1/16.
//   * Consumer warps work in groups; every group owns whole tiles (all stages of a 16-row tile)
//     and the groups take alternate tiles, so the latency bubbles of one group (barrier waits, the
//     hand-off at the end of a tile) are covered by the others.  A warp that finishes its share
//     of a tile drops its partial sums into a ring in shared memory and moves on; the reducer
//     warp adds the partials in warp order (fixed order -> run-to-run deterministic), recombines
//     digits, adds bias, stores y.  Consumer warps never wait for one another.
//   * Activation planes too large for shared memory (e.g. K = 8192 at M = 16) are processed in
//     phases over K: the planes of one K range are resident while ALL tiles of the CTA stream their
//     weights of that range; later phases add into y.  The weights are still read exactly once.
//
// Error against the reference's single fp32 chain: see gemv_prepare.cuh (at most ~1e-4 of an
// output's scale for any activation distribution, ~1e-6 for one or two rows); everything up to the
// group sums is exact, the rest is fp32.
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

namespace {

constexpr int kRows = 16;                  // rows of W per tile (mma M)
constexpr int kStepK = 256;                // k per step (one 128-byte swizzle row per weight row)
constexpr int kStepsPerStage = 8;
constexpr int kWStepBytes = kRows * 128;   // 2048
constexpr int kSChunkBytes = kRows * 128;  // 16 rows x 32 fp32: the scales of 4 steps
constexpr int kStageW = kStepsPerStage * kWStepBytes;   // 16384
constexpr int kStageS = 2 * kSChunkBytes;               // 4096
constexpr int kStageBytes = kStageW + kStageS;          // 20480
constexpr int kMaxStages = 8;
constexpr int kMaxSlots = 8;               // ring of per-tile partial-sum buffers: two per warp group
constexpr int kSmemLimit = 227 * 1024;
constexpr int kCompactSmem = 113 * 1024;   // a CTA that leaves room for a second one on the same SM
constexpr int kMaxM = 16;

// Consumer organisation: NWARPS consumer warps in groups of `warps_per_tile(NWARPS)`; a group works
// on one tile at a time (each warp a fixed share of the steps of every stage), the NWARPS /
// warps_per_tile groups take alternate tiles.
__host__ __device__ constexpr int warps_per_tile(int nwarps) { return nwarps == 16 ? 8 : 4; }

// Partial-sum slots per warp group: two, so that a group can start its next tile while the reducer still
// reads the last one; one where the sums of a tile are large (many column sets) and shared memory is short.
__host__ __device__ constexpr int slots_per_group(int nmain) { return nmain <= 2 ? 2 : 1; }

struct Smem {
    uint32_t x_off, sx_off, flag_off, low_off, partial_off, misc_off, total;   // from a 1024-byte aligned base; stages first
};

// groups: 32-k groups of ONE phase; nmain / nlow: column sets (gemv_prepare.cuh).  The main digit planes,
// main scales and flags are always resident; the low parts only when the CTAs convert the activations
// themselves (low_resident) — prepared activations keep them in global memory.
__host__ __device__ inline Smem smem_layout(int nstages, uint32_t groups, int nmain, int nlow, int nwarps, bool low_resident) {
    Smem s;
    s.x_off = nstages * kStageBytes;
    s.sx_off = s.x_off + groups * 256u * nmain;
    s.flag_off = s.sx_off + groups * 32u * nmain;
    s.low_off = s.flag_off + (nlow ? groups * 16u : 0u);
    s.partial_off = s.low_off + (low_resident ? groups * (256u + 32u) * nlow : 0u);
    s.misc_off = s.partial_off + slots_per_group(nmain) * nwarps * (512u * nmain + 16u);   // slots x warps per tile x padded partial sums
    s.total = s.misc_off + (2u * kMaxStages + 2u * kMaxSlots + 2u) * 8u;
    return s;
}

__device__ __forceinline__ void report(uint32_t code, uint32_t detail) {
    atomicCAS(&g_status_gemv, 0u, (code << 24) | (detail & 0xFFFFFFu));
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

// Activation planes converted once into global scratch, in the prepared layout.  grid (rows, ceil(K / 1024)):
// a CTA converts 1024 consecutive k of one row, so that even a few rows spread over many SMs.
constexpr int kPrepThreads = 128;
__global__ void __launch_bounds__(kPrepThreads) gemv_prepare_x_kernel(const float* __restrict__ x, int64_t K, int mode, int nmain,
                                                                     int nlow, uint8_t* __restrict__ planes,
                                                                     const unsigned long long* wait_slots, int wait_world,
                                                                     const unsigned long long* wait_epoch, unsigned int wait_budget) {
    pdl_launch_dependents();
    pdl_wait();                                        // x comes from the kernel before this one
    // Deferred exchange between GPUs: x may hold slices that other GPUs store, so this kernel waits as the decode
    // kernel itself does in its prologue (every rank has finished the exchanges this GPU has finished).
    if (wait_slots != nullptr && !peer_wait_epoch(wait_slots, wait_world, wait_epoch, threadIdx.x & 31, wait_budget)) {
        if ((threadIdx.x & 31) == 0) report(kDevErrPeerWait, 0x30000u);
    }
    const int m = blockIdx.x, M = gridDim.x;
    const int chunks = static_cast<int>(K / 8);
    const PreparedParts pp = prepared_parts(planes, static_cast<size_t>(K / 32), nmain, nlow);
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<int64_t>(m) * K);
    const int c = blockIdx.y * kPrepThreads + threadIdx.x;
    if (c < chunks) {                                  // chunks % 32 == 0: whole warps
        const float4 a = __ldg(xr + 2 * c), b = __ldg(xr + 2 * c + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        convert_groups<kOrderNibble>(v, m, M, static_cast<size_t>(c >> 5) * 8, mode, nmain, nlow, 0.0625f, pp);
    }
}

enum : int { kFlagEarlyWeights = 1, kFlagPrepared = 2 };

// NM / NL: main and low sets of 8 digit columns (gemv_prepare.cuh; NL > 0: batches of three rows or
// more); NWARPS: consumer warps (16, or 8 in the compact two-CTAs-per-SM form); HALF: one row, only
// even columns carry data and the odd accumulators are skipped.
template <int NM, int NL, int NWARPS, bool HALF, bool SPLIT>
__global__ void __launch_bounds__((NWARPS + 2) * 32, NWARPS == 8 ? 2 : 1)
gemv_int4_nk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                    const float* __restrict__ x, const uint8_t* __restrict__ planes, const float* __restrict__ bias,
                    float* __restrict__ y, int M, int64_t K, int64_t N, int64_t ldy, int nstages, int nphases, int flags,
                    const __grid_constant__ PeerOut peers) {
    constexpr int kMode = NL > 0 ? 2 : (HALF ? 0 : 1);
    constexpr int kDigitsOut = NL > 0 ? 2 : 3;
    constexpr int WPT = warps_per_tile(NWARPS);
    constexpr int kGroups = NWARPS / WPT;              // warp groups = tiles in work at any time
    constexpr int kSlots = slots_per_group(NM) * kGroups;
    constexpr int GPW = 64 / WPT;                      // 32-k groups of a stage per warp (8 or 16)
    constexpr int kConsumerThreads = NWARPS * 32;
    constexpr int kPStride = 128 * NM + 4;             // floats per warp in a partial-sum slot (padded against bank conflicts)
    static_assert(GPW % 8 == 0, "a warp takes whole steps");
    static_assert(kSlots <= kMaxSlots, "partial-sum ring");

    extern __shared__ uint8_t smem_raw[];
    // aligned by pointer arithmetic on the shared array itself: a round trip through an integer would make the
    // compiler lose the address space and emit generic loads for every shared-memory access below
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int spt = static_cast<int>(K / kStepK);      // steps per tile (K % 256 == 0)
    const int sp = spt / nphases;                      // steps per tile and phase
    const bool prepared = (flags & kFlagPrepared) != 0;
    const Smem L = smem_layout(nstages, static_cast<uint32_t>(sp) * 8u, NM, NL, NWARPS, !prepared);
    uint8_t* stages = smem;
    uint8_t* xs = smem + L.x_off;
    float* sxs = reinterpret_cast<float*>(smem + L.sx_off);
    uint8_t* flg = smem + L.flag_off;
    float* partial = reinterpret_cast<float*>(smem + L.partial_off);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.misc_off);
    uint64_t* empty = full + kMaxStages;
    uint64_t* pfull = empty + kMaxStages;      // [kSlots] every warp of the tile's group has left its partial sums
    uint64_t* pempty = pfull + kMaxSlots;      // [kSlots] the reducer is done with the slot
    uint64_t* xfull = pempty + kMaxSlots;      // the activation planes of a phase have landed
    uint64_t* xempty = xfull + 1;              // every consumer warp is done with the planes of a phase

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t ntiles = (N + kRows - 1) / kRows;
    const int ring_slots = nstages / kGroups;          // stage slots per warp group (nstages >= kGroups)
    // Split form (no CTA has more than one tile, so one warp group would idle): the stages of the tile alternate
    // between the groups, each group leaves its partial sums in a slot of its own and the reducer adds both.
    // (a template parameter: the checks below cost the whole-tile form 3 % when they are decided at run time)
    constexpr bool split = SPLIT;
    constexpr int kSPG = kSlots / kGroups;             // partial-sum slots per group

    pdl_launch_dependents();            // the next kernel may begin its prologue; it waits for this grid before touching data
    if (threadIdx.x == NWARPS * 32) {   // the producer thread: start fetching both descriptors now
        tma_prefetch_descriptor(&map_w);
        tma_prefetch_descriptor(&map_s);
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < nstages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], WPT);
        }
        for (int i = 0; i < kSlots; ++i) {
            mbar_init(&pfull[i], WPT);
            mbar_init(&pempty[i], 1);
        }
        mbar_init(xfull, 1);
        mbar_init(xempty, NWARPS);
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    __syncthreads();
    // Everything above touches no global data.  From here on every thread except the producer
    // first waits for the kernels this launch depends on (they wrote x / the planes, and may still
    // be reading y); the producer decides for itself below, because weights are not their output.
    if (warp != NWARPS) pdl_wait();

    if (warp == NWARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            // Weights and scales are parameters, not the output of the kernel before this one: with
            // early weights the first ring of stages is requested before the dependency wait, so the
            // weight stream overlaps the tail of that kernel.  The activation planes are its output
            // and are copied only after the wait.
            bool synced = false;
            auto dependency_sync = [&]() {
                if (synced) return;
                synced = true;
                pdl_wait();
                if (prepared) fence_proxy_async_all();      // the planes were written through the generic proxy
            };
            auto copy_planes = [&](int ph) {
                // main digit planes, main scales and flags of this phase: contiguous ranges, in pieces of <= 32 KiB
                const uint32_t pgroups = static_cast<uint32_t>(sp) * 8u;
                const uint32_t dbytes = pgroups * 256u * NM, sbytes = pgroups * 32u * NM, fbytes = NL ? pgroups * 16u : 0u;
                const size_t groups_all = static_cast<size_t>(K / 32);
                const uint8_t* dsrc = planes + static_cast<size_t>(ph) * dbytes;
                const uint8_t* ssrc = planes + groups_all * 256u * (NM + NL) + static_cast<size_t>(ph) * sbytes;
                const uint8_t* fsrc = planes + groups_all * (256u + 32u) * (NM + NL) + static_cast<size_t>(ph) * fbytes;
                mbar_arrive_expect_tx(xfull, dbytes + sbytes + fbytes);
                for (uint32_t off = 0; off < dbytes; off += 32768u)
                    bulk_copy_g2s(xs + off, dsrc + off, (dbytes - off < 32768u) ? dbytes - off : 32768u, xfull);
                for (uint32_t off = 0; off < sbytes; off += 32768u)
                    bulk_copy_g2s(reinterpret_cast<uint8_t*>(sxs) + off, ssrc + off, (sbytes - off < 32768u) ? sbytes - off : 32768u, xfull);
                if (NL) bulk_copy_g2s(flg, fsrc, fbytes, xfull);
            };
            if (!(flags & kFlagEarlyWeights)) dependency_sync();
            // Every warp group has its own part of the stage ring (ring_slots consecutive slots) and its own
            // stage counter: a slot is then always filled for, and waited on by, the same group, use after
            // use, so a waiting warp can never be a whole barrier phase ahead of the slot it looks at.
            uint32_t gseq[kGroups];
#pragma unroll
            for (int q = 0; q < kGroups; ++q) gseq[q] = 0;
            uint32_t tcount = 0;
            bool ok = true, planes_sent = false;
            for (int ph = 0; ph < nphases && ok; ++ph) {
                if (ph > 0) {
                    if (!mbar_wait(xempty, (ph - 1) & 1u)) {
                        report(kDevErrEmptyWait, 0x400000u | ph);
                        break;
                    }
                    copy_planes(ph);
                }
                for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
                    for (int c0 = 0; c0 < sp; c0 += kStepsPerStage) {
                        const int q = split ? (c0 / kStepsPerStage) % kGroups : static_cast<int>(tcount % kGroups);
                        uint32_t seq = 0;
#pragma unroll
                        for (int qq = 0; qq < kGroups; ++qq)
                            if (qq == q) seq = gseq[qq]++;
                        if (ph == 0 && !planes_sent && seq >= static_cast<uint32_t>(ring_slots)) {
                            // this group's part of the ring is full: nothing more to request early, and the wait
                            // below needs consumers that have their activations
                            dependency_sync();
                            if (prepared) copy_planes(0);
                            planes_sent = true;
                        }
                        const int st = q * ring_slots + static_cast<int>(seq % ring_slots);
                        const uint32_t par = (seq / ring_slots) & 1u;
                        if (!mbar_wait(&empty[st], par ^ 1u)) {
                            report(kDevErrEmptyWait, seq);
                            ok = false;
                            break;
                        }
                        // steps past the end of K are out of range in the third dimension: zero-filled, still counted
                        mbar_arrive_expect_tx(&full[st], kStageBytes);
                        uint8_t* sw = stages + st * kStageBytes;
                        const int32_t step0 = ph * sp + c0;
                        tma_load_3d(sw, &map_w, &full[st], 0, static_cast<int32_t>(tile * kRows), step0);
                        // scales of steps step0 .. step0+3 and step0+4 .. step0+7 (columns past K/32 are zero-filled)
                        tma_load_2d(sw + kStageW, &map_s, &full[st], step0 * 8, static_cast<int32_t>(tile * kRows));
                        tma_load_2d(sw + kStageW + kSChunkBytes, &map_s, &full[st], step0 * 8 + 32, static_cast<int32_t>(tile * kRows));
                    }
                }
                if (ph == 0 && !planes_sent) {
                    dependency_sync();
                    if (prepared) copy_planes(0);
                    planes_sent = true;
                }
            }
            dependency_sync();
        }
        return;
    }

    const int64_t my_tiles = (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x;      // per phase

    if (warp == NWARPS + 1) {
        // ---------------- reducer ----------------
        // lane -> output pairs (tile row r, batch row m); per digit column the partial sums of the
        // tile's warps are added in warp order, then digits are recombined: y = sum_j 256^j v_j + bias.
        uint32_t tcount = 0;
        const int pairs = kRows * M;
        bool ok = true;
        for (int ph = 0; ph < nphases && ok; ++ph) {
            for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
                // whole tiles: tile t is group t % kGroups' and uses slot t % kSlots; split: both groups, slots
                // (t % kSPG) * kGroups + group
                const int slot = split ? static_cast<int>(tcount % kSPG) * kGroups : static_cast<int>(tcount % kSlots);
                const uint32_t pph = split ? (tcount / kSPG) & 1u : (tcount / kSlots) & 1u;
                if (!mbar_wait(&pfull[slot], pph) || (split && !mbar_wait(&pfull[slot + 1], pph))) {
                    report(kDevErrFullWait, 0x800000u | tcount);
                    ok = false;
                    break;
                }
                float* pbuf = partial + slot * (WPT * kPStride);
                // Step 1: add the warps' partial sums fragment-wise, in warp order (fixed order -> the same
                // bits every run): lane L owns the float4 every consumer lane L wrote, so these are
                // conflict-free 128-bit reads.  The sum goes back into the first warp's part of the slot.
#pragma unroll
                for (int s = 0; s < NM; ++s) {
                    float4 sum = *reinterpret_cast<const float4*>(pbuf + (s * 32 + lane) * 4);
#pragma unroll
                    for (int w = 1; w < (split ? 2 * WPT : WPT); ++w) {       // split: the second group's slot lies right behind
                        const float4 v = *reinterpret_cast<const float4*>(pbuf + w * kPStride + (s * 32 + lane) * 4);
                        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                    }
                    *reinterpret_cast<float4*>(pbuf + (s * 32 + lane) * 4) = sum;
                }
                __syncwarp();
                // Step 2: one value per (output, digit): recombine the digits, add bias, store.
                for (int p = lane; p < pairs; p += 32) {
                    const int r = p & 15, m = p >> 4;
                    const int gg = r & 7, hi = r >> 3;
                    float acc = 0.0f, weight = 1.0f;
#pragma unroll
                    for (int j = 3 - kDigitsOut; j < 3; ++j, weight *= 256.0f) {
                        int set, cc;
                        digit_slot(kMode, m, j, &set, &cc);
                        const float v = pbuf[(set * 32 + gg * 4 + (cc >> 1)) * 4 + hi * 2 + (cc & 1)];
                        acc = __fmaf_rn(weight, v, acc);
                    }
                    const int64_t n = tile * kRows + r;
                    if (n < N) {
                        float v = acc;
                        if (ph == 0) {
                            if (bias) v += bias[n];
                        } else {
                            v += y[static_cast<int64_t>(m) * ldy + n];        // written by this same lane in the phase before
                        }
                        if (peers.n == 0) {
                            y[static_cast<int64_t>(m) * ldy + n] = v;
                        } else {
                            // fused all-gather: the slice goes into every GPU's full-width output (plain peer stores)
                            for (int r2 = 0; r2 < peers.n; ++r2) peers.p[r2][static_cast<int64_t>(m) * ldy + n] = v;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&pempty[slot]);
                    if (split) mbar_arrive(&pempty[slot + 1]);
                }
            }
        }
        if (peers.n > 0 && peers.sig[0] != nullptr && peers.deferred) {
            // Deferred exchange: this CTA's slices are out; it counts itself with every rank and is done.  The next
            // kernel on these signals waits, in its prologue, until every rank's count has reached its own.
            peer_arrive(peers.sig, peers.rank, peers.n, peers.state, lane);
        } else if (peers.n > 0 && peers.sig[0] != nullptr) {
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
                if (!peer_signal_and_wait(peers.sig, peers.rank, peers.n, peers.state, lane, &late, peers.poll_budget) && lane == 0)
                    report(kDevErrPeerWait, 0x10000u);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    bool alive = true;   // false after a wait ran out: skip the math but keep every barrier balanced
    if (peers.n > 0 && peers.deferred && peers.sig[0] != nullptr) {
        // Deferred exchange: the kernels before this one only signalled.  Before this kernel reads activations
        // that other GPUs may have stored here, or stores into buffers other GPUs may still read, every rank
        // must have finished the exchanges this GPU has finished (its own epoch, written by the kernel before).
        if (!peer_wait_epoch(peers.sig[peers.rank], peers.n, peers.state, lane, peers.poll_budget)) {
            if (lane == 0) report(kDevErrPeerWait, 0x20000u);
        }
    }
    if (!prepared) {
        // Activations -> digit planes inside the CTA (small batches, one phase).  A warp converts 256 k
        // per iteration; M * K / 8 is a multiple of 32, so whole warps are in or out.
        const int chunks = static_cast<int>(K / 8);
        const int items = chunks * M;
        PreparedParts pp;
        pp.dmain = xs;
        pp.smain = sxs;
        pp.flags = flg;
        pp.dlow = smem + L.low_off;
        pp.slow = reinterpret_cast<float*>(smem + L.low_off + static_cast<uint32_t>(sp) * 8u * 256u * NL);
        for (int it = threadIdx.x; it < items; it += kConsumerThreads) {
            const int m = it / chunks, c = it - m * chunks;
            const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * static_cast<int64_t>(it));
            const float4 b = __ldg(reinterpret_cast<const float4*>(x) + 2 * static_cast<int64_t>(it) + 1);
            const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            convert_groups<kOrderNibble>(v, m, M, static_cast<size_t>(c >> 5) * 8, kMode, NM, NL, 0.0625f, pp);
        }
        named_barrier_sync(1, kConsumerThreads);
    }

    const int g = lane >> 2, t = lane & 3;
    const int my_group = warp / WPT, wj = warp % WPT;
    // ldmatrix row address of this lane inside a step box, for group pair (2i, 2i+1): matrix (lane >> 3)
    // = (rows 0-7 | rows 8-15) x (group 2i | 2i+1); 128-byte swizzle: 16-byte chunk index ^ (row & 7)
    const uint32_t lm_row = (lane & 7) + 8 * ((lane >> 3) & 1);
    const uint32_t lm_sel = lane >> 4;
    uint32_t lm_off[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) lm_off[i] = lm_row * 128 + (((2 * i + lm_sel) ^ (lane & 7)) << 4);
    const uint32_t stages_u32 = smem_u32(stages);

    uint32_t seq = 0, tcount = 0;         // seq: stages of THIS group so far
    for (int ph = 0; ph < nphases; ++ph) {
        // Low digit planes and scales of this phase: in global memory behind the prepared buffer, or in shared
        // memory when this CTA converted the activations itself (generic pointers: the loads work on either).
        const uint8_t* lowd = smem + L.low_off;
        const float* lows = reinterpret_cast<const float*>(smem + L.low_off + static_cast<uint32_t>(sp) * 8u * 256u * NL);
        if (prepared && NL > 0) {
            const size_t groups_all = static_cast<size_t>(K / 32), g0 = static_cast<size_t>(ph) * sp * 8;
            lowd = planes + groups_all * 256u * NM + g0 * 256u * NL;
            lows = reinterpret_cast<const float*>(planes + groups_all * (256u * (NM + NL) + 32u * NM)) + g0 * 8u * NL;
        }
        if (prepared && alive && !mbar_wait(xfull, ph & 1u)) {
            report(kDevErrFullWait, 0x400000u | ph);
            alive = false;
        }
        for (int64_t ti = 0; ti < my_tiles; ++ti, ++tcount) {
            if (!split && static_cast<int>(tcount % kGroups) != my_group) continue;       // another group's tile
            float total[NM + NL][4];
#pragma unroll
            for (int s = 0; s < NM + NL; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i) total[s][i] = 0.0f;

            for (int c0 = 0; c0 < sp; c0 += kStepsPerStage) {
                if (split && (c0 / kStepsPerStage) % kGroups != my_group) continue;       // the other group's stage
                const int st = my_group * ring_slots + static_cast<int>(seq % ring_slots);
                const uint32_t par = (seq / ring_slots) & 1u;
                if (alive && !mbar_wait(&full[st], par)) {
                    report(kDevErrFullWait, seq);
                    alive = false;
                }
#pragma unroll
                for (int u = 0; u < GPW / 8; ++u) {
                    const int step_in_stage = wj * (GPW / 8) + u;
                    const int step = c0 + step_in_stage;                 // within the phase
                    if (alive && step < sp) {
                        const uint32_t wbox = stages_u32 + st * kStageBytes + step_in_stage * kWStepBytes;
                        // scales: [2 chunks of 4 steps][16 rows][128 B], 16-byte units swizzled by the row like the weights
                        const uint8_t* sbox = stages + st * kStageBytes + kStageW + (step_in_stage >> 2) * kSChunkBytes + g * 128;
                        const int su = (step_in_stage & 3) * 2;
                        const uint8_t* xg = xs + static_cast<size_t>(step) * 8 * (256 * NM);
                        const float* sg = sxs + (static_cast<size_t>(step) * 8 * 4 + t) * (2 * NM);      // this lane's group scales
                        const uint8_t* fg = flg + static_cast<size_t>(step) * 8 * 16;
                        constexpr int BG = NM <= 2 ? 4 : 2;              // 32-k groups whose MMAs are in flight together
#pragma unroll
                        for (int hb = 0; hb < 8 / BG; ++hb) {
                            const int hh = (hb * BG) >> 2;               // which half of the step: 16-byte unit of the scales
                            const float4 sc_lo = *reinterpret_cast<const float4*>(sbox + (((su + hh) ^ g) << 4));          // scales of row g
                            const float4 sc_hi = *reinterpret_cast<const float4*>(sbox + 1024 + (((su + hh) ^ g) << 4));   // and of row g + 8
                            uint32_t wv[BG / 2][4];                      // [pair of groups]{rows 0-7, rows 8-15} x 2
#pragma unroll
                            for (int pq = 0; pq < BG / 2; ++pq) ldmatrix_x4(wv[pq], wbox + lm_off[(hb * BG) / 2 + pq]);
                            // The main-set MMAs of these groups are issued before any of their results is used, so
                            // that the tensor-pipe latency of one group is covered by the issue of the others.
                            int d[BG][NM][4];
                            float2 sxv[BG][NM];                          // activation scales of columns 2t, 2t+1 of every main set
                            uint32_t av[BG][4];
#pragma unroll
                            for (int i = 0; i < BG; ++i) {
                                const int gi = hb * BG + i;              // group within the step
                                const uint32_t w_lo = wv[i >> 1][(i & 1) * 2], w_hi = wv[i >> 1][(i & 1) * 2 + 1];
                                av[i][0] = (w_lo << 4) & 0xF0F0F0F0u;    // row g,   k = 8t + {0,2,4,6}: 16 * code as s8
                                av[i][1] = (w_hi << 4) & 0xF0F0F0F0u;    // row g+8
                                av[i][2] = w_lo & 0xF0F0F0F0u;           // row g,   k = 8t + {1,3,5,7}
                                av[i][3] = w_hi & 0xF0F0F0F0u;           // row g+8
                                const uint8_t* xgi = xg + gi * (256 * NM);
                                const float* sgi = sg + gi * (8 * NM);
#pragma unroll
                                for (int s2 = 0; s2 < NM; ++s2) sxv[i][s2] = *reinterpret_cast<const float2*>(sgi + 2 * s2);
#pragma unroll
                                for (int s2 = 0; s2 < NM; ++s2) {
                                    if ((s2 & 1) == 0 && s2 + 1 < NM) {  // two main sets side by side: one 128-bit load per lane
                                        const uint4 q = *reinterpret_cast<const uint4*>(xgi + (s2 >> 1) * 512 + lane * 16);
                                        mma_s8s8_16832_magic(d[i][s2], av[i], q.x, q.y);
                                        mma_s8s8_16832_magic(d[i][s2 + 1], av[i], q.z, q.w);
                                    } else if ((s2 & 1) == 0) {
                                        const uint2 q = *reinterpret_cast<const uint2*>(xgi + plane_offset(0, NM, s2, lane));
                                        mma_s8s8_16832_magic(d[i][s2], av[i], q.x, q.y);
                                    }
                                }
                            }
#pragma unroll
                            for (int i = 0; i < BG; ++i) {
                                const int gi = hb * BG + i, gq = gi & 3;
                                const float s_lo = gq == 0 ? sc_lo.x : gq == 1 ? sc_lo.y : gq == 2 ? sc_lo.z : sc_lo.w;
                                const float s_hi = gq == 0 ? sc_hi.x : gq == 1 ? sc_hi.y : gq == 2 ? sc_hi.z : sc_hi.w;
#pragma unroll
                                for (int s2 = 0; s2 < NM; ++s2) {
                                    // d holds 12582912.0f + 16 * (exact group sum) as fp32 bits
                                    const float f_lo = __fmul_rn(s_lo, sxv[i][s2].x), f_hi = __fmul_rn(s_hi, sxv[i][s2].x);
                                    total[s2][0] = __fmaf_rn(f_lo, __fsub_rn(__int_as_float(d[i][s2][0]), kMagicF), total[s2][0]);
                                    total[s2][2] = __fmaf_rn(f_hi, __fsub_rn(__int_as_float(d[i][s2][2]), kMagicF), total[s2][2]);
                                    if (kMode == 2) {                    // columns 2t and 2t+1 belong to the same batch row: one scale
                                        total[s2][1] = __fmaf_rn(f_lo, __fsub_rn(__int_as_float(d[i][s2][1]), kMagicF), total[s2][1]);
                                        total[s2][3] = __fmaf_rn(f_hi, __fsub_rn(__int_as_float(d[i][s2][3]), kMagicF), total[s2][3]);
                                    } else if (kMode == 1) {
                                        const float e_lo = __fmul_rn(s_lo, sxv[i][s2].y), e_hi = __fmul_rn(s_hi, sxv[i][s2].y);
                                        total[s2][1] = __fmaf_rn(e_lo, __fsub_rn(__int_as_float(d[i][s2][1]), kMagicF), total[s2][1]);
                                        total[s2][3] = __fmaf_rn(e_hi, __fsub_rn(__int_as_float(d[i][s2][3]), kMagicF), total[s2][3]);
                                    }
                                }
                                // low digits: only where a row of the set flagged this group (rare: one value dominating its group)
#pragma unroll
                                for (int l = 0; l < NL; ++l) {
                                    const uint2 fl = *reinterpret_cast<const uint2*>(fg + gi * 16 + l * 8);
                                    if ((fl.x | fl.y) != 0u) {           // the same for every lane of the warp
                                        const size_t grp = static_cast<size_t>(step) * 8 + gi;       // group within the phase
                                        const uint2 q = *reinterpret_cast<const uint2*>(lowd + plane_offset(grp, NL, l, lane));
                                        const float2 sl = *reinterpret_cast<const float2*>(lows + ((grp * 4 + t) * NL + l) * 2);
                                        int dl[4];
                                        mma_s8s8_16832_magic(dl, av[i], q.x, q.y);
                                        total[NM + l][0] = __fmaf_rn(__fmul_rn(s_lo, sl.x), __fsub_rn(__int_as_float(dl[0]), kMagicF), total[NM + l][0]);
                                        total[NM + l][1] = __fmaf_rn(__fmul_rn(s_lo, sl.y), __fsub_rn(__int_as_float(dl[1]), kMagicF), total[NM + l][1]);
                                        total[NM + l][2] = __fmaf_rn(__fmul_rn(s_hi, sl.x), __fsub_rn(__int_as_float(dl[2]), kMagicF), total[NM + l][2]);
                                        total[NM + l][3] = __fmaf_rn(__fmul_rn(s_hi, sl.y), __fsub_rn(__int_as_float(dl[3]), kMagicF), total[NM + l][3]);
                                    }
                                }
                            }
                        }
                    }
                }
                // everything loaded from the stage has been consumed once the accumulators are final
                uint32_t fold = 0;
#pragma unroll
                for (int s = 0; s < NM + NL; ++s) fold ^= __float_as_uint(total[s][0]) ^ __float_as_uint(total[s][2]);
                const uint32_t landed = loads_landed(fold);
                if (lane == 0) mbar_arrive_after(&empty[st], landed);
                ++seq;
            }

            // ---- hand the tile's partial sums to the reducer warp ----
            {
                const int slot = split ? static_cast<int>(tcount % kSPG) * kGroups + my_group : static_cast<int>(tcount % kSlots);
                const uint32_t pph = split ? (tcount / kSPG) & 1u : (tcount / kSlots) & 1u;
                if (alive && !mbar_wait(&pempty[slot], pph ^ 1u)) {
                    report(kDevErrEmptyWait, 0x800000u | tcount);
                    alive = false;
                }
                // Low-digit sums join the accumulator of digit 1 of their batch row (the main scales carry the
                // factor 256 between the digits).  Low set l holds row 8l + 2t + e in column 2t + e of lane t; that
                // row's digit-1 accumulator is column 2t' of main set (8l + 2t + e) / 4 in lane t' = 2 (t & 1) + e.
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
                float* pbuf = partial + slot * (WPT * kPStride) + wj * kPStride;
#pragma unroll
                for (int s = 0; s < NM; ++s)
                    *reinterpret_cast<float4*>(pbuf + (s * 32 + lane) * 4) =
                        make_float4(total[s][0], total[s][1], total[s][2], total[s][3]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&pfull[slot]);
            }
        }
        if (nphases > 1) {
            __syncwarp();
            if (lane == 0) mbar_arrive(xempty);
        }
    }
}

struct Plan {
    PreparedLayout L;
    int nwarps, nstages, nphases;
    bool pre;          // activation planes prepared by a separate launch into the workspace
    uint32_t smem;
    size_t planes_bytes;
};

// Finds the fewest K phases (1, 2, 4, ...) whose activation planes fit in shared memory next to at
// least `min_stages` pipeline stages.  A phase covers whole stages (steps per phase % 8 == 0) unless
// there is only one.  compact: a CTA that leaves room for a second one on the same SM (half the
// shared memory, 10 warps); with overlapped launches the CTA of the NEXT kernel then sits beside the
// one still running and streams its first weight stages in the meantime.
bool make_plan(int64_t M, int64_t K, bool have_workspace, Plan* p, bool compact = false, bool allow_phases = true) {
    if (M < 1 || M > kMaxM || K < kStepK || (K % kStepK) != 0) return false;
    p->L = prepared_layout(M, K);
    p->planes_bytes = p->L.bytes;
    p->nwarps = compact ? 8 : 16;
    const int limit = compact ? kCompactSmem : kSmemLimit;
    const int spt = static_cast<int>(K / kStepK);
    for (int nph = 1; nph <= spt; nph *= 2) {
        if (spt % nph) break;
        const int sp = spt / nph;
        if (nph > 1 && (sp % kStepsPerStage) != 0) break;
        if (nph > 1 && (!have_workspace || !allow_phases)) break;      // phases need the planes in global memory
        const int min_stages = 2;                          // one slot for each of the two warp groups
        for (int st = kMaxStages; st >= min_stages; --st) {
            // in-CTA conversion while it is a few items per thread; larger batches are converted once by a pre-kernel
            const bool pre = have_workspace && (nph > 1 || M * (K / 8) > 2 * p->nwarps * 32);
            const Smem S = smem_layout(st, static_cast<uint32_t>(sp) * 8u, p->L.nmain, p->L.nlow, p->nwarps, !pre);
            if (S.total + 1024 <= static_cast<uint32_t>(limit)) {
                p->nstages = st;
                p->nphases = nph;
                p->smem = S.total + 1024;
                p->pre = pre;
                return true;
            }
        }
    }
    return false;
}

// Rows of the batch one launch can take without a workspace: the largest m <= M whose activation
// planes fit in shared memory next to the pipeline stages (0: not even one row fits).  Larger
// batches then run as several launches over row blocks; each streams the weights again, which is
// still far better than the any-shape kernel.
int64_t rows_per_launch(int64_t M, int64_t K, bool have_workspace, bool allow_phases = true) {
    Plan p;
    // the whole batch in one pass over K — unless it is a wide batch that leaves the pipeline fewer than four stages
    if (make_plan(M, K, have_workspace, &p, false, false) && (M <= 8 || p.nstages >= 4)) return M;
    if (M > 8) {
        // two or more launches of at most 8 rows each: measured faster than K phases over wide column sets
        const int64_t blocks = (M + 7) / 8, rows = (M + blocks - 1) / blocks;
        if (make_plan(rows, K, have_workspace, &p, false, false)) return rows;
    }
    if (allow_phases && make_plan(M, K, have_workspace, &p)) return M;           // K phases
    for (int64_t m = M - 1; m >= 1; --m)
        if (make_plan(m, K, have_workspace, &p, false, allow_phases)) return m;
    return 0;
}

template <int NM, int NL, int NWARPS, bool HALF, bool SPLIT = false>
int launch_variant(const LinearArgs& a, const Plan& p, const CUtensorMap& map_w, const CUtensorMap& map_s, int grid,
                   bool planes_ready) {
    // no CTA with more than one tile, tiles of two stages or more, one phase: the stages alternate between the warp groups
    if (!SPLIT && NWARPS == 16 && ceil_div(a.N, kRows) <= grid && p.nphases == 1 && a.K / kStepK > kStepsPerStage)
        return launch_variant<NM, NL, NWARPS, HALF, NWARPS == 16>(a, p, map_w, map_s, grid, planes_ready);
    static SmemOptIn optin;
    auto kernel = gemv_int4_nk_kernel<NM, NL, NWARPS, HALF, SPLIT>;
    SGQ_CUDA_TRY(optin.ensure(kernel, NWARPS == 8 ? kCompactSmem : kSmemLimit));
    const uint8_t* planes = static_cast<const uint8_t*>(a.workspace);
    const bool overlap = stream_overlap_enabled();
    if (p.pre && !planes_ready) {
        const bool wait = a.peers.n > 0 && a.peers.deferred && a.peers.sig[0] != nullptr;
        SGQ_CUDA_TRY(launch_kernel(gemv_prepare_x_kernel, dim3(static_cast<unsigned>(a.M), static_cast<unsigned>(ceil_div(a.K / 8, kPrepThreads))), dim3(kPrepThreads), 0, a.stream, overlap,
                                   a.x, a.K, p.L.mode, p.L.nmain, p.L.nlow, static_cast<uint8_t*>(a.workspace),
                                   wait ? a.peers.sig[a.peers.rank] : nullptr, a.peers.n, a.peers.state, a.peers.poll_budget));
    }
    const int flags = (overlap ? kFlagEarlyWeights : 0) | (p.pre ? kFlagPrepared : 0);
    SGQ_CUDA_TRY(launch_kernel(kernel, dim3(static_cast<unsigned>(grid)), dim3((NWARPS + 2) * 32), p.smem, a.stream, overlap, map_w,
                               map_s, a.x, planes, a.bias, a.y, static_cast<int>(a.M), a.K, a.N, a.ldy, p.nstages, p.nphases, flags,
                               a.peers));
    return SGQ_OK;
}

template <int NM, int NL, bool HALF>
int launch_nsets(const LinearArgs& a, const Plan& p, const CUtensorMap& map_w, const CUtensorMap& map_s, int grid,
                 bool planes_ready) {
    return p.nwarps == 8 ? launch_variant<NM, NL, 8, HALF>(a, p, map_w, map_s, grid, planes_ready)
                         : launch_variant<NM, NL, 16, HALF>(a, p, map_w, map_s, grid, planes_ready);
}

bool shape_ok(int64_t M, int64_t K, int64_t N) {
    return M >= 1 && M <= kMaxM && K >= kStepK && (K % kStepK) == 0 && K < (1LL << 24) && N >= 1 && N < (1LL << 31);
}

}  // namespace

bool gemv_supported(const LinearArgs& a) {
    return a.bits == 4 && a.layout == SGQ_LAYOUT_NK && a.group == 32 && shape_ok(a.M, a.K, a.N) && aligned(a.wq, 16) &&
           aligned(a.scales, 16) && aligned(a.x, 16) && rows_per_launch(a.M, a.K, false) >= 1;
}

// Scratch for the prepared activation planes (batches converted by the pre-kernel); 0 when the
// conversion happens inside the CTAs.
size_t gemv_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout) {
    if (bits != 4 || layout != SGQ_LAYOUT_NK || !shape_ok(M, K, N > 0 ? N : 1)) return 0;
    Plan p, c;
    const int64_t rows = rows_per_launch(M, K, true);                     // row blocks reuse one scratch
    if (rows < 1 || !make_plan(rows, K, true, &p)) return 0;
    const bool compact_pre = make_plan(rows, K, true, &c, true) && c.pre;  // what an overlapped launch in compact form would want
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
    if (!shape_ok(M, K, 1) || !make_plan(M, K, true, &p)) return 0;
    return (p.planes_bytes + 255) / 256 * 256;
}

int launch_prepare_x(const float* x, int64_t M, int64_t K, void* prepared, cudaStream_t s) {
    const PreparedLayout L = prepared_layout(M, K);
    SGQ_CUDA_TRY(launch_kernel(gemv_prepare_x_kernel, dim3(static_cast<unsigned>(M), static_cast<unsigned>(ceil_div(K / 8, kPrepThreads))), dim3(kPrepThreads), 0, s,
                               stream_overlap_enabled(), x, K, L.mode, L.nmain, L.nlow, static_cast<uint8_t*>(prepared),
                               static_cast<const unsigned long long*>(nullptr), 0, static_cast<const unsigned long long*>(nullptr), 0u));
    return SGQ_OK;
}

namespace {
int launch_gemv_impl(const LinearArgs& a, bool planes_ready) {
    Plan p;
    const size_t want = planes_ready ? gemv_prepared_bytes(a.M, a.K) : gemv_workspace_bytes(a.bits, a.M, a.K, a.N, a.layout);
    // K phases add into y in place, which the fused all-gather (stores into other GPUs) cannot do; the planes in
    // the scratch (converted by the kernel in front) it can use like any other launch
    bool have_ws = a.workspace != nullptr && want > 0 && a.workspace_bytes >= want;
    const bool phases_ok = a.peers.n == 0;
    // (a batch whose planes fit in shared memory keeps the conversion inside the CTAs there: one launch less)
    if (a.peers.n > 0 && !planes_ready && rows_per_launch(a.M, a.K, false, false) >= a.M) have_ws = false;
    if (!planes_ready && a.bits == 4 && shape_ok(a.M, a.K, a.N)) {
        const int64_t rows = rows_per_launch(a.M, a.K, have_ws, phases_ok);
        if (rows >= 1 && rows < a.M) {               // planes of the whole batch do not fit: row blocks
            for (int64_t m0 = 0; m0 < a.M; m0 += rows) {
                LinearArgs sub = a;
                sub.M = (a.M - m0 < rows) ? a.M - m0 : rows;
                sub.x = a.x + m0 * a.K;
                sub.y = a.y + m0 * a.ldy;
                for (int r = 0; r < sub.peers.n; ++r) sub.peers.p[r] = a.peers.p[r] + m0 * a.ldy;
                // a fused barrier belongs to the last block only (the deferred form signals and waits per block)
                if (m0 + sub.M < a.M && !a.peers.deferred) sub.peers.sig[0] = nullptr;
                const int rc = launch_gemv_impl(sub, false);
                if (rc != SGQ_OK) return rc;
            }
            return SGQ_OK;
        }
    }
    LinearArgs probe = a;
    if (planes_ready) probe.x = static_cast<const float*>(a.workspace);      // x is not read: only its alignment rule is waived
    const bool compact = stream_overlap_compact();
    if (!gemv_supported(probe) || (planes_ready && !have_ws) ||
        !((compact && make_plan(a.M, a.K, have_ws, &p, true, phases_ok)) || make_plan(a.M, a.K, have_ws, &p, false, phases_ok))) {
        set_error("decode path needs INT4 g=32, layout NK, M<=16, K%%256==0, x digits fitting in shared memory, "
                  "16-byte aligned x/packed/scales");
        return SGQ_ERR_UNSUPPORTED;
    }
    if (planes_ready) {
        if (a.peers.n != 0 && p.nphases > 1) {
            set_error("prepared activations of this size cannot be combined with the fused all-gather");
            return SGQ_ERR_UNSUPPORTED;
        }
        p.pre = true;
    }
    // packed weights as (128 B, N rows, K/256 steps); scales as (K/32 fp32, N rows) in boxes of 32 x 16
    CUtensorMap map_w, map_s;
    const uint64_t steps = static_cast<uint64_t>(a.K / kStepK);
    {
        const uint64_t dims[3] = {128, static_cast<uint64_t>(a.N), steps};
        const uint64_t strides[2] = {static_cast<uint64_t>(a.K / 2), 128};
        const uint32_t box[3] = {128, kRows, kStepsPerStage};
        if (!make_tensor_map(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return SGQ_ERR_CUDA;
    }
    if (!make_tensor_map_2d(&map_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.scales, static_cast<uint64_t>(a.K / 32),
                            static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 32) * 4, 32, kRows, CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    const int64_t ntiles = ceil_div(a.N, kRows);
    const int64_t ctas = static_cast<int64_t>(sm_count()) * (p.nwarps == 8 ? 2 : 1);
    const int grid = static_cast<int>(ntiles < ctas ? ntiles : ctas);
    if (p.L.mode == 0) return launch_nsets<1, 0, true>(a, p, map_w, map_s, grid, planes_ready);
    if (p.L.mode == 1) return launch_nsets<1, 0, false>(a, p, map_w, map_s, grid, planes_ready);
    switch (p.L.nmain) {                 // three rows or more: ceil(M / 4) main sets, ceil(M / 8) low sets
        case 1: return launch_nsets<1, 1, false>(a, p, map_w, map_s, grid, planes_ready);
        case 2: return launch_nsets<2, 1, false>(a, p, map_w, map_s, grid, planes_ready);
        case 3: return launch_nsets<3, 2, false>(a, p, map_w, map_s, grid, planes_ready);
        default: return launch_nsets<4, 2, false>(a, p, map_w, map_s, grid, planes_ready);
    }
}
}  // namespace

// ---- entry point without any allocation ---------------------------------------------------
// Some callers of the decode forward cannot obtain device memory at call time: code running
// under a fixed memory budget that was handed out at start-up, a plugin loaded into a host that
// owns every allocation, or a serving loop that must not touch the allocator (and its locks)
// between tokens.  For them the activation planes live in this file-scope array instead of a
// caller workspace.  Every GPU that loads the library reserves these bytes until the process
// exits.  The size bounds the batches this entry point accepts: (K/32) * (sets * 288 + 16) bytes
// with sets = ceil(M/4) + ceil(M/8), e.g. K = 4096 with M = 16 or K = 8192 with M = 8.
constexpr size_t kStaticPlanesBytes = 448 * 1024;
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
    if (!shape_ok(a.M, a.K, a.N)) {
        set_error("decode path needs M<=16 and K%%256==0");
        return SGQ_ERR_UNSUPPORTED;
    }
    // the limit is stated for the whole batch: its prepared planes must fit the built-in scratch
    const size_t need = (prepared_layout(a.M, a.K).bytes + 255) / 256 * 256;
    if (need > kStaticPlanesBytes) {
        set_error("this batch needs %zu bytes of activation scratch; the built-in scratch holds %zu "
                  "(use sgq_linear_int4 with a caller workspace)", need, kStaticPlanesBytes);
        return SGQ_ERR_WORKSPACE;
    }
    void* planes = nullptr;
    int rc = static_planes_address(&planes);
    if (rc != SGQ_OK) return rc;
    a.workspace = planes;
    a.workspace_bytes = kStaticPlanesBytes;
    return launch_linear_gemv(a);
}

}  // namespace sgq
