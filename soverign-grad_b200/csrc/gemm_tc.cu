// Prefill-shape forward on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// weights stored [N,K]:  y[M,N] = x[M,K] * deq(W)^T + bias.
//
// Two modes share one persistent, warp-specialised kernel (one CTA per SM, 256 x 256 output
// tile = two 128-row halves, each with its own 256-column TMEM accumulator, sharing every B tile:
// half the B traffic and half the dequant work per flop of a 128 x 256 tile):
//   kI8   kind::i8 — INT8 weight codes and per-row quantized INT8 activations go from HBM to
//         shared memory by TMA untouched (128-byte swizzle), int32 accumulation is exact, the
//         epilogue applies sx[m] * sw[n].  k-block = 128.
//   kBF16 kind::f16 (bf16 x bf16 -> fp32) — activations are pre-converted to bf16; packed INT4
//         weights arrive by TMA as raw nibbles and dequant warps expand them in shared memory
//         to bf16 (exact integer from one LOP3 per pair, times the bf16-rounded group scale)
//         directly in the swizzled K-major layout the MMA reads.  k-block = 64 (two groups).
//
// Warp roles: 0 = TMA producer of A, 1 = MMA issuer (one thread), 2..5 = epilogue (TMEM lane
// quarter = warp % 4), 6 = TMA producer of B / raw nibbles, 7..22 = dequant (kBF16 only; 512
// threads, two per weight row).  All waits are bounded; a wait that runs out records a code in the device status
// word and the role winds down to the common exit.
#include <cuda_bf16.h>

#include <cstring>

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

// W8A8 | bf16 x INT4 g=32 | bf16 x INT8 codes (scale in the epilogue) | bf16 x bf16 weights already expanded in
// global memory (the [K,N] layouts: a kernel in front dequantizes and transposes them once per forward)
enum Mode { kI8 = 0, kBF16 = 1, kBF16W8 = 2, kBF16Plain = 3 };
// both operands arrive by TMA in their final shared-memory form: no dequant warps, no raw ring
__host__ __device__ constexpr bool direct_b(int mode) { return mode == kI8 || mode == kBF16Plain; }

constexpr int BM = 256, BN = 256;     // two UMMA_M = 128 halves per tile
constexpr int kHalfM = 128;
constexpr int kABytes = BM * 128;     // 256 rows x 128 B (rows 128.. are the second half)
constexpr int kBBytes = BN * 128;     // 256 rows x 128 B
constexpr int kRawBytes = BN * 32;    // 256 rows x 64 nibbles (kBF16); the INT8 form is twice that, Cfg::kRawStageBytes
constexpr int kDequantWarps = 16;     // two threads per row of the 256-row weight tile (one 32-k group each)
constexpr int kEpilogueWarp0 = 2;
constexpr int kBProducerWarp = 6;     // loads B (kI8) or the raw nibbles (kBF16)
constexpr int kDequantWarp0 = 7;
constexpr int kTmemCols = 512;

// Three rings with their own depth, so that the latency of a TMA load never sits in the chain
// "MMA frees a slot -> slot refilled -> MMA": A tiles and raw nibbles are requested several
// k-blocks ahead; the (large) bf16 B tiles only need to cover the dequant time.
template <int MODE>
struct Cfg {
    static constexpr int kBlockK = MODE == kI8 ? 128 : 64;          // elements per k-block
    static constexpr int kUmmaK = MODE == kI8 ? 32 : 16;            // elements per instruction (32 bytes)
    static constexpr int kAStages = MODE == kBF16W8 ? 2 : 3;         // the INT8 raw ring takes the room of one A stage
    static constexpr int kBStages = 3;
    static constexpr int kRawStages = direct_b(MODE) ? 0 : 3;
    static constexpr int kRawStageBytes = MODE == kBF16W8 ? BN * 64 : kRawBytes;
    static constexpr int kWarps = direct_b(MODE) ? 7 : 7 + kDequantWarps;
    static constexpr int kThreads = kWarps * 32;
    static constexpr int kAOff = 0;
    static constexpr int kBOff = kAStages * kABytes;
    static constexpr int kRawOff = kBOff + kBStages * kBBytes;
    static constexpr int kOutOff = kRawOff + kRawStages * kRawStageBytes;   // 4 epilogue warps x [16 rows x 32 fp32], swizzled
    static constexpr int kBarOffset = kOutOff + 4 * 2048;
    static constexpr int kNumBars = 2 * kAStages + 2 * kBStages + 2 * (kRawStages ? kRawStages : 1) + 4;
    static constexpr int kSmemBytes = kBarOffset + kNumBars * 8 + 16 + 1024;   // barriers + tmem slot + alignment slack
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
    int vec_store;          // y is 16-byte aligned with ldy % 4 == 0: 128-bit stores
    int split_last;         // the tiles of the last, partial round are taken as two 128-row halves by two CTAs
    // kBF16Plain behind an ordered expansion launch (see expand_nk_ordered_kernel): the operands are still being
    // written when this kernel starts.  They become complete slice of K by slice of K; ready[q] counts the
    // expansion CTAs that have finished slice q of x and of W.
    // Column-sharded layer: the output tile goes into every GPU's full-width output (plain peer stores from the
    // epilogue), so the all-gather needs no pass of its own.  n_peers == 0: y only.
    float* peer_y[kMaxPeers];
    int n_peers;
    const uint32_t* ready;      // null: both operands are complete before the launch
    uint32_t ready_target;      // CTAs of the expansion launch
    int ready_part_kblocks;     // k-blocks per slice
};

__device__ __forceinline__ void report(uint32_t code, uint32_t detail) {
    atomicCAS(&g_status_gemm, 0u, (code << 24) | (detail & 0xFFFFFFu));
}

// Waits (bounded: about a second) until `target` CTAs of the expansion launch have counted themselves into *cnt,
// then orders the TMA loads that follow behind what those CTAs wrote.  false = gave up.
__device__ __forceinline__ bool wait_expanded(const uint32_t* cnt, uint32_t target) {
    for (uint32_t n = 0; n < (1u << 22); ++n) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
        if (v >= target) {
            fence_proxy_async_all();
            return true;
        }
        __nanosleep(200);
    }
    return false;
}

// Position in a ring of N slots and the mbarrier phase that goes with it, advanced by steps of
// `stride` without any division (these loops run in single threads that feed the tensor core).
template <int N>
struct Ring {
    int slot = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance(int stride = 1) {
        slot += stride;
        while (slot >= N) {
            slot -= N;
            phase ^= 1u;
        }
    }
};

// Walks this CTA's (tile, k-block) sequence: tiles blockIdx.x, +gridDim.x, ...; kb = 0..kblocks-1.
// When the last round is split, the CTA's item number `switch_at` is `last_tile` instead.
struct Walk {
    int64_t tile;
    int kb;
    uint32_t tcount = 0;   // tiles completed so far
    int64_t switch_at, last_tile;
    __device__ __forceinline__ Walk(int64_t first_tile, int64_t switch_at_ = -1, int64_t last_tile_ = 0)
        : tile(switch_at_ == 0 ? last_tile_ : first_tile), kb(0), switch_at(switch_at_), last_tile(last_tile_) {}
    __device__ __forceinline__ void advance(int stride, int kblocks, int64_t tile_stride) {
        kb += stride;
        while (kb >= kblocks) {
            kb -= kblocks;
            tile += tile_stride;
            ++tcount;
            if (static_cast<int64_t>(tcount) == switch_at) tile = last_tile;
        }
    }
};

// PEERS: the epilogue stores every tile into p.n_peers outputs (a column-sharded layer; a form of its own so that
// the single-output epilogue keeps its straight-line stores).
template <int MODE, bool PEERS = false>
__global__ void __launch_bounds__(Cfg<MODE>::kThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, Params p) {
    using C = Cfg<MODE>;
    constexpr int NA = C::kAStages, NB = C::kBStages, NR = C::kRawStages ? C::kRawStages : 1;
    extern __shared__ uint8_t smem_raw[];
    // aligned by pointer arithmetic on the shared array itself: a round trip through an integer would make the
    // compiler lose the address space and emit generic loads for every shared-memory access below
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBarOffset);
    uint64_t* a_full = bars;                 // [NA] A tile landed
    uint64_t* a_empty = a_full + NA;         // [NA] the MMAs reading it completed
    uint64_t* b_full = a_empty + NA;         // [NB] B tile ready (TMA landed, or dequant warps done)
    uint64_t* b_empty = b_full + NB;         // [NB] the MMAs reading it completed
    uint64_t* raw_full = b_empty + NB;       // [NR] packed nibbles landed (kBF16)
    uint64_t* raw_empty = raw_full + NR;     // [NR] packed nibbles are in registers (kBF16)
    uint64_t* tmem_full = raw_empty + NR;    // [2] (one used) both accumulators of the tile complete
    uint64_t* tmem_empty = tmem_full + 2;    // [2] (one used) both accumulators drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
    const int64_t tiles = m_tiles * n_tiles;
    const int kblocks = static_cast<int>((p.K + C::kBlockK - 1) / C::kBlockK);
    // this CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...; `it` counts its k-blocks across tiles
    int64_t my_tiles = (tiles > blockIdx.x) ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // Split last round (both operands by TMA only): when the tiles left for the last round fill at most half of the
    // CTAs, each of them goes to two CTAs as two 128-row halves (one accumulator each), and the round takes half the
    // time.  The CTA's items are then `rounds` whole tiles and, for the first 2 * last CTAs, one half tile.
    const int64_t rounds = tiles / gridDim.x, last = tiles - rounds * gridDim.x;
    const bool split = direct_b(MODE) && p.split_last && last > 0 && 2 * last <= gridDim.x;
    int64_t switch_at = -1, last_tile = 0;
    int half_row0 = 0;                     // row offset of this CTA's half inside the split tile
    if (split) {
        const bool mine = blockIdx.x < 2 * last;
        my_tiles = rounds + (mine ? 1 : 0);
        if (mine) {
            switch_at = rounds;
            last_tile = rounds * gridDim.x + blockIdx.x / 2;
            half_row0 = static_cast<int>(blockIdx.x & 1) * kHalfM;
        }
    }
    const int64_t total_its = my_tiles * kblocks;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NA; ++i) { mbar_init(&a_full[i], 1); mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < NB; ++i) { mbar_init(&b_full[i], direct_b(MODE) ? 1 : kDequantWarps); mbar_init(&b_empty[i], 1); }
        for (int i = 0; i < NR; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], kDequantWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(&tmem_full[i], 1); mbar_init(&tmem_empty[i], 4); }
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
        // ------------------------------- A producer ---------------------------------
        if (lane == 0) {
            tma_prefetch_descriptor(&map_a);
            Ring<NA> ra;
            Walk w(blockIdx.x, switch_at, last_tile);
            auto row0 = [&]() {       // a half tile loads the box that starts at its own 128 rows (the rest is not used)
                return static_cast<int32_t>((w.tile % m_tiles) * BM + (static_cast<int64_t>(w.tcount) == switch_at ? half_row0 : 0));
            };
            int32_t m0 = row0();
            uint32_t seen_tile = 0;
            int parts_seen = 0;                             // slices of K known to be complete (they fill in order)
            for (int64_t it = 0; it < total_its; ++it, ra.advance(), w.advance(1, kblocks, gridDim.x)) {
                if (w.tcount != seen_tile) { seen_tile = w.tcount; m0 = row0(); }
                if (MODE == kBF16Plain && p.ready != nullptr && w.kb >= parts_seen * p.ready_part_kblocks) {
                    const int q = w.kb / p.ready_part_kblocks;
                    if (!wait_expanded(p.ready + q, p.ready_target)) { report(kDevErrFullWait, 0x400000u | q); break; }
                    parts_seen = q + 1;
                }
                const int s = ra.slot;
                if (!mbar_wait(&a_empty[s], ra.phase ^ 1u)) { report(kDevErrEmptyWait, static_cast<uint32_t>(it)); break; }
                mbar_arrive_expect_tx(&a_full[s], kABytes);
                tma_load_2d(smem + C::kAOff + s * kABytes, &map_a, &a_full[s], w.kb * C::kBlockK, m0);
            }
        }
    } else if (warp == kBProducerWarp) {
        // ------------------------------- B / raw producer ---------------------------
        if (lane == 0) {
            tma_prefetch_descriptor(&map_b);
            Ring<NB> rb;
            Ring<NR> rr;
            Walk w(blockIdx.x, switch_at, last_tile);
            int32_t n0 = static_cast<int32_t>((w.tile / m_tiles) * BN);
            uint32_t seen_tile = 0;
            int parts_seen = 0;
            for (int64_t it = 0; it < total_its; ++it, rb.advance(), rr.advance(), w.advance(1, kblocks, gridDim.x)) {
                if (w.tcount != seen_tile) { seen_tile = w.tcount; n0 = static_cast<int32_t>((w.tile / m_tiles) * BN); }
                if (MODE == kBF16Plain && p.ready != nullptr && w.kb >= parts_seen * p.ready_part_kblocks) {
                    const int q = w.kb / p.ready_part_kblocks;
                    if (!wait_expanded(p.ready + q, p.ready_target)) { report(kDevErrFullWait, 0x410000u | q); break; }
                    parts_seen = q + 1;
                }
                if (direct_b(MODE)) {
                    const int s = rb.slot;
                    if (!mbar_wait(&b_empty[s], rb.phase ^ 1u)) { report(kDevErrEmptyWait, 0x800000u | static_cast<uint32_t>(it)); break; }
                    mbar_arrive_expect_tx(&b_full[s], kBBytes);
                    tma_load_2d(smem + C::kBOff + s * kBBytes, &map_b, &b_full[s], w.kb * C::kBlockK, n0);
                } else {
                    const int s = rr.slot;
                    if (!mbar_wait(&raw_empty[s], rr.phase ^ 1u)) { report(kDevErrEmptyWait, 0x800000u | static_cast<uint32_t>(it)); break; }
                    mbar_arrive_expect_tx(&raw_full[s], C::kRawStageBytes);
                    tma_load_2d(smem + C::kRawOff + s * C::kRawStageBytes, &map_b, &raw_full[s],
                                w.kb * (MODE == kBF16W8 ? C::kBlockK : C::kBlockK / 2), n0);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0) {
            const uint32_t idesc = (MODE == kI8) ? umma_idesc(2u, 1u, kHalfM, BN) : umma_idesc(1u, 1u, kHalfM, BN);
            Ring<NA> ra;
            Ring<NB> rb;
            Walk w(blockIdx.x, switch_at, last_tile);
            for (int64_t it = 0; it < total_its; ++it, ra.advance(), rb.advance(), w.advance(1, kblocks, gridDim.x)) {
                const int kb = w.kb;
                const uint32_t tcount = w.tcount;
                const int halves = static_cast<int64_t>(tcount) == switch_at ? 1 : 2;      // a half tile uses the first accumulator
                if (kb == 0) {
                    // both accumulators are reused by every tile: wait until the epilogue has drained them
                    if (!mbar_wait(&tmem_empty[0], (tcount & 1u) ^ 1u)) { report(kDevErrMmaWait, tcount); break; }
                    tcgen05_fence_after();
                }
                const int sa = ra.slot, sb = rb.slot;
                if (!mbar_wait(&a_full[sa], ra.phase)) { report(kDevErrFullWait, static_cast<uint32_t>(it)); break; }
                if (!mbar_wait(&b_full[sb], rb.phase)) { report(kDevErrFullWait, 0x800000u | static_cast<uint32_t>(it)); break; }
                tcgen05_fence_after();
                const uint64_t bdesc = umma_desc_sw128(smem_u32(smem + C::kBOff + sb * kBBytes));
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half >= halves) break;
                    const uint32_t tmem_d = tmem_base + half * BN;
                    const uint64_t adesc = umma_desc_sw128(smem_u32(smem + C::kAOff + sa * kABytes + half * (kHalfM * 128)));
#pragma unroll
                    for (int k = 0; k < C::kBlockK / C::kUmmaK; ++k) {
                        // +32 bytes per instruction inside the 128-byte swizzle row: +2 in the address field
                        if (MODE == kI8)
                            tcgen05_mma_i8(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                        else
                            tcgen05_mma_f16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                }
                tcgen05_commit(&a_empty[sa]);
                tcgen05_commit(&b_empty[sb]);
                if (kb == kblocks - 1) tcgen05_commit(&tmem_full[0]);
            }
        }
    } else if (warp >= kEpilogueWarp0 && warp < kEpilogueWarp0 + 4) {
        // ------------------------------- epilogue -----------------------------------
        const int quarter = warp & 3;
        uint32_t tcount = 0;
        bool alive = true;
        // Transposing epilogue.  TMEM hands lane i row i of a [32 x 32] block; stored like that each
        // store instruction would touch 32 different 128-byte lines.  The block goes through shared
        // memory instead, 16 rows at a time (16-byte chunk j of row i at position j ^ (i & 7):
        // conflict free both ways), and leaves with every instruction writing 4 complete 128-byte
        // row segments.
        uint8_t* stage_out = smem + C::kOutOff + (warp - kEpilogueWarp0) * 2048;
        const int cq = lane & 7, rq = lane >> 3;                  // after the transpose: columns 4cq..4cq+3, rows rq + 4i
        // weight scale applied per output column here (expanded INT8 codes: when the caller left it to the epilogue)
        const bool kScaleN = MODE == kI8 || MODE == kBF16W8 || (MODE == kBF16Plain && p.sw != nullptr);
        const float sw_all = (kScaleN && !p.sw_per_row) ? p.sw[0] : 1.0f;
        for (; static_cast<int64_t>(tcount) < my_tiles && alive; ++tcount) {
            const bool half_item = static_cast<int64_t>(tcount) == switch_at;
            const int64_t tile = half_item ? last_tile : blockIdx.x + static_cast<int64_t>(tcount) * gridDim.x;
            const int64_t m0 = (tile % m_tiles) * BM + (half_item ? half_row0 : 0), n0 = (tile / m_tiles) * BN;
            if (!mbar_wait(&tmem_full[0], tcount & 1u)) { report(kDevErrMmaWait, 0x800000u | tcount); alive = false; break; }
            tcgen05_fence_after();
            for (int half = 0; half < (half_item ? 1 : 2); ++half) {
                const int64_t mrow0 = m0 + half * kHalfM + quarter * 32;   // first row of this warp's block
                const int64_t m = mrow0 + lane;
                float sxm = 1.0f;
                if (MODE == kI8 && m < p.M) sxm = p.sx[m];
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(tmem_base + half * BN + c * 32 + (static_cast<uint32_t>(quarter * 32) << 16), v);
                    tmem_ld_wait();
                    const int64_t nb = n0 + c * 32;
                    if (nb >= p.N || mrow0 >= p.M) continue;          // uniform across the warp
                    if (MODE == kI8 && p.acc_out && m < p.M) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (nb + j < p.N) p.acc_out[m * p.N + nb + j] = static_cast<int32_t>(v[j]);
                    }
                    // column-dependent factors of this lane's 4 columns after the transpose
                    const int64_t n4 = nb + 4 * cq;
                    float swv[4] = {sw_all, sw_all, sw_all, sw_all}, bv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (n4 + e < p.N) {
                            if (kScaleN && p.sw_per_row) swv[e] = p.sw[n4 + e];
                            if (p.bias) bv[e] = p.bias[n4 + e];
                        }
                    }
                    const bool vec = p.vec_store && n4 + 4 <= p.N;
#pragma unroll
                    for (int part = 0; part < 2; ++part) {            // rows 0..15, then 16..31 of the block
                        __syncwarp();                                  // the previous part has been read out
                        if ((lane >> 4) == part) {
                            const int lr = lane & 15;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                float4 o;
                                if (MODE == kI8) {                 // row scale first: y = ((float)acc * sx[m]) * sw[n] + bias[n]
                                    o.x = __fmul_rn(static_cast<float>(static_cast<int32_t>(v[4 * j + 0])), sxm);
                                    o.y = __fmul_rn(static_cast<float>(static_cast<int32_t>(v[4 * j + 1])), sxm);
                                    o.z = __fmul_rn(static_cast<float>(static_cast<int32_t>(v[4 * j + 2])), sxm);
                                    o.w = __fmul_rn(static_cast<float>(static_cast<int32_t>(v[4 * j + 3])), sxm);
                                } else {
                                    o = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                    __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                                }
                                *reinterpret_cast<float4*>(stage_out + lr * 128 + ((j ^ (lr & 7)) << 4)) = o;
                            }
                        }
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int row = rq + 4 * i;                // 0..15 inside the part
                            const int64_t mm = mrow0 + part * 16 + row;
                            float4 o = *reinterpret_cast<const float4*>(stage_out + row * 128 + ((cq ^ (row & 7)) << 4));
                            if (kScaleN) {
                                o.x = __fmul_rn(o.x, swv[0]); o.y = __fmul_rn(o.y, swv[1]); o.z = __fmul_rn(o.z, swv[2]); o.w = __fmul_rn(o.w, swv[3]);
                            }
                            if (p.bias) {
                                o.x = __fadd_rn(o.x, bv[0]); o.y = __fadd_rn(o.y, bv[1]); o.z = __fadd_rn(o.z, bv[2]); o.w = __fadd_rn(o.w, bv[3]);
                            }
                            if constexpr (PEERS) {
                                if (mm < p.M) {
#pragma unroll 1
                                    for (int r = 0; r < p.n_peers; ++r) {
                                        float* dst = p.peer_y[r] + mm * p.ldy + n4;
                                        if (vec) {
                                            *reinterpret_cast<float4*>(dst) = o;
                                        } else {
                                            if (n4 + 0 < p.N) dst[0] = o.x;
                                            if (n4 + 1 < p.N) dst[1] = o.y;
                                            if (n4 + 2 < p.N) dst[2] = o.z;
                                            if (n4 + 3 < p.N) dst[3] = o.w;
                                        }
                                    }
                                }
                            } else {
                                if (mm < p.M) {
                                    float* dst = p.y + mm * p.ldy + n4;
                                    if (vec) {
                                        *reinterpret_cast<float4*>(dst) = o;
                                    } else {
                                        if (n4 + 0 < p.N) dst[0] = o.x;
                                        if (n4 + 1 < p.N) dst[1] = o.y;
                                        if (n4 + 2 < p.N) dst[2] = o.z;
                                        if (n4 + 3 < p.N) dst[3] = o.w;
                                    }
                                }
                            }
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[0]);
        }
    } else if (MODE == kBF16W8 && warp >= kDequantWarp0) {
        // ------------------------------- int8 -> bf16 --------------------------------
        // Thread (r, h) owns 32 consecutive codes of row r (32 bytes in, 64 bytes of bf16 out).  A code
        // c = 16*hi + lo (hi signed, lo unsigned nibble) is built exactly from two magic numbers:
        // 0x4300|lo = 128 + lo, 0x4300|(hi^8) = 136 + hi, t = fma(136 + hi, 16, -2304) = 16 hi - 128,
        // c = fma(128 + lo, 1, t).  The weight scale is applied in fp32 by the epilogue, so the only
        // rounding of this path is x -> bf16.  Bytes (0,2) and (1,3) of a word leave as pairs: inside
        // every 4 codes the order is k+{0,2,1,3}, which is the order the activations were stored in.
        const int tid = threadIdx.x - kDequantWarp0 * 32;
        const int r = tid >> 1, h = tid & 1;
        Ring<NR> rr;
        Ring<NB> rb;
        bool alive = true;
        for (int64_t it = 0; it < total_its && alive; ++it) {
            const int sr = rr.slot, sb = rb.slot;
            if (!mbar_wait(&raw_full[sr], rr.phase)) { report(kDevErrFullWait, 0x400000u | static_cast<uint32_t>(it)); alive = false; break; }
            const uint8_t* src = smem + C::kRawOff + sr * C::kRawStageBytes + r * 64 + h * 32;
            const uint4 w0 = *reinterpret_cast<const uint4*>(src);
            const uint4 w1 = *reinterpret_cast<const uint4*>(src + 16);
            // the slot is handed back only once the codes really are in registers
            const uint32_t landed = loads_landed(w0.x ^ w0.y ^ w0.z ^ w0.w ^ w1.x ^ w1.y ^ w1.z ^ w1.w);
            if (lane == 0) mbar_arrive_after(&raw_empty[sr], landed);
            if (!mbar_wait(&b_empty[sb], rb.phase ^ 1u)) { report(kDevErrEmptyWait, 0x400000u | static_cast<uint32_t>(it)); alive = false; break; }
            const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            uint8_t* brow = smem + C::kBOff + sb * kBBytes + r * 128;
#pragma unroll
            for (int w = 0; w < 4; ++w) {                           // output chunk w: words 2w and 2w+1
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t word = words[2 * w + (j >> 1)] >> (8 * (j & 1));     // bytes (0,2), then (1,3)
                    const uint32_t lo = (word & 0x000F000Fu) | 0x43004300u;            // 128 + lo
                    const uint32_t hi = ((word >> 4) & 0x000F000Fu) ^ 0x43084308u;     // 136 + hi
                    uint32_t t;
                    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(t) : "r"(hi), "r"(0x41804180u), "r"(0xC510C510u));   // 16 hi - 128
                    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[j]) : "r"(lo), "r"(0x3F803F80u), "r"(t));
                }
                *reinterpret_cast<uint4*>(brow + (((4 * h + w) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&b_full[sb]);
            rr.advance();
            rb.advance();
        }
    } else if (MODE == kBF16 && warp >= kDequantWarp0) {
        // ------------------------------- dequant ------------------------------------
        // Thread (r, h) owns half h (one 32-k group: 16 packed bytes in, 64 bytes of bf16 out) of row r of
        // the 256-row weight tile.  The group's scale is requested one k-block ahead so that its L2
        // latency is never waited for.
        const int tid = threadIdx.x - kDequantWarp0 * 32;
        const int r = tid >> 1, h = tid & 1;
        const int64_t sgroups = p.K / 32;
        Walk wn(blockIdx.x);                      // walks one k-block ahead, for the scale prefetch
        auto load_scale = [&](int64_t it, const Walk& w) {
            float sc = 0.0f;
            if (it < total_its) {
                const int64_t n = (w.tile / m_tiles) * BN + r;
                if (n < p.N) sc = __ldg(p.wscales + n * sgroups + 2 * w.kb + h);
            }
            return sc;
        };
        // scales are requested kAhead k-blocks before they are used (an L2 round trip is several
        // k-blocks long at full speed)
        constexpr int kAhead = 4;
        float scq[kAhead];
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
            scq[u] = load_scale(u, wn);
            wn.advance(1, kblocks, gridDim.x);
        }
        Ring<NR> rr;
        Ring<NB> rb;
        bool alive = true;
        for (int64_t it0 = 0; it0 < total_its && alive; it0 += kAhead) {
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int64_t it = it0 + u;
                if (it >= total_its || !alive) break;
                const float sc = scq[u];
                scq[u] = load_scale(it + kAhead, wn);
                wn.advance(1, kblocks, gridDim.x);
                const int sr = rr.slot, sb = rb.slot;
                if (!mbar_wait(&raw_full[sr], rr.phase)) { report(kDevErrFullWait, 0x400000u | static_cast<uint32_t>(it)); alive = false; break; }
                const uint4 w0 = *reinterpret_cast<const uint4*>(smem + C::kRawOff + sr * kRawBytes + r * 32 + h * 16);
                // make sure the load has returned before the slot is handed back to the TMA producer
                // the slot is handed back only once the nibbles really are in registers
                const uint32_t landed = loads_landed(w0.x ^ w0.y ^ w0.z ^ w0.w);
                if (lane == 0) mbar_arrive_after(&raw_empty[sr], landed);
                if (!mbar_wait(&b_empty[sb], rb.phase ^ 1u)) { report(kDevErrEmptyWait, 0x400000u | static_cast<uint32_t>(it)); alive = false; break; }
                const uint32_t words[4] = {w0.x, w0.y, w0.z, w0.w};
                const uint32_t sx2 = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(sc))) * 0x00010001u;
                uint8_t* brow = smem + C::kBOff + sb * kBBytes + r * 128;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t v = ((words[w] >> (4 * j)) & 0x000F000Fu) ^ 0x43084308u;  // 136 + code
                        // (v - 136) is exact in bf16, then one rounding for code * scale; both as fused
                        // multiply-adds, which the half-precision pipe executes natively
                        uint32_t c;
                        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(c) : "r"(v), "r"(0x3F803F80u), "r"(0xC308C308u));
                        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[j]) : "r"(c), "r"(sx2), "r"(0x80008000u));
                    }
                    // chunk (4h + w) of the row goes to chunk ((4h + w) ^ (r & 7)): the 128-byte swizzle the MMA expects
                    *reinterpret_cast<uint4*>(brow + (((4 * h + w) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&b_full[sb]);
                rr.advance();
                rb.advance();
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

// x fp32 [M,K] -> bf16 [M,K].  ORDER 0: inside every aligned group of 8 the order is k+{0,4,1,5,2,6,3,7},
// the order in which the dequant warps emit the 8 nibbles of a packed word.  ORDER 1 (INT8 weights):
// k+{0,2,1,3,4,6,5,7}.  ORDER 2: natural order (weights expanded to bf16 in global memory).
template <int ORDER>
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
        out[i] = ORDER == 1   ? make_uint4(pk(a.x, a.z), pk(a.y, a.w), pk(b.x, b.z), pk(b.y, b.w))
                 : ORDER == 0 ? make_uint4(pk(a.x, b.x), pk(a.y, b.y), pk(a.z, b.z), pk(a.w, b.w))
                              : make_uint4(pk(a.x, a.y), pk(a.z, a.w), pk(b.x, b.y), pk(b.z, b.w));
    }
}

// Weights stored [K,N] (the reference module's layout) -> bf16 [N,K] in global memory, dequantized with the
// reference's code * scale product in fp32 and rounded once.  A CTA transposes a tile of 64 k x 128 n through
// shared memory: a thread reads 32 consecutive n of one k (INT4: one 16-byte load = one quantization group,
// which runs along n in this layout; INT8: two loads), and the tile leaves as 128-byte rows of one n each.
// N % 32 == 0 (groups never straddle rows), K % 64 == 0.  INT8 scales: [1] or one per ROW OF THE STORED TENSOR,
// i.e. per k.
constexpr int kTrK = 64, kTrN = 128, kTrStride = kTrK + 8;      // bf16 elements per shared-memory row (16-byte multiple)
template <int BITS>
__global__ void __launch_bounds__(256) dequant_kn_to_nk_bf16_kernel(const uint8_t* __restrict__ wq, const float* __restrict__ scales,
                                                                   int per_row, int64_t group, int64_t K, int64_t N,
                                                                   __nv_bfloat16* __restrict__ out) {
    __shared__ __align__(16) __nv_bfloat16 tile[kTrN * kTrStride];
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kTrN, k0 = static_cast<int64_t>(blockIdx.y) * kTrK;
    const int kk = threadIdx.x >> 2, nq = threadIdx.x & 3;
    const int64_t k = k0 + kk, n = n0 + 32 * nq;
    if (n < N) {        // K % 64 == 0: k is always in range
        const int64_t e = k * N + n;                                  // flat element index of the first of 32
        if (BITS == 4) {
            const uint4 w = *reinterpret_cast<const uint4*>(wq + e / 2);
            const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float sc = scales[(e + 8 * i) / group];           // group % 8 == 0: a word never straddles groups
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int code = static_cast<int>(words[i] << (28 - 4 * j)) >> 28;      // nibble j, sign-extended
                    tile[(32 * nq + 8 * i + j) * kTrStride + kk] = __float2bfloat16_rn(__fmul_rn(static_cast<float>(code), sc));
                }
            }
        } else {
            const float sc = per_row ? scales[k] : scales[0];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 w = *reinterpret_cast<const uint4*>(wq + e + 16 * h);
                const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int code = static_cast<int>(words[i] << (24 - 8 * j)) >> 24;
                        tile[(32 * nq + 16 * h + 4 * i + j) * kTrStride + kk] =
                            __float2bfloat16_rn(__fmul_rn(static_cast<float>(code), sc));
                    }
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = threadIdx.x + 256 * i, r = idx >> 3, c = idx & 7;
        if (n0 + r < N)
            *reinterpret_cast<uint4*>(out + (n0 + r) * K + k0 + 8 * c) = *reinterpret_cast<const uint4*>(tile + r * kTrStride + 8 * c);
    }
}

// Weights stored [N,K] -> bf16 [N,K] in global memory, eight elements per step (one packed word, or eight code
// bytes).  INT4: code * scale in fp32, rounded once.  INT8: the codes themselves (exact in bf16); their scale (per
// tensor or per output row) is applied by the GEMM's epilogue in fp32.  The same launch converts the activations
// (x fp32 [M,K] -> bf16, natural order), and the GEMM starts while it runs: the grid is one resident wave that
// leaves room for the GEMM's CTA on every SM, and the work is ordered by `parts` equal slices of K: slice 0 of x,
// slice 0 of W, slice 1 of x, ...  ready[q] counts the CTAs that have finished slice q of both; a CTA counts
// itself after a fence behind all of its stores, so a reader that sees gridDim.x in ready[q] (acquire load) may
// read slices 0 .. q.  The counters must be zero at launch.  Indices are 32-bit: the host takes one slice when
// the weight has 2^31 steps or more.
constexpr int kExpandCtasPerSm = 2;
constexpr int kReadyParts = 8;            // at most
constexpr size_t kReadyBytes = 256;       // reserved behind the expanded weight for the counters
template <int BITS>
__global__ void __maxnreg__(48)            // per SM quarter: 4 of these warps (4 x 48 x 32) beside 2 of the GEMM (2 x 160 x 32)
expand_nk_ordered_kernel(const uint8_t* __restrict__ wq, const float* __restrict__ scales, uint32_t group, uint32_t N, uint32_t K,
                         uint32_t parts, uint4* __restrict__ out, const float* __restrict__ x, uint32_t M, uint4* __restrict__ xout,
                         uint32_t* __restrict__ ready) {
    pdl_launch_dependents();             // the GEMM behind this launch may take its places now; it waits on `ready`
    auto pk = [](float lo, float hi) {
        return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
               (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
    };
    const uint32_t first = blockIdx.x * 256u + threadIdx.x, stride = gridDim.x * 256u;
    const uint32_t row = K / 8, slice = row / parts;                     // steps per row / per row and slice (x and W alike)
    auto step_of = [&](uint32_t v, uint32_t part) {                      // v-th step of the slice -> index in the whole tensor
        const uint32_t r = v / slice;
        return r * row + part * slice + (v - r * slice);
    };
    auto expand = [&](uint32_t i, uint32_t lo, uint32_t hi, float sc) {
        float v[8];
        if (BITS == 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(static_cast<float>(static_cast<int>(lo << (28 - 4 * j)) >> 28), sc);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] = static_cast<float>(static_cast<int>(lo << (24 - 8 * j)) >> 24);
                v[4 + j] = static_cast<float>(static_cast<int>(hi << (24 - 8 * j)) >> 24);
            }
        }
        out[i] = make_uint4(pk(v[0], v[1]), pk(v[2], v[3]), pk(v[4], v[5]), pk(v[6], v[7]));
    };
    auto signal = [&](uint32_t part) {                                   // called by whole CTAs only
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) atomicAdd(ready + part, 1u);
    };
    for (uint32_t part = 0; part < parts; ++part) {
        const uint32_t xtotal = M * slice;
        for (uint32_t v0 = blockIdx.x * 256u; v0 < xtotal; v0 += 2 * stride) {      // two chunks in flight per thread;
            const uint32_t v = v0 + threadIdx.x;                                    // the trip count is the CTA's
            const bool one = v < xtotal, two = v + stride < xtotal;
            const uint32_t j0 = step_of(one ? v : 0, part), j1 = two ? step_of(v + stride, part) : j0;
            const float4 a0 = reinterpret_cast<const float4*>(x)[2 * static_cast<size_t>(j0)], b0 = reinterpret_cast<const float4*>(x)[2 * static_cast<size_t>(j0) + 1];
            const float4 a1 = reinterpret_cast<const float4*>(x)[2 * static_cast<size_t>(j1)], b1 = reinterpret_cast<const float4*>(x)[2 * static_cast<size_t>(j1) + 1];
            if (one) xout[j0] = make_uint4(pk(a0.x, a0.y), pk(a0.z, a0.w), pk(b0.x, b0.y), pk(b0.z, b0.w));
            if (two) xout[j1] = make_uint4(pk(a1.x, a1.y), pk(a1.z, a1.w), pk(b1.x, b1.y), pk(b1.z, b1.w));
        }
        // Four words and their scales per thread and pass, and the loads of the next pass are issued before the
        // current one is converted: with two CTAs per SM the loads have to overlap the arithmetic inside a thread.
        const uint32_t total = N * slice;
        uint32_t i[4], in[4];
        uint32_t lo[4], hi[4], lon[4], hin[4];
        float sc[4], scn[4];
        auto fetch = [&](uint32_t v, uint32_t (&ii)[4], uint32_t (&l)[4], uint32_t (&h)[4], float (&f)[4]) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t vq = v + q * stride;
                ii[q] = step_of(vq < total ? vq : v, part);
                if (BITS == 4) {
                    l[q] = reinterpret_cast<const uint32_t*>(wq)[ii[q]];
                    h[q] = 0;
                    f[q] = scales[ii[q] / (group / 8)];                    // group % 8 == 0: a word never straddles groups
                } else {
                    const uint2 w = reinterpret_cast<const uint2*>(wq)[ii[q]];
                    l[q] = w.x;
                    h[q] = w.y;
                    f[q] = 1.0f;
                }
            }
        };
        if (first < total) fetch(first, i, lo, hi, sc);
        for (uint32_t v = first; v < total; v += 4 * stride) {
            const uint32_t vn = v + 4 * stride;
            if (vn < total) fetch(vn, in, lon, hin, scn);
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (q == 0 || v + q * stride < total) expand(i[q], lo[q], hi[q], sc[q]);
#pragma unroll
            for (int q = 0; q < 4; ++q) { i[q] = in[q]; lo[q] = lon[q]; hi[q] = hin[q]; sc[q] = scn[q]; }
        }
        signal(part);
    }
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <int MODE>
int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, Params p, cudaStream_t stream, bool overlap = false) {
    using C = Cfg<MODE>;
    p.vec_store = (aligned(p.y, 16) && (p.ldy % 4) == 0) ? 1 : 0;
    for (int r = 0; r < p.n_peers; ++r)
        if (!aligned(p.peer_y[r], 16)) p.vec_store = 0;
    const int64_t tiles = ceil_div(p.M, BM) * ceil_div(p.N, BN);
    int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    p.split_last = 0;
    if (direct_b(MODE)) {
        // the tiles of the last, partial round as half tiles on twice as many CTAs, where they fit
        const int64_t sms = sm_count(), last = tiles % sms;
        if (last > 0 && 2 * last <= sms) {
            p.split_last = 1;
            if (tiles < sms) grid = static_cast<int>(2 * tiles);
        }
    }
    // overlap: the kernel may start while the expansion launch in front of it is still running (it waits on p.ready)
    if (p.n_peers > 0) {
        if (MODE != kBF16Plain) {
            set_error("the fused all-gather of the tensor-core path needs the scratch for the expanded weight");
            return SGQ_ERR_WORKSPACE;
        }
        static SmemOptIn optin_peers;
        SGQ_CUDA_TRY(optin_peers.ensure(linear_tc_kernel<kBF16Plain, true>, Cfg<kBF16Plain>::kSmemBytes));
        SGQ_CUDA_TRY(launch_kernel(linear_tc_kernel<kBF16Plain, true>, dim3(static_cast<unsigned>(grid)), dim3(Cfg<kBF16Plain>::kThreads),
                                   Cfg<kBF16Plain>::kSmemBytes, stream, overlap, ma, mb, p));
        return SGQ_OK;
    }
    static SmemOptIn optin;   // one per MODE instantiation
    SGQ_CUDA_TRY(optin.ensure(linear_tc_kernel<MODE>, C::kSmemBytes));
    SGQ_CUDA_TRY(launch_kernel(linear_tc_kernel<MODE>, dim3(static_cast<unsigned>(grid)), dim3(C::kThreads), C::kSmemBytes, stream,
                               overlap, ma, mb, p));
    return SGQ_OK;
}

}  // namespace

bool tc_bf16_supported(int bits, int64_t M, int64_t K, int64_t N, int layout, int64_t group) {
    // INT4: any group that is a multiple of 8 (the weight is expanded word by word); 32 also has the form that
    // dequantizes in shared memory
    if (!(((bits == 4 && group >= 8 && (group % 8) == 0) || bits == 8) && M >= 1 && N >= 1 && K >= 64 && (K % 64) == 0 &&
          M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31)))
        return false;
    // [K,N]: quantization groups run along N and must not straddle rows of the stored tensor
    return layout == SGQ_LAYOUT_NK || (layout == SGQ_LAYOUT_KN && (N % 32) == 0);
}

// bf16 activations plus the whole weight expanded to bf16 [N,K]: the faster form (a GEMM whose operands both
// arrive by TMA), and the only one for weights stored [K,N]
size_t tc_bf16_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout) {
    (void)bits; (void)layout;
    return round_up(static_cast<size_t>(M) * static_cast<size_t>(K) * 2, 256) +
           round_up(static_cast<size_t>(N) * static_cast<size_t>(K) * 2, 256) + kReadyBytes;
}

// the least the path runs with: weights stored [N,K] can be dequantized tile by tile in shared memory instead
size_t tc_bf16_min_workspace_bytes(int bits, int64_t M, int64_t K, int64_t N, int layout, int64_t group) {
    if (layout == SGQ_LAYOUT_KN || (bits == 4 && group != 32)) return tc_bf16_workspace_bytes(bits, M, K, N, layout);
    return round_up(static_cast<size_t>(M) * static_cast<size_t>(K) * 2, 256);
}

int launch_linear_tc_bf16(const LinearArgs& a) {
    if (!tc_bf16_supported(a.bits, a.M, a.K, a.N, a.layout, a.group)) {
        set_error("bf16 tensor-core path needs INT4 (group a multiple of 8) or INT8 weights, K%%64==0, and N%%32==0 when stored [K,N]");
        return SGQ_ERR_UNSUPPORTED;
    }
    if (!aligned(a.x, 16) || !aligned(a.wq, 16) || !aligned(a.scales, 8)) {
        set_error("bf16 tensor-core path needs 16-byte aligned x and packed weights, 8-byte aligned scales");
        return SGQ_ERR_ALIGNMENT;
    }
    const size_t need = tc_bf16_min_workspace_bytes(a.bits, a.M, a.K, a.N, a.layout, a.group);
    const bool expand = a.workspace && a.workspace_bytes >= tc_bf16_workspace_bytes(a.bits, a.M, a.K, a.N, a.layout);
    if (!a.workspace || a.workspace_bytes < need) {
        set_error("bf16 tensor-core path needs %zu workspace bytes, got %zu", need, a.workspace ? a.workspace_bytes : 0);
        return SGQ_ERR_WORKSPACE;
    }
    const int64_t chunks = a.M * a.K / 8;
    int64_t blocks = ceil_div(chunks, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    const int cgrid = static_cast<int>(blocks < cap ? blocks : cap);
    if (!(expand && a.layout == SGQ_LAYOUT_NK)) {       // (that form converts x in its weight-expansion launch below)
        if (expand)
            convert_x_bf16_kernel<2><<<cgrid, 256, 0, a.stream>>>(a.x, static_cast<uint4*>(a.workspace), chunks);
        else if (a.bits == 8)
            convert_x_bf16_kernel<1><<<cgrid, 256, 0, a.stream>>>(a.x, static_cast<uint4*>(a.workspace), chunks);
        else
            convert_x_bf16_kernel<0><<<cgrid, 256, 0, a.stream>>>(a.x, static_cast<uint4*>(a.workspace), chunks);
        SGQ_LAUNCH_CHECK("convert_x_bf16_kernel");
    }

    CUtensorMap ma, mb;
    if (!make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.workspace, static_cast<uint64_t>(a.K),
                            static_cast<uint64_t>(a.M), static_cast<uint64_t>(a.K) * 2, 64, BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return SGQ_ERR_CUDA;
    Params p{};
    p.bias = a.bias; p.y = a.y; p.ldy = a.ldy; p.M = a.M; p.N = a.N; p.K = a.K;
    p.n_peers = a.peers.n;
    for (int r = 0; r < a.peers.n; ++r) p.peer_y[r] = a.peers.p[r];
    if (expand) {
        // expand the stored weight to bf16 [N,K] behind the activations in the workspace, then a GEMM whose
        // operands both arrive by TMA
        __nv_bfloat16* wt = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(a.workspace) +
                                                             round_up(static_cast<size_t>(a.M) * static_cast<size_t>(a.K) * 2, 256));
        if (a.layout == SGQ_LAYOUT_KN) {
            const dim3 tgrid(static_cast<unsigned>(ceil_div(a.N, kTrN)), static_cast<unsigned>(a.K / kTrK));
            if (a.bits == 4)
                dequant_kn_to_nk_bf16_kernel<4><<<tgrid, 256, 0, a.stream>>>(static_cast<const uint8_t*>(a.wq), a.scales, 0, a.group, a.K, a.N, wt);
            else
                dequant_kn_to_nk_bf16_kernel<8><<<tgrid, 256, 0, a.stream>>>(static_cast<const uint8_t*>(a.wq), a.scales,
                                                                            a.scheme == SGQ_PER_ROW ? 1 : 0, 32, a.K, a.N, wt);
            SGQ_LAUNCH_CHECK("dequant_kn_to_nk_bf16_kernel");
        } else {
            // One resident wave converts x and the weight slice of K by slice of K, counting finished slices into
            // `ready`; the GEMM is launched behind it with programmatic serialization and starts on the first slice
            // while the rest is still being expanded.
            const int64_t wsteps = a.N * a.K / 8;
            const int64_t most = wsteps > chunks ? wsteps : chunks;
            // (without overlapped launches the GEMM starts behind the whole expansion anyway: then the grid fills the
            // machine and the weight is one slice)
            // Beside the GEMM only while the register budget of an SM quarter holds: 2 GEMM warps of at most 160
            // registers a thread next to 4 expansion warps of 48 (16384 in all); a compiler that needs more for
            // the GEMM gets the serial form instead of a silent loss of the overlap.
            static const bool fits = [] {
                cudaFuncAttributes fa{};
                return cudaFuncGetAttributes(&fa, linear_tc_kernel<kBF16Plain>) == cudaSuccess && fa.numRegs <= 160;
            }();
            const bool beside = stream_overlap_enabled() && fits && a.peers.n == 0;
            const int64_t wave = static_cast<int64_t>(sm_count()) * (beside ? kExpandCtasPerSm : 16);
            const int egrid = static_cast<int>(ceil_div(most, 1024) < wave ? ceil_div(most, 1024) : wave);
            const int64_t kblocks = a.K / 64;
            int parts = beside ? kReadyParts : 1;
            while (kblocks % parts) parts /= 2;
            if (most >= (1LL << 31) - 4LL * egrid * 256) {
                set_error("bf16 tensor-core path: more than 2^31 expansion steps");
                return SGQ_ERR_UNSUPPORTED;
            }
            uint32_t* ready = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(wt) +
                                                          round_up(static_cast<size_t>(a.N) * static_cast<size_t>(a.K) * 2, 256));
            SGQ_CUDA_TRY(cudaMemsetAsync(ready, 0, kReadyBytes, a.stream));
            const uint32_t N32 = static_cast<uint32_t>(a.N), K32 = static_cast<uint32_t>(a.K), M32 = static_cast<uint32_t>(a.M);
            if (stream_overlap_enabled())     // the GEMM's CTA can only join an SM that runs under the same memory split
                prefer_max_shared(a.bits == 4 ? reinterpret_cast<const void*>(expand_nk_ordered_kernel<4>)
                                              : reinterpret_cast<const void*>(expand_nk_ordered_kernel<8>));
            if (a.bits == 4)
                expand_nk_ordered_kernel<4><<<egrid, 256, 0, a.stream>>>(static_cast<const uint8_t*>(a.wq), a.scales,
                                                                        static_cast<uint32_t>(a.group), N32, K32, parts,
                                                                        reinterpret_cast<uint4*>(wt), a.x, M32,
                                                                        static_cast<uint4*>(a.workspace), ready);
            else
                expand_nk_ordered_kernel<8><<<egrid, 256, 0, a.stream>>>(static_cast<const uint8_t*>(a.wq), a.scales, 32u, N32, K32, parts,
                                                                        reinterpret_cast<uint4*>(wt), a.x, M32,
                                                                        static_cast<uint4*>(a.workspace), ready);
            SGQ_LAUNCH_CHECK("expand_nk_ordered_kernel");
            if (a.bits == 8) {          // codes are exact in bf16: their scale goes to the epilogue
                p.sw = a.scales;
                p.sw_per_row = (a.scheme == SGQ_PER_ROW) ? 1 : 0;
            }
            p.ready = ready;
            p.ready_target = static_cast<uint32_t>(egrid);
            p.ready_part_kblocks = static_cast<int>(kblocks / parts);
        }
        if (!make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, wt, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N),
                                static_cast<uint64_t>(a.K) * 2, 64, BN, CU_TENSOR_MAP_SWIZZLE_128B))
            return SGQ_ERR_CUDA;
        return launch_tc<kBF16Plain>(ma, mb, p, a.stream, p.ready != nullptr && stream_overlap_enabled());
    }
    if (a.bits == 8) {
        if (!make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.N),
                                static_cast<uint64_t>(a.K), 64, BN, CU_TENSOR_MAP_SWIZZLE_NONE))
            return SGQ_ERR_CUDA;
        p.sw = a.scales;
        p.sw_per_row = (a.scheme == SGQ_PER_ROW) ? 1 : 0;
        return launch_tc<kBF16W8>(ma, mb, p, a.stream);
    }
    if (!make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.wq, static_cast<uint64_t>(a.K / 2),
                            static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 2), 32, BN, CU_TENSOR_MAP_SWIZZLE_NONE))
        return SGQ_ERR_CUDA;
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
