// Conversion of fp32 activation rows into the decode kernels' operand format ("prepared
// activations"): group-scaled fixed point, split into balanced base-256 int8 digits that are laid
// out as mma.sync B fragments.  Shared by the decode kernels (conversion inside their CTAs), the
// stand-alone conversion kernels, and the decoder operators that emit this format directly.
//
// Arithmetic.  Every 32 consecutive k of a row (the span of one INT4 weight group) have their own
// scale: with gmax the group's absmax, q = rint(x * (Q / gmax)), Q = 8355000, and
// q = d0 + 256 d1 + 65536 d2 with every digit in [-128, 127] (24 bits below the group's absmax:
// finer than the rounding of the reference's own fp32 chain).  The kernels form exact integer dot
// products per digit and group and multiply them by gmax / Q in fp32.
//   Batches of one or two rows always use all three digits.  Larger batches keep the low digit d0
// in separate MMA column sets and skip them, group by group, where the digit cannot matter: a
// group is flagged (its low digit is used) when one value dominates it, 32 gmax^2 > 16 sum x^2;
// in every other group gmax < 4 rms(group), so dropping d0 (which, the digits being balanced, is a
// round-to-nearest to 16 bits) costs at most 1.53e-5 gmax < 6.2e-5 rms(group) per activation.
// Hence no activation distribution can push the error of an output beyond ~1e-4 of the output's
// own scale: a few huge channels cost the rest of the row nothing.  A group whose absmax is NaN or
// Inf gets a NaN scale (the output row becomes NaN); a group whose absmax is below 1e-30
// contributes zero.
//
// Layout of a prepared buffer for M rows of K values (K % 32 == 0), five parts one after the other:
//   main digit planes  [group K/32][set pair][fragment lane 32][sets of the pair x 8 bytes]
//   low digit planes   the same for the low sets (three rows or more)
//   main scales        [group K/32][t 4][set][2] fp32: the scales that belong to columns 2t and 2t+1
//                      of the set (a lane of an MMA holds exactly these two accumulator columns)
//   low scales         the same for the low sets
//   flags              [group K/32][16] bytes (three rows or more): row m's low digit is needed
// The kernels keep the main parts and the flags in shared memory and fetch low digits and scales
// from wherever the buffer lies, for the flagged groups only.
// A "set" is one group of eight B-fragment columns (one MMA).  Column of digit j of row m:
//   one row     set 0, column 2j (only even columns carry data; the kernels skip the odd accumulators)
//   two rows    set 0, column 3m + j
//   more rows   d1, d2: column 2m + j - 1 counted through the `nmain` main sets (a row owns columns 2t, 2t+1
//               of its set; the scales of these sets carry a factor 256); d0: column m counted through
//               the `nlow` low sets.
// Sets are stored in pairs so that a lane fetches the fragments of two sets with one 128-bit load; a
// last unpaired set uses 8 bytes per lane.
#pragma once

#include "sgq_common.cuh"

namespace sgq {

constexpr int kPreparedMaxM = 16;

// The accumulator of an integer MMA starts at kMagicBits: the int32 result, read as fp32 bits,
// then equals 12582912.0f + S for the exact integer sum S (|S| < 2^22), so the kernels get S as a
// float with one full-rate subtraction instead of an int-to-float conversion.
constexpr int kMagicBits = 0x4B400000;
constexpr float kMagicF = 12582912.0f;

constexpr float kDigitRange = 8355000.0f;    // |q| <= 8355711 = 127 * 65793 must hold after rounding

struct PreparedLayout {
    int mode;                  // 0: one row, 1: two rows, 2: three rows or more (main and low sets)
    int nmain, nlow;
    int ndigits_out;           // digits a kernel recombines per output: 3, or 2 when the low digit is folded in before
    size_t off_dlow, off_smain, off_slow, off_flags, bytes;    // part offsets (the main digit planes start at 0)
};

inline PreparedLayout prepared_layout(int64_t M, int64_t K) {
    PreparedLayout L;
    L.mode = (M <= 1) ? 0 : (M == 2 ? 1 : 2);
    L.nmain = L.mode == 2 ? static_cast<int>((M + 3) / 4) : 1;
    L.nlow = L.mode == 2 ? static_cast<int>((M + 7) / 8) : 0;
    L.ndigits_out = L.mode == 2 ? 2 : 3;
    const size_t groups = static_cast<size_t>(K / 32);
    L.off_dlow = groups * L.nmain * 256;
    L.off_smain = L.off_dlow + groups * L.nlow * 256;
    L.off_slow = L.off_smain + groups * L.nmain * 32;
    L.off_flags = L.off_slow + groups * L.nlow * 32;
    L.bytes = L.off_flags + (L.mode == 2 ? groups * 16 : 0);
    return L;
}

// Main set and column of digit j of row m (three rows or more: j = 1, 2 only; the low digit j = 0 sits in
// column m & 7 of low set m >> 3).
__host__ __device__ inline void digit_slot(int mode, int m, int j, int* set, int* cc) {
    if (mode == 0) {
        *set = 0;
        *cc = 2 * j;
    } else if (mode == 1) {
        *set = 0;
        *cc = 3 * m + j;
    } else {
        const int cm = 2 * m + j - 1;
        *set = cm >> 3;
        *cc = cm & 7;
    }
}

#ifdef __CUDACC__

// Byte offset of the 8 fragment bytes of (group, set, fragment lane) inside the digit planes.
__host__ __device__ __forceinline__ size_t plane_offset(size_t group, int nsets, int set, int frag_lane) {
    const int pair = set >> 1;
    const bool full = 2 * pair + 1 < nsets;
    return group * static_cast<size_t>(nsets) * 256 + static_cast<size_t>(pair) * 512 +
           (full ? frag_lane * 16 + (set & 1) * 8 : frag_lane * 8);
}

// Balanced base-256 digits of q: q = d0 + 256 d1 + 65536 d2 with every d in [-128, 127].
// Adding 128 to each digit makes them unsigned bytes without carries between byte positions, so
// the bytes of (q + 0x808080) are d_j + 128 and one more XOR turns them back into signed bytes.
__device__ __forceinline__ uint32_t digit_bytes(int q) {
    return (static_cast<uint32_t>(q) + 0x00808080u) ^ 0x00808080u;
}
// byte j of four words -> one word (a.j, b.j, c.j, d.j)
__device__ __forceinline__ uint32_t gather_byte(uint32_t a, uint32_t b, uint32_t c, uint32_t d, int j) {
    const uint32_t ab = __byte_perm(a, b, 0x0040 + 0x11 * j);   // (a.j, b.j, -, -)
    const uint32_t cd = __byte_perm(c, d, 0x0040 + 0x11 * j);
    return __byte_perm(ab, cd, 0x5410);
}

// Order of the k positions inside a 32-k group:
//   kOrderNibble  fragment lane t holds k = 8t + {0,2,4,6} (b0) and 8t + {1,3,5,7} (b1): the order
//                 in which the INT4 kernel's two mask operations deliver the nibbles of a word;
//   kOrderNatural fragment lane t holds k = 4t + {0..3} (b0) and 16 + 4t + {0..3} (b1): int8 codes
//                 as they lie in memory.
enum { kOrderNibble = 0, kOrderNatural = 1 };

// Where the parts of a prepared buffer of `groups` 32-k groups start.
struct PreparedParts {
    uint8_t* dmain;
    uint8_t* dlow;
    float* smain;
    float* slow;
    uint8_t* flags;
};
__host__ __device__ inline PreparedParts prepared_parts(uint8_t* base, size_t groups, int nmain, int nlow) {
    PreparedParts p;
    p.dmain = base;
    p.dlow = p.dmain + groups * nmain * 256;
    p.smain = reinterpret_cast<float*>(p.dlow + groups * nlow * 256);
    p.slow = p.smain + groups * nmain * 8;
    p.flags = reinterpret_cast<uint8_t*>(p.slow + groups * nlow * 8);
    return p;
}

// Converts 256 consecutive k (eight 32-k groups, the first being group `group0`) of row m of an
// M-row batch.  Must be called by all 32 lanes of a warp together, lane l holding the 8 consecutive
// activations k = 32 * group0 + 8 l .. + 7 in v: four neighbouring lanes share a group.
// `scale_mul` is folded into the stored scales (the INT4 kernel feeds its codes to the tensor core
// as 16 * code and passes 1/16).  A lane with store == false (beyond the end of a row) passes zeros
// and writes nothing.
// BLOCK = 4: four consecutive groups (128 k, 16 lanes) share one scale and one low-digit flag, both stored with
// every group of the four (the INT8 decode kernel, which has no per-group weight scale, then adds the exact sums
// of the four groups in int32 and scales once); the rule for the low digit is the same with the block in the
// place of the group: it is dropped where the block's absmax is below 4 rms(block).
template <int ORDER, int BLOCK = 1>
__device__ __forceinline__ void convert_groups(const float (&v)[8], int m, int M, size_t group0, int mode, int nmain, int nlow,
                                               float scale_mul, const PreparedParts& pp, bool store = true) {
    static_assert(BLOCK == 1 || BLOCK == 4, "scale blocks of one or four groups");
    const int lane = threadIdx.x & 31;
    uint32_t mb = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t b = __float_as_uint(v[j]) & 0x7FFFFFFFu;    // |x| as bits: orders like the value, NaN above Inf
        mb = b > mb ? b : mb;
    }
    {
        uint32_t o = __shfl_xor_sync(0xffffffffu, mb, 1);
        mb = o > mb ? o : mb;
        o = __shfl_xor_sync(0xffffffffu, mb, 2);
        mb = o > mb ? o : mb;
        if (BLOCK == 4) {
            o = __shfl_xor_sync(0xffffffffu, mb, 4);
            mb = o > mb ? o : mb;
            o = __shfl_xor_sync(0xffffffffu, mb, 8);
            mb = o > mb ? o : mb;
        }
    }
    const float gmax = __uint_as_float(mb);
    float P, sx;
    if (mb >= 0x7F800000u) {            // NaN or Inf somewhere in the group: the output row becomes NaN
        P = 0.0f;
        sx = __uint_as_float(0x7FC00000u);
    } else if (gmax < 1e-30f) {         // zero (or vanishing) group
        P = 0.0f;
        sx = 0.0f;
    } else {
        P = __fdiv_rn(kDigitRange, gmax);
        sx = __fmul_rn(__fdiv_rn(gmax, kDigitRange), scale_mul);
    }
    uint32_t db[8];
    float sq = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int q = __float2int_rn(__fmul_rn(v[j], P));
        const float qf = static_cast<float>(q);
        sq = __fmaf_rn(qf, qf, sq);
        db[j] = digit_bytes(q);
    }
    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    if (BLOCK == 4) {
        sq += __shfl_xor_sync(0xffffffffu, sq, 4);
        sq += __shfl_xor_sync(0xffffffffu, sq, 8);
    }
    if (!store) return;
    const size_t group = group0 + (lane >> 2);
    const int q4 = lane & 3;            // which quarter of the group this lane holds
    if (mode == 2 && q4 == 0) {
        // one value dominates the group (32 gmax^2 > 16 sum x^2, in units of the scaled integers): keep the low digit
        pp.flags[group * 16 + m] = (P != 0.0f && sq < (2.0f * BLOCK) * kDigitRange * kDigitRange) ? 1 : 0;
        if (m == 0)
            for (int z = M; z < 16; ++z) pp.flags[group * 16 + z] = 0;     // rows this batch does not have
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        int set, cc, nsets;
        uint8_t* digits;
        if (mode == 2 && j == 0) {          // the low digit: its own sets, its own parts of the buffer
            set = m >> 3;
            cc = m & 7;
            nsets = nlow;
            digits = pp.dlow;
            if (q4 == 0) pp.slow[((group * 4 + (cc >> 1)) * nsets + set) * 2 + (cc & 1)] = sx;
        } else {
            digit_slot(mode, m, j, &set, &cc);
            nsets = nmain;
            digits = pp.dmain;
            if (q4 == 0) pp.smain[((group * 4 + (cc >> 1)) * nsets + set) * 2 + (cc & 1)] = (mode == 2) ? sx * 256.0f : sx;
        }
        if (ORDER == kOrderNibble) {
            const uint32_t b0 = gather_byte(db[0], db[2], db[4], db[6], j);
            const uint32_t b1 = gather_byte(db[1], db[3], db[5], db[7], j);
            *reinterpret_cast<uint2*>(digits + plane_offset(group, nsets, set, cc * 4 + q4)) = make_uint2(b0, b1);
        } else {
            // k = 8q .. 8q+7: the first four go to fragment lane t0 = 2 (q & 1), the next four to t0 + 1,
            // in b0 when k < 16 and in b1 otherwise
            const int t0 = 2 * (q4 & 1), half = q4 >> 1;
            *reinterpret_cast<uint32_t*>(digits + plane_offset(group, nsets, set, cc * 4 + t0) + half * 4) =
                gather_byte(db[0], db[1], db[2], db[3], j);
            *reinterpret_cast<uint32_t*>(digits + plane_offset(group, nsets, set, cc * 4 + t0 + 1) + half * 4) =
                gather_byte(db[4], db[5], db[6], db[7], j);
        }
    }
}

// Block-wide conversion of one row (row index m of an M-row batch) whose K values lie at x_row in
// global memory (values this thread block wrote itself are visible after the caller's
// __syncthreads).  THREADS must be a multiple of 32 and K a multiple of 256, so that whole warps
// take part in every conversion call.  `planes` is the prepared buffer of the INT4 decode kernel.
template <int THREADS>
__device__ __forceinline__ void prepare_row_block(const float* x_row, int m, int M, int64_t K, int mode, int nmain, int nlow,
                                                  uint8_t* __restrict__ planes) {
    const int chunks = static_cast<int>(K / 8);
    const PreparedParts pp = prepared_parts(planes, static_cast<size_t>(K / 32), nmain, nlow);
    for (int c = threadIdx.x; c < chunks; c += THREADS) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(x_row) + 2 * c);     // L2: coherent with this block's own stores
        const float4 b = __ldcg(reinterpret_cast<const float4*>(x_row) + 2 * c + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        convert_groups<kOrderNibble>(v, m, M, static_cast<size_t>(c >> 5) * 8, mode, nmain, nlow, 0.0625f, pp);
    }
}

#endif  // __CUDACC__

}  // namespace sgq
