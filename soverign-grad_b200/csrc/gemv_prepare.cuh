// Conversion of fp32 activation rows into the decode kernels' operand format ("prepared
// activations"): group-scaled fixed point, split into balanced base-256 int8 digits that are laid
// out as mma.sync B fragments.  Shared by the decode kernels (conversion inside their CTAs), the
// stand-alone conversion kernels, and the decoder operators that emit this format directly.
//
// Arithmetic.  Every 32 consecutive k of a row (the span of one INT4 weight group) have their own
// scale: with gmax the group's absmax, q = rint(x * (Q / gmax)) with Q = 32600 (two digits) or
// 8355000 (three digits, single-row batches), q = d0 + 256 d1 (+ 65536 d2) with every digit in
// [-128, 127].  The kernels form exact integer dot products per digit and group and multiply them
// by gmax / Q in fp32.  The rounding error of one activation is at most gmax / (2 Q): relative to
// the largest of its 32 neighbours, not to the largest value of the row, so a few huge channels
// cost the rest of the row nothing (rms error of an output <= sqrt(32) * 0.29 / Q = 5e-5 of the
// output's own scale with two digits, whatever the distribution of the activations).  A group
// whose absmax is NaN or Inf gets a NaN scale (the output row becomes NaN); a group whose absmax is
// below 1e-30 contributes zero.
//
// Layout of a prepared buffer for M rows of K values (K % 32 == 0):
//   digit planes  [group K/32][set pair][fragment lane 32][sets of the pair x 8 bytes]
//   group scales  [group K/32][t 4][set] fp32: the scale of the batch row whose digits sit in
//                 columns 2t and 2t+1 of the set (a lane of an MMA holds exactly these two columns)
// A "set" is one group of eight B-fragment columns (one MMA); column = (m * ndigits + j) * colmul
// for digit j of row m; colmul = 2 when all columns then still fit one set (only even columns
// carry data and the kernels skip the odd accumulators).  With two digits a row owns columns 2t and
// 2t+1 of its set.  Sets are stored in pairs so that a lane fetches the fragments of two sets with
// one 128-bit load; a last unpaired set uses 8 bytes per lane.
#pragma once

#include "sgq_common.cuh"

namespace sgq {

constexpr int kPreparedMaxM = 16;

// The accumulator of an integer MMA starts at kMagicBits: the int32 result, read as fp32 bits,
// then equals 12582912.0f + S for the exact integer sum S (|S| < 2^22), so the kernels get S as a
// float with one full-rate subtraction instead of an int-to-float conversion.
constexpr int kMagicBits = 0x4B400000;
constexpr float kMagicF = 12582912.0f;

constexpr float kDigitRange2 = 32600.0f;     // |q| <= 32639 = 127 * 257 must hold after rounding
constexpr float kDigitRange3 = 8355000.0f;   // |q| <= 8355711 = 127 * 65793

struct PreparedLayout {
    int ndigits, nsets, colmul;
    size_t digit_bytes, scale_bytes, bytes;
};

inline PreparedLayout prepared_layout(int64_t M, int64_t K) {
    PreparedLayout L;
    L.ndigits = (M == 1) ? 3 : 2;
    L.colmul = (M * L.ndigits <= 4) ? 2 : 1;
    L.nsets = static_cast<int>((M * L.ndigits * L.colmul + 7) / 8);
    L.digit_bytes = static_cast<size_t>(K / 32) * L.nsets * 256;
    L.scale_bytes = static_cast<size_t>(K / 32) * L.nsets * 16;
    L.bytes = L.digit_bytes + L.scale_bytes;
    return L;
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

// Converts 256 consecutive k (eight 32-k groups, the first being group `group0`) of row m.  Must be
// called by all 32 lanes of a warp together, lane l holding the 8 consecutive activations
// k = 32 * group0 + 8 l .. + 7 in v: four neighbouring lanes share a group.  `scale_mul` is folded
// into the stored scales (the INT4 kernel feeds its codes to the tensor core as 16 * code and
// passes 1/16).  A lane with store == false (beyond the end of a row) passes zeros and writes nothing.
template <int ORDER>
__device__ __forceinline__ void convert_groups(const float (&v)[8], int m, size_t group0, int ndigits, int nsets, int colmul,
                                               float scale_mul, uint8_t* __restrict__ digits, float* __restrict__ scales,
                                               bool store = true) {
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
    }
    const float gmax = __uint_as_float(mb);
    const float range = (ndigits == 3) ? kDigitRange3 : kDigitRange2;
    float P, sx;
    if (mb >= 0x7F800000u) {            // NaN or Inf somewhere in the group: the output row becomes NaN
        P = 0.0f;
        sx = __uint_as_float(0x7FC00000u);
    } else if (gmax < 1e-30f) {         // zero (or vanishing) group
        P = 0.0f;
        sx = 0.0f;
    } else {
        P = __fdiv_rn(range, gmax);
        sx = __fmul_rn(__fdiv_rn(gmax, range), scale_mul);
    }
    if (!store) return;
    uint32_t db[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) db[j] = digit_bytes(__float2int_rn(__fmul_rn(v[j], P)));
    const size_t group = group0 + (lane >> 2);
    const int q = lane & 3;             // which quarter of the group this lane holds
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        if (j < ndigits) {
            const int col = (m * ndigits + j) * colmul, set = col >> 3, cc = col & 7;
            if (q == 0) scales[(group * 4 + (cc >> 1)) * nsets + set] = sx;
            if (ORDER == kOrderNibble) {
                const uint32_t b0 = gather_byte(db[0], db[2], db[4], db[6], j);
                const uint32_t b1 = gather_byte(db[1], db[3], db[5], db[7], j);
                *reinterpret_cast<uint2*>(digits + plane_offset(group, nsets, set, cc * 4 + q)) = make_uint2(b0, b1);
            } else {
                // k = 8q .. 8q+7: the first four go to fragment lane t0 = 2 (q & 1), the next four to t0 + 1,
                // in b0 when k < 16 and in b1 otherwise
                const int t0 = 2 * (q & 1), half = q >> 1;
                *reinterpret_cast<uint32_t*>(digits + plane_offset(group, nsets, set, cc * 4 + t0) + half * 4) =
                    gather_byte(db[0], db[1], db[2], db[3], j);
                *reinterpret_cast<uint32_t*>(digits + plane_offset(group, nsets, set, cc * 4 + t0 + 1) + half * 4) =
                    gather_byte(db[4], db[5], db[6], db[7], j);
            }
        }
    }
}

// Block-wide conversion of one row (row index m of the batch) whose K values lie at x_row in
// global memory (values this thread block wrote itself are visible after the caller's
// __syncthreads).  THREADS must be a multiple of 32 and K a multiple of 256, so that whole warps
// take part in every conversion call.  `planes` is the prepared buffer of the INT4 decode kernel.
template <int THREADS>
__device__ __forceinline__ void prepare_row_block(const float* x_row, int m, int64_t K, int ndigits, int nsets, int colmul,
                                                  uint8_t* __restrict__ planes) {
    const int chunks = static_cast<int>(K / 8);
    float* scales = reinterpret_cast<float*>(planes + static_cast<size_t>(K / 32) * nsets * 256);
    for (int c = threadIdx.x; c < chunks; c += THREADS) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(x_row) + 2 * c);     // L2: coherent with this block's own stores
        const float4 b = __ldcg(reinterpret_cast<const float4*>(x_row) + 2 * c + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        convert_groups<kOrderNibble>(v, m, static_cast<size_t>(c >> 5) * 8, ndigits, nsets, colmul, 0.0625f, planes, scales);
    }
}

#endif  // __CUDACC__

}  // namespace sgq
