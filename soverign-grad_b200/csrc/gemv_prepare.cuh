// Conversion of fp32 activation rows into the decode kernel's operand format ("prepared
// activations"): balanced base-256 int8 digit planes laid out as mma.sync B fragments, the
// per-group corrections that cancel the +8 offset of the unpacked nibbles, and one power-of-two
// scale per row.  Shared by the decode kernel (conversion inside its CTAs), the stand-alone
// conversion kernel, and the decoder operators that emit this format directly.
//
// Layout of a prepared buffer for M rows of K values (K % 256 == 0), with ndigits = 3 (M <= 2) or
// 2 and nsets = ceil(M * ndigits / 8):
//   [digit planes: (K/32) * nsets * 256 B][corrections: (K/32) * nsets * 32 B][inv scale: 16 fp32]
#pragma once

#include "sgq_common.cuh"

namespace sgq {

constexpr int kPreparedMaxM = 16;

// The accumulator of a group's integer MMA starts at (-8 * sum of digits) + kGroupSumBias.  The first
// term cancels the +8 offset of the unpacked nibbles; the second makes the int32 result, read as
// fp32 bits, equal to 12582912.0f + S for the exact group sum S (|S| <= 32 * 15 * 128 < 2^22), so the
// kernel gets S as a float with one full-rate subtraction instead of an int-to-float conversion.
constexpr int kGroupSumBias = 0x4B400000;
constexpr float kGroupSumBiasF = 12582912.0f;

struct PreparedLayout {
    int ndigits, nsets;
    size_t bytes;          // digit planes + corrections + row scales
};

inline PreparedLayout prepared_layout(int64_t M, int64_t K) {
    PreparedLayout L;
    L.ndigits = (M <= 2) ? 3 : 2;        // 2 digits: M = 3, 4 still fit one set of 8 columns
    L.nsets = static_cast<int>((M * L.ndigits + 7) / 8);
    L.bytes = static_cast<size_t>(K / 32) * L.nsets * 288 + kPreparedMaxM * 4;
    return L;
}

#ifdef __CUDACC__

// Balanced base-256 digits of q (|q| <= 2^22): q = d0 + 256 d1 + 65536 d2 with every d in [-128, 127].
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

// One item = 8 consecutive activations (m, chunk c) already scaled knowledge: row bound bits `mb`.
// Writes the item's digit bytes into the B-fragment plane and, for the lane with t == 0, the
// group's correction.  The four lanes holding the four chunks of a 32-k group must call together.
//   xs  : [group][set][col 8][t 4] x 8 bytes; the 8 bytes of (col, t) are the digits of
//         k = 32*group + 8t + {0,2,4,6} (b0) and + {1,3,5,7} (b1); column col = m*ndigits + j.
//   corr: [group][set][col 8] int32 = kGroupSumBias - 8 * sum over the group's 32 k of that column's digits.
__device__ __forceinline__ void row_scale(uint32_t mb, int frac_bits, float* P, float* invP) {
    // P = 2^(frac_bits - e) with 2^e > absmax (e = exponent of absmax + 1); absmax 0 -> P = 1
    const int e = static_cast<int>(mb >> 23) - 127 + 1;
    int sh = frac_bits - e;                 // kept inside the normal range
    sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
    *P = (mb == 0) ? 1.0f : __uint_as_float(static_cast<uint32_t>(127 + sh) << 23);
    *invP = (mb == 0) ? 1.0f : __uint_as_float(static_cast<uint32_t>(127 - sh) << 23);
}

__device__ __forceinline__ void digits_item(const float (&v)[8], float P, int m, int c, int ndigits, int nsets,
                                            uint8_t* xs, uint8_t* corr) {
    uint32_t db[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) db[j] = digit_bytes(__float2int_rn(v[j] * P));
    const int group = c >> 2, t = c & 3;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
        if (j < ndigits) {
            const uint32_t b0 = gather_byte(db[0], db[2], db[4], db[6], j);   // k = 8t + {0,2,4,6}
            const uint32_t b1 = gather_byte(db[1], db[3], db[5], db[7], j);   // k = 8t + {1,3,5,7}
            int sum = __dp4a(static_cast<int>(b0), 0x01010101, __dp4a(static_cast<int>(b1), 0x01010101, 0));
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            const int col = m * ndigits + j, set = col >> 3, cc = col & 7;
            *reinterpret_cast<uint2*>(xs + (static_cast<size_t>(group) * nsets + set) * 256 + (cc * 4 + t) * 8) =
                make_uint2(b0, b1);
            if (t == 0)
                *reinterpret_cast<int*>(corr + (static_cast<size_t>(group) * nsets + set) * 32 + cc * 4) = kGroupSumBias - 8 * sum;
        }
    }
}

__device__ __forceinline__ float absmax8(const float (&v)[8]) {
    return fmaxf(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))),
                 fmaxf(fmaxf(fabsf(v[4]), fabsf(v[5])), fmaxf(fabsf(v[6]), fabsf(v[7]))));
}


// Block-wide conversion of one row (row index m of the batch) whose K values lie at x_row in
// global memory (values this block wrote itself are visible after the caller's __syncthreads).
// `all_max` is the row's absmax, already known to every thread.  K / 8 must be a multiple of 32
// so that whole warps take part in each digits_item call.
template <int THREADS>
__device__ __forceinline__ void prepare_row_block(const float* x_row, float all_max, int m, int64_t K, int ndigits,
                                                  int nsets, uint8_t* __restrict__ planes) {
    const int chunks = static_cast<int>(K / 8);
    const size_t groups = static_cast<size_t>(K / 32);
    uint8_t* xs = planes;
    uint8_t* corr = planes + groups * nsets * 256;
    float* inv_p = reinterpret_cast<float*>(corr + groups * nsets * 32);
    float P, invP;
    row_scale(__float_as_uint(all_max), ndigits == 3 ? 22 : 14, &P, &invP);
    if (threadIdx.x == 0) inv_p[m] = invP;
    for (int c = threadIdx.x; c < chunks; c += THREADS) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(x_row) + 2 * c);     // L2: coherent with this block's own stores
        const float4 b = __ldcg(reinterpret_cast<const float4*>(x_row) + 2 * c + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        digits_item(v, P, m, c, ndigits, nsets, xs, corr);
    }
}

#endif  // __CUDACC__

}  // namespace sgq
