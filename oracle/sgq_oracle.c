/* TEST INFRASTRUCTURE — plain-C restatement of the SovereignGrad quantization hot path.
 * See sgq_oracle.h for the contract and for who may load this.  Build: `make -C oracle port`
 * (-ffp-contract=off: every fused multiply-add below is spelled fmaf on purpose).
 */
#include "sgq_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* std::min(hi, v) then std::max(lo, .) exactly as written in src/quantization.cpp:36,68,151:
 * std::min(a,b) = (b < a) ? b : a and std::max(a,b) = (a < b) ? b : a, so a NaN product
 * becomes +hi (the comparisons are false) and the result is never NaN. */
static inline float clamp_like_reference(float v, float lo, float hi) {
    float m = (v < hi) ? v : hi;
    return (lo < m) ? m : lo;
}

/* src/quantization.cpp:23-27,57-61,140-144: running max starts at 1e-8f, strict '>' compare,
 * hence NaN inputs never raise it. */
static inline float absmax_like_reference(const float* x, int64_t n) {
    float max_abs = 1e-8f;
    for (int64_t i = 0; i < n; ++i) {
        float a = fabsf(x[i]);
        if (a > max_abs) max_abs = a;
    }
    return max_abs;
}

static inline int code_of(float x, float inv_scale, float lo, float hi) {
    /* src/quantization.cpp:35-36: multiply by inv_scale (not divide by scale), std::round =
     * half away from zero = C roundf. */
    float v = roundf(x * inv_scale);
    return (int)clamp_like_reference(v, lo, hi);
}

void sgqo_quantize_int8_tensor(const float* x, int64_t n, int8_t* codes, float* scale) {
    float max_abs = absmax_like_reference(x, n);
    float s = max_abs / 127.0f;         /* :29 */
    float inv_scale = 127.0f / max_abs; /* :30 — a second, separate division */
    for (int64_t i = 0; i < n; ++i) codes[i] = (int8_t)code_of(x[i], inv_scale, -127.0f, 127.0f);
    *scale = s;
}

void sgqo_quantize_int8_rows(const float* x, int64_t rows, int64_t cols, int8_t* codes, float* scales) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        float max_abs = absmax_like_reference(xr, cols);
        float inv_scale = 127.0f / max_abs;
        scales[r] = max_abs / 127.0f;
        for (int64_t c = 0; c < cols; ++c) codes[r * cols + c] = (int8_t)code_of(xr[c], inv_scale, -127.0f, 127.0f);
    }
}

void sgqo_quantize_int4(const float* x, int64_t n, int64_t group, uint8_t* packed, float* scales) {
    if (group <= 0) group = 32; /* :118 */
    int64_t num_groups = (n + group - 1) / group;
    int64_t nbytes = (n + 1) / 2;
    int8_t* codes = (int8_t*)malloc((size_t)(n > 0 ? n : 1));
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < num_groups; ++g) {
        int64_t g_start = g * group;
        int64_t g_end = g_start + group < n ? g_start + group : n;
        float max_abs = absmax_like_reference(x + g_start, g_end - g_start);
        float inv_scale = 7.0f / max_abs; /* :147 */
        scales[g] = max_abs / 7.0f;       /* :146 */
        for (int64_t i = g_start; i < g_end; ++i) codes[i] = (int8_t)code_of(x[i], inv_scale, -8.0f, 7.0f);
    }
    for (int64_t b = 0; b < nbytes; ++b) {
        unsigned lo = (unsigned)codes[2 * b] & 0xFu;
        unsigned hi = (2 * b + 1 < n) ? ((unsigned)codes[2 * b + 1] & 0xFu) : 0u;
        packed[b] = (uint8_t)(lo | (hi << 4));
    }
    free(codes);
}

void sgqo_pack_int4_codes(const float* codes_f32, int64_t n, uint8_t* packed) {
    int64_t nbytes = (n + 1) / 2;
    for (int64_t b = 0; b < nbytes; ++b) {
        unsigned lo = (unsigned)(int)codes_f32[2 * b] & 0xFu;
        unsigned hi = (2 * b + 1 < n) ? ((unsigned)(int)codes_f32[2 * b + 1] & 0xFu) : 0u;
        packed[b] = (uint8_t)(lo | (hi << 4));
    }
}

static inline int nibble_at(const uint8_t* packed, int64_t i) {
    unsigned v = (packed[i >> 1] >> ((i & 1) * 4)) & 0xFu;
    return (int)(v ^ 8u) - 8; /* sign-extend a 4-bit two's-complement value */
}

void sgqo_unpack_int4_codes(const uint8_t* packed, int64_t n, float* codes_f32) {
    for (int64_t i = 0; i < n; ++i) codes_f32[i] = (float)nibble_at(packed, i);
}

void sgqo_pack_int8_codes(const float* codes_f32, int64_t n, int8_t* codes) {
    for (int64_t i = 0; i < n; ++i) codes[i] = (int8_t)(int)codes_f32[i];
}

void sgqo_unpack_int8_codes(const int8_t* codes, int64_t n, float* codes_f32) {
    for (int64_t i = 0; i < n; ++i) codes_f32[i] = (float)codes[i];
}

void sgqo_dequantize_int8(const int8_t* codes, const float* scales, int64_t rows, int64_t cols, int scheme,
                          float* out) {
    if (scheme == SGQO_PER_TENSOR) { /* :91-95 */
        float s = scales[0];
        for (int64_t i = 0; i < rows * cols; ++i) out[i] = (float)codes[i] * s;
    } else { /* :96-108 */
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            float s = scales[r];
            for (int64_t c = 0; c < cols; ++c) out[r * cols + c] = (float)codes[r * cols + c] * s;
        }
    }
}

void sgqo_dequantize_int4(const uint8_t* packed, const float* scales, int64_t n, int64_t group, float* out) {
    if (group <= 0) group = 32;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = (float)nibble_at(packed, i) * scales[i / group]; /* :176-183 */
}

static inline float w_at(const float* w, int layout, int64_t K, int64_t N, int64_t k, int64_t n) {
    return layout == SGQO_LAYOUT_KN ? w[k * N + n] : w[n * K + k];
}

/* Accumulation order of src/ops.cpp:398-446 with the AVX2 micro-kernel of simd.hpp:152-221.
 * Output blocks are 32 rows x 64 columns, k in blocks of 128.
 *  - rows in a full group of 8 and columns in a full group of 8: the micro-kernel loads C,
 *    runs one fused multiply-add per k and stores C, block after block -> one fmaf chain over
 *    all k starting from 0.
 *  - rows in a full group of 8, column in the <8 tail: per k-block `acc = 0; acc += a*b`
 *    (contracted to fma by the reference's compiler flags), then `C += acc`.
 *  - rows in the <8 tail of the 32-row block: `C += a*b` for k ascending -> one fmaf chain. */
void sgqo_linear_f32(const float* x, int64_t M, int64_t K, int64_t N, const float* w, int layout,
                     const float* bias, float* y) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            int64_t i0 = (i / 32) * 32, j0 = (j / 64) * 64;
            int64_t i_max = i0 + 32 < M ? i0 + 32 : M, j_max = j0 + 64 < N ? j0 + 64 : N;
            int row_in_8 = (i - i0) < 8 * ((i_max - i0) / 8);
            int col_in_8 = (j - j0) < 8 * ((j_max - j0) / 8);
            const float* xr = x + i * K;
            float c = 0.0f;
            if (!row_in_8 || col_in_8) {
                for (int64_t k = 0; k < K; ++k) c = fmaf(xr[k], w_at(w, layout, K, N, k, j), c);
            } else {
                for (int64_t k0 = 0; k0 < K; k0 += 128) {
                    int64_t k_max = k0 + 128 < K ? k0 + 128 : K;
                    float acc = 0.0f;
                    for (int64_t k = k0; k < k_max; ++k) acc = acc + xr[k] * w_at(w, layout, K, N, k, j);
                    c = c + acc;
                }
            }
            if (bias) c = c + bias[j];
            y[i * N + j] = c;
        }
    }
}

void sgqo_linear_f64(const float* x, int64_t M, int64_t K, int64_t N, const float* w, int layout,
                     const float* bias, double* y) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            double c = 0.0;
            for (int64_t k = 0; k < K; ++k) c += (double)x[i * K + k] * (double)w_at(w, layout, K, N, k, j);
            if (bias) c += (double)bias[j];
            y[i * N + j] = c;
        }
    }
}

void sgqo_qlinear_int4(const float* x, int64_t M, int64_t K, int64_t N, const uint8_t* packed,
                       const float* scales, int layout, int64_t group, const float* bias, float* y) {
    float* w = (float*)malloc(sizeof(float) * (size_t)(K * N > 0 ? K * N : 1));
    sgqo_dequantize_int4(packed, scales, K * N, group, w);
    sgqo_linear_f32(x, M, K, N, w, layout, bias, y);
    free(w);
}

void sgqo_qlinear_int8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* codes, const float* scales,
                       int layout, int scheme, const float* bias, float* y) {
    float* w = (float*)malloc(sizeof(float) * (size_t)(K * N > 0 ? K * N : 1));
    int64_t rows = layout == SGQO_LAYOUT_KN ? K : N;
    sgqo_dequantize_int8(codes, scales, rows, (K * N) / (rows > 0 ? rows : 1), scheme, w);
    sgqo_linear_f32(x, M, K, N, w, layout, bias, y);
    free(w);
}

void sgqo_igemm_s8(const int8_t* xq, const int8_t* wq, int64_t M, int64_t K, int64_t N, int layout, int32_t* acc) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            int32_t a = 0;
            for (int64_t k = 0; k < K; ++k) {
                int32_t wv = layout == SGQO_LAYOUT_KN ? wq[k * N + j] : wq[j * K + k];
                a += (int32_t)xq[i * K + k] * wv;
            }
            acc[i * N + j] = a;
        }
    }
}

void sgqo_qlinear_w8a8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* wq, const float* wscales,
                       int layout, int scheme, const float* bias, int8_t* xq_out, float* sx_out, int32_t* acc_out,
                       float* y) {
    sgqo_quantize_int8_rows(x, M, K, xq_out, sx_out);
    sgqo_igemm_s8(xq_out, wq, M, K, N, layout, acc_out);
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            float sw = scheme == SGQO_PER_TENSOR ? wscales[0] : wscales[j];
            float v = ((float)acc_out[i * N + j] * sx_out[i]) * sw;
            if (bias) v = v + bias[j];
            y[i * N + j] = v;
        }
    }
}
