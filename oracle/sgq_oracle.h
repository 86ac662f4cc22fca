/* TEST INFRASTRUCTURE — plain-C restatement of the SovereignGrad quantization hot path.
 *
 * Only tests/, __graft_entry__.smoke() and the cpu_baseline leg of bench.py may load this;
 * the shipped library never does.  Every function names the reference lines it follows
 * (paths relative to the reference checkout).  Parity of this restatement is pinned by
 * tests/test_oracle.py against (a) fixtures under tests/golden/ that were produced by the
 * compiled, unmodified reference (oracle/_ref/libsgref.so) and (b) that library itself when
 * it is present.
 *
 * Byte layout (the reference stores codes as fp32 and defines no bytes, so this is the
 * contract of this repository):
 *   INT8: one two's-complement int8 per element, flat row-major order.
 *   INT4: two two's-complement nibbles per byte, element 2i in the LOW nibble, element 2i+1
 *         in the HIGH nibble, ceil(numel/2) bytes, odd tail -> high nibble 0.
 *   scales: fp32, reference order (1 | rows | ceil(numel/group)).
 */
#ifndef SGQ_ORACLE_H
#define SGQ_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { SGQO_LAYOUT_KN = 0, SGQO_LAYOUT_NK = 1 };
enum { SGQO_PER_TENSOR = 0, SGQO_PER_ROW = 1 };

/* src/quantization.cpp:22-41 */
void sgqo_quantize_int8_tensor(const float* x, int64_t n, int8_t* codes, float* scale);
/* src/quantization.cpp:42-75 */
void sgqo_quantize_int8_rows(const float* x, int64_t rows, int64_t cols, int8_t* codes, float* scales);
/* src/quantization.cpp:113-159; group <= 0 -> 32 (:118) */
void sgqo_quantize_int4(const float* x, int64_t n, int64_t group, uint8_t* packed, float* scales);

/* canonical byte layout <-> the reference's fp32 code tensor */
void sgqo_pack_int4_codes(const float* codes_f32, int64_t n, uint8_t* packed);
void sgqo_unpack_int4_codes(const uint8_t* packed, int64_t n, float* codes_f32);
void sgqo_pack_int8_codes(const float* codes_f32, int64_t n, int8_t* codes);
void sgqo_unpack_int8_codes(const int8_t* codes, int64_t n, float* codes_f32);

/* src/quantization.cpp:80-111 (scheme per-tensor also taken when nscales == 1) */
void sgqo_dequantize_int8(const int8_t* codes, const float* scales, int64_t rows, int64_t cols, int scheme,
                          float* out);
/* src/quantization.cpp:161-187 */
void sgqo_dequantize_int4(const uint8_t* packed, const float* scales, int64_t n, int64_t group, float* out);

/* y[M,N] = x[M,K] * W (+ bias[N]); w is the DEQUANTIZED fp32 weight, [K,N] (layout KN) or
 * [N,K] (layout NK, y = x * w^T).  fp32, in the accumulation order of the reference's CPU
 * matmul: src/ops.cpp:378-455 + include/sovereigngrad/simd.hpp:152-221; bias as a separate
 * fp32 add, src/quantization.cpp:193-195. */
void sgqo_linear_f32(const float* x, int64_t M, int64_t K, int64_t N, const float* w, int layout,
                     const float* bias, float* y);
/* same product in fp64 (error attribution) */
void sgqo_linear_f64(const float* x, int64_t M, int64_t K, int64_t N, const float* w, int layout,
                     const float* bias, double* y);

/* src/quantization.cpp:189-206: dequantize, multiply, add bias. */
void sgqo_qlinear_int4(const float* x, int64_t M, int64_t K, int64_t N, const uint8_t* packed,
                       const float* scales, int layout, int64_t group, const float* bias, float* y);
void sgqo_qlinear_int8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* codes, const float* scales,
                       int layout, int scheme, const float* bias, float* y);

/* Integer sub-path (no counterpart in the reference, which never quantizes activations):
 * exact int32 GEMM of int8 codes, acc[m,n] = sum_k xq[m,k] * wq[k,n | n,k]. */
void sgqo_igemm_s8(const int8_t* xq, const int8_t* wq, int64_t M, int64_t K, int64_t N, int layout, int32_t* acc);
/* W8A8 forward: xq,sx = reference per-row quantizer applied to x (src/quantization.cpp:42-75);
 * acc = exact int32; y = ((float)acc * sx[m]) * sw + bias, sw = scales[0] (per-tensor) or the
 * per-row scale of the stored weight tensor (row = k for KN, n for NK).  Per-row KN scales
 * cannot be factored out of the k-sum, so scheme PER_ROW requires layout NK here. */
void sgqo_qlinear_w8a8(const float* x, int64_t M, int64_t K, int64_t N, const int8_t* wq, const float* wscales,
                       int layout, int scheme, const float* bias, int8_t* xq_out, float* sx_out, int32_t* acc_out,
                       float* y);

#ifdef __cplusplus
}
#endif
#endif
