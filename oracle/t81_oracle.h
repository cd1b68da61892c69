/*
 * TEST INFRASTRUCTURE — NOT THE PRODUCT.
 *
 * Plain-C restatement, for the CPU, of the packed balanced-ternary matmul path
 * of t81lib.  Only the test suite, the smoke check and the CPU-baseline leg of
 * the benchmark may link or load this; the shipped library never does.
 *
 * Parity pin: every function here is checked (tests/test_oracle_pin.py) against
 * the reference's own compiled code (oracle/_ref, built from the reference
 * sources by oracle/Makefile), against the committed fixtures in tests/golden/
 * that were generated from it, and against the reference's known-answer tests
 * (tests/python/test_bindings.py:17-39).  The "absmean" rule has no counterpart
 * in the reference; it is pinned only to its own definition (see below).
 *
 * Layout contract (include/t81/core/limb.hpp:95-235,708; core/detail/lut.hpp:13-49):
 *   a limb is 16 bytes, byte i is the tryte of trits 3i..3i+2,
 *   byte = t0 + 3*t1 + 9*t2 + 13  (0..26, zero tryte = 13).
 *   A (rows, cols) matrix packs row-wise into (rows, ceil(cols/48), 16) bytes,
 *   tail trits are 0 (python/bindings.cpp:470-516).
 */
#ifndef T81_ORACLE_H
#define T81_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define T81O_TRITS_PER_LIMB 48
#define T81O_BYTES_PER_LIMB 16
#define T81O_ABSMEAN_LANES 128 /* partial sums of the absmean reduction */

/* python/bindings.cpp:405-414 — clamp to [-1,1], inclusive compares in fp32. */
int8_t t81o_quantize_trit(float value, float threshold);

/* python/bindings.cpp:416-445 (loop body). */
void t81o_quantize_to_trits(const float *src, size_t n, float threshold, int8_t *dst);

/* t81/torch/__init__.py:68-80 (_pack_rowwise) on already-quantized trits. */
void t81o_pack_trits_rowwise(const int8_t *trits, int64_t rows, int64_t cols, uint8_t *packed);

/* t81/torch/__init__.py:83-97 (_pack_columnwise): trits is (k, cols) row-major,
 * packed is (ceil(k/48), cols, 16). */
void t81o_pack_trits_columnwise(const int8_t *trits, int64_t k, int64_t cols, uint8_t *packed);

/* Rule "fixed": python/bindings.cpp:460-517 (pack_dense_matrix). */
void t81o_pack_dense_matrix(const float *w, int64_t rows, int64_t cols, int64_t ld,
                            float threshold, uint8_t *packed);

/* Rule "absmean" (no reference counterpart; shaped after quantize_row_tq1_0,
 * src/t81/core/gguf_quants.h:55-64,116-144, with the row mean of |w| in place
 * of the row absmax):
 *   group sum g(j) = fp32 (|w[r,4j]| + |w[r,4j+1]|) + (|w[r,4j+2]| + |w[r,4j+3]|), each of the three additions
 *                rounded to fp32, elements past cols counting 0;
 *   partial[i], i = 0..127 = double sum, in increasing j, of the g(j) with ((j / 96) % 4) * 32 + (j % 96) % 32 == i
 *                (chunks of 96 groups go round four blocks of 32 partials; inside a chunk group j feeds j % 32);
 *   the 128 partials are folded by halving trees: inside each group of 32 consecutive partials (offsets
 *   16,8,4,2,1: v[j] += v[j+off]), then over the 4 group sums (offsets 2,1);
 *   s_r = float(total) / float(cols), an fp32 division;  cut = s_r > 0 ? threshold * s_r (one fp32 multiply) : +inf;
 *   trit = w <= -cut ? -1 : (w >= cut ? +1 : 0)   (the weight itself is compared: no per-weight arithmetic).
 * row_scale[r] = s_r. */
void t81o_pack_dense_matrix_absmean(const float *w, int64_t rows, int64_t cols, int64_t ld,
                                    float threshold, uint8_t *packed, float *row_scale);

/* python/bindings.cpp:640-686 (unpack_packed_limbs).  Returns 0, or -1 when a
 * byte > 26 is met (limb::from_bytes rejects it, limb.hpp:160-169). */
int t81o_unpack_packed_limbs(const uint8_t *packed, int64_t rows, int64_t k_limbs,
                             int64_t cols, int8_t *trits);

/* LIMB mode — src/linalg/gemm_cpu.cpp:8-71 with include/t81/linalg/gemm.hpp:28-64:
 * C[i][j] = float(double(C[i][j])*beta + sum_k value(A[i][k])*value(B[k][j])*double(alpha)),
 * the product formed as the exact 96-trit integer, then low + high*3^48 in fp64.
 * A is (M, k_limbs) limbs, B is (k_limbs, N) limbs, C is (M, N) fp32. */
void t81o_gemm_limb(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                    int64_t k_limbs, float alpha, float beta);

/* TRIT mode — the rounding structure of gemm_cpu.cpp:34-68 applied to
 * unpacked trits times dense activations:
 *   acc = double(C)*beta; acc += double(trit)*double(B[k][j])*double(alpha), k ascending;
 *   C = float(acc).
 * A is (M, ceil(K/48)) limbs; B is fp32 with element (k, j) at B[k*ldb_k + j*ldb_n];
 * C element (i, j) at C[i*ldc_m + j*ldc_n].  beta == 0 never reads C. */
void t81o_gemm_trit(const uint8_t *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                    int64_t ldb_k, int64_t ldb_n, int64_t ldc_m, int64_t ldc_n,
                    float alpha, float beta);

/* Linear forward in the form of the reference's QAT forward
 * (t81/nn/linear.py:42-45,72-80): y[t][o] = float(scale[o]*sum_k trit[o][k]*x[t][k] + bias[o]),
 * fp64 accumulation in k order.  row_scale and bias may be NULL. */
void t81o_linear_forward(const uint8_t *W, const float *row_scale, const float *bias,
                         const float *x, float *y, int64_t tokens, int64_t out_features,
                         int64_t in_features);

/* Host threads (pthreads, disjoint row ranges) the gemm/linear/pack loops use; default 1. */
int t81o_num_threads(void);
void t81o_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
