/*
 * CPU oracle for lloom-tensor's quantized matmul (Q8_0, Q4_K, Q6_K weights, and the
 * formats that ride the same two activation arms: Q4_0, Q5_0, Q5_K; Q8_0 / Q8_K activations).
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, in plain C, the reference's
 * CPU algorithm so that the CUDA kernels can be checked against it and so that
 * a CPU baseline can be timed beside them.  Nothing in the product path links,
 * loads or calls it.
 *
 * Parity status: PINNED.  The restatement reproduces every golden value the
 * reference's own tests hold for these formats that does not depend on Rust's
 * random generator (quantize/dequantize ramps, ggml-like cosine vectors,
 * block sizes, the GEMM-equals-GEMV bit identity); see tests/test_oracle_golden.py.
 *
 * dtype codes are the GGUF type ids the reference uses
 * (lloom-tensor/src/quantized/mod.rs:505-568): Q4_0 = 2, Q5_0 = 6, Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14, Q8_K = 15.
 */
#ifndef LLOOM_ORACLE_H
#define LLOOM_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LO_Q4_0 2
#define LO_Q5_0 6
#define LO_Q8_0 8
#define LO_Q4_K 12
#define LO_Q5_K 13
#define LO_Q6_K 14
#define LO_Q8_K 15

/* summation orders for vec_dot / matmul */
#define LO_ORDER_UNOPT 0      /* GgmlType::vec_dot_unopt (scalar generic form) */
#define LO_ORDER_AVX2_EMU 1   /* the AVX2 arm's lane order, emulated in portable C */
#define LO_ORDER_AVX2 2       /* the AVX2 arm with real intrinsics (needs an AVX2+FMA host) */

int lo_has_avx2(void);
int64_t lo_block_elems(int dtype);   /* 32 or 256, 0 if unknown */
int64_t lo_block_bytes(int dtype);   /* 34 / 144 / 210 / 292, 0 if unknown */

uint16_t lo_f32_to_f16(float f);
float lo_f16_to_f32(uint16_t h);

/* T::from_float for one row of k elements (k a multiple of the block size). */
int lo_quantize_row(int dtype, const float *x, void *blocks, int64_t k);
/* Same over `rows` rows of k elements, rows split over nthreads (setup helper). */
int lo_quantize_rows(int dtype, const float *x, void *blocks, int64_t rows, int64_t k, int nthreads);
/* T::from_float_imatrix for one row (k = n_per_row; imatrix: k importance weights); -2 for types without one. */
int lo_quantize_row_imatrix(int dtype, const float *x, void *blocks, int64_t k, const float *imatrix);
/* T::to_float */
int lo_dequantize_row(int dtype, const void *blocks, float *y, int64_t k);

/* T::vec_dot(k, w_row, act_row) in the requested order. */
float lo_vec_dot(int w_dtype, int64_t k, const void *w, const void *act, int order);
/* Sum of the magnitudes of the f32 summands the AVX2 arm adds for this dot product (eight lane terms
 * per block, plus four min-lane terms for Q4_K): the scale a re-ordered f32 summation is bounded by. */
float lo_vec_dot_absum(int w_dtype, int64_t k, const void *w, const void *act);

/* k_quants::matmul: lhs f32 [m,k] is quantized row by row with the weight
 * type's VecDotType, dst[r*n+c] = vec_dot(W[c], A[r]).  Columns are split into
 * quads of four, spread evenly over nthreads, as the reference does.
 * Returns 0, or -1 when dst_len < m*n with m > 1 (the reference's error), -2 bad dtype/shape. */
int lo_matmul(int w_dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *w,
              float *dst, int64_t dst_len, int nthreads, int order);
/* Same traversal, writing lo_vec_dot_absum per output element. */
int lo_matmul_absum(int w_dtype, int64_t m, int64_t k, int64_t n, const float *lhs, const void *w,
                    float *dst, int nthreads);
/* Cluster size of the thread pool's two-level tree (utils::BarrierPool, utils.rs:62-103): the reference hard-codes 6
 * on macOS and a flat tree elsewhere; 0 or 1 = flat (the default).  Takes effect with the next threaded call. */
void lo_set_cluster_size(int cluster_size);
/* Activation quantizer only (what matmul does to lhs first). */
int lo_quantize_act(int w_dtype, const float *lhs, void *act_blocks, int64_t m, int64_t k);

#ifdef __cplusplus
}
#endif
#endif
