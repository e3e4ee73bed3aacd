/*
 * CPU oracle for the ternary matrix product  C[M,N] int32 = A[M,K] int8 x W[K,N] ternary.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's CPU algorithm.
 * It exists so that the CUDA path can be checked bit-for-bit; it is never linked into, called
 * from, or used as a fallback by the product library.  Only the test-suite, the smoke check
 * and the benchmark's cpu-baseline leg may load it.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle.py) against
 *   - the reference's own sources compiled unmodified (oracle/_ref, built by oracle/Makefile), and
 *   - golden vectors generated from those sources with the reference tests' shapes and seeds
 *     (tests/golden/, made by tests/golden/make_golden.py).
 *
 * Packed format (reference: src/bitpack.cpp:5-15, README.md:48-54):
 *   row-major K x (N/4) bytes; weight j of a group of four sits in bits 2j..2j+1 of its byte;
 *   code 00 -> 0, 01 -> +1, 11 -> -1.  Code 10 is never produced by the packer; the reference
 *   kernels disagree on it, so parity is defined on packer output only.
 */
#ifndef TERNARY_ORACLE_H
#define TERNARY_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference: src/bitpack.cpp:5-15  (processes size/4 bytes; a tail of size%4 elements is dropped) */
void oracle_pack_ternary(uint8_t *packed, const int8_t *unpacked, size_t size);
/* reference: src/bitpack.cpp:17-27 (code 10 -> 0) */
void oracle_unpack_ternary(int8_t *unpacked, const uint8_t *packed, size_t size);
/* reference: src/bitpack.cpp:29-33 (identity copy of size/4 bytes) */
void oracle_interleave_offline(uint8_t *out, const uint8_t *packed, size_t size);

/* reference: src/mul_mat_ternary.cpp:38-58  (i-k-j, w = (bits&1) - (bits&2); needs N % 4 == 0) */
void oracle_matmul_scalar(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N);
/* reference: src/mul_mat_ternary.cpp:8-36   (i-j-k, branching decode, code 10 -> 0) */
void oracle_matmul_naive(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N);
/* reference: src/mul_mat_ternary.cpp:60-105 and :107-152.  Same arithmetic as the AVX2 kernels in
 * the same k order: per 8-column block, lane w = sign-extended 2-bit field, product = psignd(a, w).
 * Needs N % 8 == 0, as the reference does (include/ternix/mul_mat_ternary.h:41). */
void oracle_matmul_avx2_semantics(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N);
/* reference: tests/test_ternary_matmul.cpp:31-39 (independent int32 GEMM on UNPACKED weights) */
void oracle_matmul_unpacked(const int8_t *A, const int8_t *W, int32_t *C, size_t M, size_t K, size_t N);

/* Fast checker used at large sizes: unpack once, then a row-parallel (pthreads) unpacked GEMM.
 * Arithmetically identical to oracle_matmul_scalar on packer output; `threads` <= 0 means all. */
int oracle_matmul_fast(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N, int threads);

/* C[i, n0:n0+Nn] of the full product, for checking column shards without computing all of C. */
int oracle_matmul_columns(const int8_t *A, const uint8_t *Wp, int32_t *Cslice, size_t M, size_t K, size_t N,
                          size_t n0, size_t Nn, int threads);

#ifdef __cplusplus
}
#endif
#endif
