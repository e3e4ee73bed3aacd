// Source-compatible with the reference's include/ternix/mul_mat_ternary.h:18-60.
//
// C[M,N] (int32) = A[M,K] (int8) x W[K,N] (ternary, packed K x N/4).  HOST pointers.
//
// In this library all four names run the same B200 path (upload, sm_100a kernel, download) and
// give the bit-identical int32 result the reference's CPU kernels give.  There is no CPU
// implementation behind them: without a usable GPU they throw std::runtime_error.  The
// reference's preconditions stay the loosest common ones: N % 4 == 0 for every name (the AVX2
// names also accept N % 8 == 4 here, where the reference's own kernels are out of contract).
#pragma once
#include <cstddef>
#include <cstdint>

namespace ternix {

void mul_mat_ternary_naive(const int8_t* __restrict A, const uint8_t* __restrict B_packed,
                           int32_t* __restrict C, size_t M, size_t K, size_t N);
void mul_mat_ternary_scalar(const int8_t* __restrict A, const uint8_t* __restrict B_packed,
                            int32_t* __restrict C, size_t M, size_t K, size_t N);
void mul_mat_ternary_avx2(const int8_t* __restrict A, const uint8_t* __restrict B_packed,
                          int32_t* __restrict C, size_t M, size_t K, size_t N);
void mul_mat_ternary_avx2_blocked(const int8_t* __restrict A, const uint8_t* __restrict B_packed,
                                  int32_t* __restrict C, size_t M, size_t K, size_t N);

}  // namespace ternix
