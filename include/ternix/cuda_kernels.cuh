// Source-compatible with the reference's include/ternix/cuda_kernels.cuh:11-21.
//
// C[M,N] (int32) = A[M,K] (int8) x W[K,N] (ternary, packed 4 per byte as K x N/4).
// Device-pointer variants are asynchronous on `stream` and return the launch status.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace ternix {

// Any M, K; N % 4 == 0 (cudaErrorInvalidValue otherwise, before any pointer is touched).
// Picks the sm_100a kernel by shape: streamed dp4a GEMV for M <= 16, TMA + tcgen05 GEMM above,
// a generic kernel for shapes whose packed rows are not 16-byte multiples.
cudaError_t mul_mat_ternary_cuda_naive(const int8_t* dA, const uint8_t* dB, int32_t* dC,
                                       int M, int K, int N, cudaStream_t stream = 0);

// Keeps the legacy contract of this name: M, N, K multiples of 64 (cudaErrorInvalidValue otherwise,
// with no memory access) and 16-byte aligned device pointers.  Same kernels as above.
cudaError_t mul_mat_ternary_cuda_tiled(const int8_t* dA, const uint8_t* dB, int32_t* dC,
                                       int M, int K, int N, cudaStream_t stream = 0);

// Convenience wrapper on host pointers (allocates, copies, runs, copies back, frees).
cudaError_t mul_mat_ternary_cuda_host(const int8_t* A, const uint8_t* B_packed, int32_t* C,
                                      int M, int K, int N, bool tiled);

}  // namespace ternix
