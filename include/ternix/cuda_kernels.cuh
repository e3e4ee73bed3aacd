// Source-compatible with the reference's include/ternix/cuda_kernels.cuh:11-21.
//
// The product computed by all three: an int32 matrix C of M rows and N columns from int8 activations A (M x K) and
// ternary weights W (K x N) that stay packed, one byte per four consecutive columns, i.e. K rows of N/4 bytes.
// The two device-pointer entry points only enqueue work on `stream` and report the launch status.
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

// The same product for operands in host memory: device buffers, both uploads, the kernel, the download of C and a
// synchronisation all happen inside the call (`tiled` keeps the multiple-of-64 contract above).
cudaError_t mul_mat_ternary_cuda_host(const int8_t* A, const uint8_t* B_packed, int32_t* C,
                                      int M, int K, int N, bool tiled);

}  // namespace ternix
