// The reference's C++ API (namespace ternix, include/ternix/*.h*) as thin callers of the C ABI.
// Same names, argument meaning and error behaviour; see each header for the interface it mirrors.
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "ternix/bitpack.hpp"
#include "ternix/cuda_kernels.cuh"
#include "ternix/mul_mat_ternary.h"
#include "ternix_b200.h"

namespace ternix {

// reference: src/bitpack.cpp:5-33
void pack_ternary_weights(uint8_t* packed, const int8_t* unpacked, size_t size) {
    ternix_b200_pack_ternary(packed, unpacked, size);
}
void unpack_ternary_weights(int8_t* unpacked, const uint8_t* packed, size_t size) {
    ternix_b200_unpack_ternary(unpacked, packed, size);
}
void interleave_weights_offline(uint8_t* interleaved, const uint8_t* packed, size_t size) {
    ternix_b200_interleave_offline(interleaved, packed, size);
}

namespace {

cudaError_t to_cuda_error(int status) {
    switch (status) {
        case TERNIX_B200_OK: return cudaSuccess;
        case TERNIX_B200_ERR_CUDA: {
            const int e = ternix_b200_last_cuda_error();
            return e ? static_cast<cudaError_t>(e) : cudaErrorUnknown;
        }
        case TERNIX_B200_ERR_TIMEOUT: return cudaErrorLaunchTimeout;
        default: return cudaErrorInvalidValue;
    }
}

// The CPU-named entry points are void in the reference (src/mul_mat_ternary.cpp); here a failure
// of the GPU path cannot be ignored, so it is thrown.
void run_host(const int8_t* A, const uint8_t* B, int32_t* C, size_t M, size_t K, size_t N, const char* name) {
    constexpr size_t kMax = 0x7fffffff;
    if (M > kMax || K > kMax || N > kMax) throw std::invalid_argument(std::string(name) + ": dimension exceeds int32");
    const int rc = ternix_b200_matmul_host(A, B, C, static_cast<int>(M), static_cast<int>(K), static_cast<int>(N),
                                           TERNIX_B200_KERNEL_AUTO);
    if (rc == TERNIX_B200_ERR_INVALID_SHAPE || rc == TERNIX_B200_ERR_INVALID_ARG)
        throw std::invalid_argument(std::string(name) + ": " + ternix_b200_status_string(rc));
    if (rc == TERNIX_B200_ERR_CUDA)
        throw std::runtime_error(std::string("CUDA error: ") +
                                 cudaGetErrorString(static_cast<cudaError_t>(ternix_b200_last_cuda_error())));
    if (rc != TERNIX_B200_OK) throw std::runtime_error(std::string(name) + ": " + ternix_b200_status_string(rc));
}

}  // namespace

// reference: src/mul_mat_ternary.cpp:8-152 (four CPU kernels, one contract)
void mul_mat_ternary_naive(const int8_t* __restrict A, const uint8_t* __restrict B, int32_t* __restrict C, size_t M,
                           size_t K, size_t N) {
    run_host(A, B, C, M, K, N, "mul_mat_ternary_naive");
}
void mul_mat_ternary_scalar(const int8_t* __restrict A, const uint8_t* __restrict B, int32_t* __restrict C, size_t M,
                            size_t K, size_t N) {
    run_host(A, B, C, M, K, N, "mul_mat_ternary_scalar");
}
void mul_mat_ternary_avx2(const int8_t* __restrict A, const uint8_t* __restrict B, int32_t* __restrict C, size_t M,
                          size_t K, size_t N) {
    run_host(A, B, C, M, K, N, "mul_mat_ternary_avx2");
}
void mul_mat_ternary_avx2_blocked(const int8_t* __restrict A, const uint8_t* __restrict B, int32_t* __restrict C,
                                  size_t M, size_t K, size_t N) {
    run_host(A, B, C, M, K, N, "mul_mat_ternary_avx2_blocked");
}

// reference: src/cuda_kernels.cu:126-132
cudaError_t mul_mat_ternary_cuda_naive(const int8_t* dA, const uint8_t* dB, int32_t* dC, int M, int K, int N,
                                       cudaStream_t stream) {
    return to_cuda_error(ternix_b200_matmul(dA, dB, dC, M, K, N, stream));
}

// reference: src/cuda_kernels.cu:134-140 -- the multiple-of-64 contract of this name is kept, and is
// checked before anything else so that null pointers are safe (tests/test_cuda_matmul.cu:41-43).
cudaError_t mul_mat_ternary_cuda_tiled(const int8_t* dA, const uint8_t* dB, int32_t* dC, int M, int K, int N,
                                       cudaStream_t stream) {
    if (M <= 0 || K <= 0 || N <= 0 || M % 64 || N % 64 || K % 64) return cudaErrorInvalidValue;
    return to_cuda_error(ternix_b200_matmul(dA, dB, dC, M, K, N, stream));
}

// reference: src/cuda_kernels.cu:142-156
cudaError_t mul_mat_ternary_cuda_host(const int8_t* A, const uint8_t* B_packed, int32_t* C, int M, int K, int N,
                                      bool tiled) {
    if (tiled && (M <= 0 || K <= 0 || N <= 0 || M % 64 || N % 64 || K % 64)) return cudaErrorInvalidValue;
    return to_cuda_error(ternix_b200_matmul_host(A, B_packed, C, M, K, N, TERNIX_B200_KERNEL_AUTO));
}

}  // namespace ternix
