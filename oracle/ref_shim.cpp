// C-linkage shim around the reference's own CPU kernels -- TEST INFRASTRUCTURE ONLY.
//
// Compiled together with the reference's unmodified src/mul_mat_ternary.cpp and src/bitpack.cpp
// (see oracle/Makefile) into oracle/_ref/libternix_ref.so.  It adds nothing to the arithmetic: it
// only gives the C++ functions unmangled names, a row-band thread runner (rows of C are
// independent, so slicing M leaves every result bit unchanged) and the libstdc++ mt19937 input
// generators that the reference's tests use, so golden vectors can be regenerated.
#include <cstdint>
#include <cstring>
#include <random>
#include <thread>
#include <vector>
#include "ternix/bitpack.hpp"
#include "ternix/mul_mat_ternary.h"

namespace {
using Kernel = void (*)(const int8_t*, const uint8_t*, int32_t*, size_t, size_t, size_t);

Kernel pick(int which) {
    switch (which) {
        case 0: return ternix::mul_mat_ternary_naive;
        case 1: return ternix::mul_mat_ternary_scalar;
        case 2: return ternix::mul_mat_ternary_avx2;
        case 3: return ternix::mul_mat_ternary_avx2_blocked;
        default: return nullptr;
    }
}
}  // namespace

extern "C" {

void ref_pack_ternary(uint8_t* packed, const int8_t* unpacked, size_t size) {
    ternix::pack_ternary_weights(packed, unpacked, size);
}
void ref_unpack_ternary(int8_t* unpacked, const uint8_t* packed, size_t size) {
    ternix::unpack_ternary_weights(unpacked, packed, size);
}
void ref_interleave_offline(uint8_t* out, const uint8_t* packed, size_t size) {
    ternix::interleave_weights_offline(out, packed, size);
}

// which: 0 naive, 1 scalar, 2 avx2, 3 avx2_blocked.  Single thread, exactly as the reference ships.
int ref_matmul(int which, const int8_t* A, const uint8_t* Wp, int32_t* C, size_t M, size_t K, size_t N) {
    Kernel f = pick(which);
    if (!f) return 1;
    if ((which == 2 || which == 3) && N % 8) return 2;   // include/ternix/mul_mat_ternary.h:41
    f(A, Wp, C, M, K, N);
    return 0;
}

// The same kernel on bands of rows, one std::thread per band.  Bands are multiples of 4 rows so that
// avx2_blocked keeps its 4-row blocking inside each band.
int ref_matmul_threads(int which, const int8_t* A, const uint8_t* Wp, int32_t* C, size_t M, size_t K, size_t N,
                       int threads) {
    Kernel f = pick(which);
    if (!f) return 1;
    if ((which == 2 || which == 3) && N % 8) return 2;
    if (threads <= 0) threads = static_cast<int>(std::thread::hardware_concurrency());
    if (threads < 1) threads = 1;
    size_t band = (M + threads - 1) / threads;
    band = (band + 3) / 4 * 4;
    std::vector<std::thread> pool;
    for (size_t r0 = 0; r0 < M; r0 += band) {
        const size_t rows = (r0 + band <= M) ? band : M - r0;
        pool.emplace_back([=] { f(A + r0 * K, Wp, C + r0 * N, rows, K, N); });
    }
    for (auto& t : pool) t.join();
    return 0;
}

// Inputs of tests/test_ternary_matmul.cpp:18-27 (lo = -127) and tests/test_cuda_matmul.cu:11-19
// (lo = -128): one mt19937(seed) feeding uniform_int_distribution for A, then for W.
void ref_make_problem(size_t M, size_t K, size_t N, uint32_t seed, int act_lo,
                      int8_t* A, int8_t* W, uint8_t* Wp) {
    std::mt19937 rng(seed);
    std::uniform_int_distribution<int> act(act_lo, 127);
    std::uniform_int_distribution<int> wt(-1, 1);
    for (size_t i = 0; i < M * K; ++i) A[i] = static_cast<int8_t>(act(rng));
    for (size_t i = 0; i < K * N; ++i) W[i] = static_cast<int8_t>(wt(rng));
    ternix::pack_ternary_weights(Wp, W, K * N);
}

}  // extern "C"
