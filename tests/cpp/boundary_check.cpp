// Executes the C++ boundary of the library: every function that include/ternix/*.h* declares, called the way the
// reference project's own unit tests call them, with the inputs those tests generate and an independent expected value.
//
//   * the four CPU-named products (include/ternix/mul_mat_ternary.h) on the shapes and mt19937 seeds of the reference's
//     tests/test_ternary_matmul.cpp:43-69, C pre-filled with -999, expected = integer GEMM on the UNPACKED weights;
//   * the extreme-activation case of the same file (A == -128, K = 4096);
//   * the three CUDA-named functions (include/ternix/cuda_kernels.cuh) on the shapes and seeds of
//     tests/test_cuda_matmul.cu:11-43: the host-pointer wrapper with tiled = false / true, and the two device-pointer
//     functions on cudaMalloc'ed buffers and a non-default stream;
//   * their error behaviour: shape errors are cudaErrorInvalidValue and are reported before any pointer is touched
//     (null pointers are passed);
//   * pack / unpack / interleave (include/ternix/bitpack.hpp) on the round-trip vector of tests/test_bitpack.cpp:6.
//
// Includes only the ternix headers, links libternix_b200.so.  Plain main(): GoogleTest is not available offline.
// Exit code 0 and a last line "boundary_check: PASS (<n> checks)" on success.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "ternix/bitpack.hpp"
#include "ternix/cuda_kernels.cuh"
#include "ternix/mul_mat_ternary.h"

namespace {

int g_checks = 0, g_failures = 0;

void expect(bool ok, const std::string& what) {
    ++g_checks;
    if (!ok) {
        ++g_failures;
        std::printf("FAIL: %s\n", what.c_str());
    }
}

struct Operands {
    int m, k, n;
    std::vector<int8_t> act, weights;       // M x K, K x N (unpacked, ternary)
    std::vector<uint8_t> packed;            // K x N/4
    std::vector<int32_t> want;              // M x N, from the unpacked weights
};

// Draw order and distributions as in the reference tests: all activations first, then all weights, from one
// std::mt19937; libstdc++'s uniform_int_distribution, as there.
Operands draw(int m, int k, int n, uint32_t seed, int act_lo) {
    Operands op{m, k, n, {}, {}, {}, {}};
    op.act.resize(static_cast<size_t>(m) * k);
    op.weights.resize(static_cast<size_t>(k) * n);
    op.packed.resize(op.weights.size() / 4);
    std::mt19937 gen(seed);
    std::uniform_int_distribution<int> a_dist(act_lo, 127), w_dist(-1, 1);
    for (int8_t& v : op.act) v = static_cast<int8_t>(a_dist(gen));
    for (int8_t& v : op.weights) v = static_cast<int8_t>(w_dist(gen));
    ternix::pack_ternary_weights(op.packed.data(), op.weights.data(), op.weights.size());
    return op;
}

void fill_expected(Operands& op) {
    op.want.assign(static_cast<size_t>(op.m) * op.n, 0);
    for (int i = 0; i < op.m; ++i)
        for (int kk = 0; kk < op.k; ++kk) {
            const int32_t a = op.act[static_cast<size_t>(i) * op.k + kk];
            const int8_t* w_row = &op.weights[static_cast<size_t>(kk) * op.n];
            int32_t* c_row = &op.want[static_cast<size_t>(i) * op.n];
            for (int j = 0; j < op.n; ++j) c_row[j] += a * w_row[j];
        }
}

std::string shape_text(const Operands& op) {
    return "M=" + std::to_string(op.m) + " K=" + std::to_string(op.k) + " N=" + std::to_string(op.n);
}

using CpuNamed = void (*)(const int8_t*, const uint8_t*, int32_t*, size_t, size_t, size_t);

void cpu_named_family() {
    const struct { CpuNamed fn; const char* name; bool needs_n8; } family[] = {
        {ternix::mul_mat_ternary_naive, "mul_mat_ternary_naive", false},
        {ternix::mul_mat_ternary_scalar, "mul_mat_ternary_scalar", false},
        {ternix::mul_mat_ternary_avx2, "mul_mat_ternary_avx2", true},
        {ternix::mul_mat_ternary_avx2_blocked, "mul_mat_ternary_avx2_blocked", true},
    };
    const int shapes[][3] = {{1, 8, 8}, {4, 16, 8}, {5, 33, 24}, {8, 64, 64}, {13, 100, 40}, {64, 256, 128}};
    for (const auto& f : family) {
        uint32_t seed = 1;
        for (const auto& s : shapes) {
            Operands op = draw(s[0], s[1], s[2], seed++, -127);
            fill_expected(op);
            std::vector<int32_t> got(op.want.size(), -999);
            f.fn(op.act.data(), op.packed.data(), got.data(), op.m, op.k, op.n);
            expect(got == op.want, std::string(f.name) + " " + shape_text(op));
        }
    }
    // int8 extremes over K = 4096 stay inside int32
    Operands op = draw(4, 4096, 16, 99, -127);
    for (int8_t& v : op.act) v = -128;
    fill_expected(op);
    std::vector<int32_t> got(op.want.size(), 0);
    ternix::mul_mat_ternary_avx2_blocked(op.act.data(), op.packed.data(), got.data(), op.m, op.k, op.n);
    expect(got == op.want, "extreme activations, K = 4096");
}

void cuda_host_wrapper() {
    const struct { int m, k, n; bool tiled; uint32_t seed; } cases[] = {
        {64, 64, 64, false, 1}, {37, 100, 52, false, 2}, {128, 512, 256, false, 3},
        {64, 64, 64, true, 4},  {128, 256, 192, true, 5}, {256, 1024, 512, true, 6}, {64, 4096, 64, true, 7},
    };
    for (const auto& c : cases) {
        Operands op = draw(c.m, c.k, c.n, c.seed, -128);
        fill_expected(op);
        std::vector<int32_t> got(op.want.size(), -1);
        const cudaError_t e = ternix::mul_mat_ternary_cuda_host(op.act.data(), op.packed.data(), got.data(), c.m, c.k, c.n, c.tiled);
        expect(e == cudaSuccess, std::string("mul_mat_ternary_cuda_host status, ") + shape_text(op));
        expect(got == op.want, std::string("mul_mat_ternary_cuda_host ") + (c.tiled ? "tiled " : "naive ") + shape_text(op));
    }
    // the wrapper with tiled = true keeps the multiple-of-64 contract of the tiled kernel
    Operands op = draw(37, 100, 52, 2, -128);
    std::vector<int32_t> got(static_cast<size_t>(37) * 52, -1);
    expect(ternix::mul_mat_ternary_cuda_host(op.act.data(), op.packed.data(), got.data(), 37, 100, 52, true) == cudaErrorInvalidValue,
           "mul_mat_ternary_cuda_host(tiled) rejects a ragged shape");
}

void cuda_device_pointers() {
    cudaStream_t stream = nullptr;
    expect(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess, "stream create");
    const struct { int m, k, n; bool tiled; uint32_t seed; } cases[] = {
        {64, 64, 64, false, 1}, {37, 100, 52, false, 2}, {128, 512, 256, false, 3}, {1, 2560, 6912, false, 8},
        {64, 64, 64, true, 4},  {128, 256, 192, true, 5}, {256, 1024, 512, true, 6}, {64, 4096, 64, true, 7},
    };
    for (const auto& c : cases) {
        Operands op = draw(c.m, c.k, c.n, c.seed, -128);
        fill_expected(op);
        int8_t* d_a = nullptr;
        uint8_t* d_w = nullptr;
        int32_t* d_c = nullptr;
        const size_t c_bytes = op.want.size() * sizeof(int32_t);
        bool ok = cudaMalloc(&d_a, op.act.size()) == cudaSuccess && cudaMalloc(&d_w, op.packed.size()) == cudaSuccess &&
                  cudaMalloc(&d_c, c_bytes) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(d_a, op.act.data(), op.act.size(), cudaMemcpyHostToDevice, stream) == cudaSuccess;
        ok = ok && cudaMemcpyAsync(d_w, op.packed.data(), op.packed.size(), cudaMemcpyHostToDevice, stream) == cudaSuccess;
        ok = ok && cudaMemsetAsync(d_c, 0xFF, c_bytes, stream) == cudaSuccess;
        expect(ok, "device buffers for " + shape_text(op));
        const cudaError_t launch = c.tiled ? ternix::mul_mat_ternary_cuda_tiled(d_a, d_w, d_c, c.m, c.k, c.n, stream)
                                           : ternix::mul_mat_ternary_cuda_naive(d_a, d_w, d_c, c.m, c.k, c.n, stream);
        expect(launch == cudaSuccess, std::string(c.tiled ? "mul_mat_ternary_cuda_tiled" : "mul_mat_ternary_cuda_naive") + " launch, " + shape_text(op));
        std::vector<int32_t> got(op.want.size(), -1);
        ok = cudaMemcpyAsync(got.data(), d_c, c_bytes, cudaMemcpyDeviceToHost, stream) == cudaSuccess &&
             cudaStreamSynchronize(stream) == cudaSuccess;
        expect(ok, "download for " + shape_text(op));
        expect(got == op.want, std::string(c.tiled ? "mul_mat_ternary_cuda_tiled " : "mul_mat_ternary_cuda_naive ") + shape_text(op));
        cudaFree(d_a);
        cudaFree(d_w);
        cudaFree(d_c);
    }
    // shape errors come back as cudaErrorInvalidValue without any memory access: null pointers are safe
    expect(ternix::mul_mat_ternary_cuda_tiled(nullptr, nullptr, nullptr, 65, 64, 64) == cudaErrorInvalidValue,
           "mul_mat_ternary_cuda_tiled rejects M = 65");
    expect(ternix::mul_mat_ternary_cuda_tiled(nullptr, nullptr, nullptr, 64, 64, 96) == cudaErrorInvalidValue,
           "mul_mat_ternary_cuda_tiled rejects N = 96");
    expect(ternix::mul_mat_ternary_cuda_naive(nullptr, nullptr, nullptr, 4, 8, 6, stream) == cudaErrorInvalidValue,
           "mul_mat_ternary_cuda_naive rejects N % 4 != 0");
    expect(ternix::mul_mat_ternary_cuda_naive(nullptr, nullptr, nullptr, -1, 8, 8, stream) == cudaErrorInvalidValue,
           "mul_mat_ternary_cuda_naive rejects a negative dimension");
    cudaStreamDestroy(stream);
}

void packed_format() {
    const std::vector<int8_t> original = {1, 0, -1, 1, -1, 0, 1, 0};
    std::vector<uint8_t> packed(2, 0xEE), copy(2, 0);
    ternix::pack_ternary_weights(packed.data(), original.data(), original.size());
    expect(packed[0] == 0x71 && packed[1] == 0x13, "pack_ternary_weights known-answer bytes 0x71 0x13");
    std::vector<int8_t> back(original.size(), 99);
    ternix::unpack_ternary_weights(back.data(), packed.data(), original.size());
    expect(back == original, "unpack_ternary_weights round trip");
    ternix::interleave_weights_offline(copy.data(), packed.data(), original.size());
    expect(copy == packed, "interleave_weights_offline is the identity layout");
    // a tail of size % 4 weights is dropped: only size / 4 bytes are written
    std::vector<int8_t> six = {1, 1, 1, 1, -1, -1};
    std::vector<uint8_t> out(2, 0xAB);
    ternix::pack_ternary_weights(out.data(), six.data(), six.size());
    expect(out[0] == 0x55 && out[1] == 0xAB, "pack_ternary_weights drops the tail of size % 4");
}

}  // namespace

int main() {
    int devices = 0;
    if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) {
        std::printf("boundary_check: no CUDA device (the product path has no CPU fallback)\n");
        return 2;
    }
    packed_format();
    try {
        cpu_named_family();
    } catch (const std::exception& e) {
        expect(false, std::string("CPU-named entry point threw: ") + e.what());
    }
    cuda_host_wrapper();
    cuda_device_pointers();
    if (g_failures) {
        std::printf("boundary_check: FAIL (%d of %d checks)\n", g_failures, g_checks);
        return 1;
    }
    std::printf("boundary_check: PASS (%d checks)\n", g_checks);
    return 0;
}
