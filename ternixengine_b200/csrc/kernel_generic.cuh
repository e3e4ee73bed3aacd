// Generic exact kernel: any M >= 1, K >= 1, N % 4 == 0, any row pitch, any pointer alignment.
//
// This is the path for shapes whose packed rows are not 16-byte multiples (TMA cannot describe
// them) and for K so deep that the scaled accumulators of the fast kernels could overflow.  It
// uses byte loads with predicated tails only, plain int32 multiply-adds and no scaling, so it has
// no limits beyond int32 itself (|C| <= 128*K < 2^31 for K < 2^24).
//
// CTA = 32 x 8 threads, output tile 32 rows x 128 columns, K walked in slabs of 64 through
// shared memory.  Thread (tx, ty) owns rows 4*ty..4*ty+3 and the four columns of packed byte tx.
// Problems with few output tiles (ragged decode shapes: a handful of rows, a thousand columns) are cut along K
// over blockIdx.z; the slices then add into a C that the host has zeroed (integer adds: still exact).
#pragma once
#include <cstdint>

namespace tb200 {

constexpr int kGenRows = 32;    // rows of C per CTA
constexpr int kGenBytes = 32;   // packed bytes (x4 columns) per CTA
constexpr int kGenK = 64;       // k-slab
constexpr int kGenThreads = 256;

__global__ void __launch_bounds__(kGenThreads)
ternary_generic_kernel(const int8_t* __restrict__ A, const uint8_t* __restrict__ W, int32_t* __restrict__ C,
                       int M, int K, int N, long long ldc, int k_per_slice) {
    __shared__ __align__(16) int8_t sA[kGenRows][kGenK];
    __shared__ __align__(16) uint8_t sW[kGenK][kGenBytes];

    const int tx = threadIdx.x & 31;
    const int ty = threadIdx.x >> 5;
    const int tid = threadIdx.x;
    const int pitch = N >> 2;                         // packed bytes per k-row
    const int row0 = blockIdx.y * kGenRows;
    const int byte0 = blockIdx.x * kGenBytes;

    int32_t acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0;

    // staging assignments: 2048 bytes of each tile, 8 per thread
    const int a_row = tid >> 3, a_k = (tid & 7) * 8;
    const int w_k = tid >> 2, w_b = (tid & 3) * 8;

    // this CTA's k-range: all of K, or slice blockIdx.z of it (k_per_slice is a multiple of the slab)
    const bool sliced = gridDim.z > 1;
    const int k_begin = sliced ? static_cast<int>(blockIdx.z) * k_per_slice : 0;
    const int k_end = sliced ? min(K, k_begin + k_per_slice) : K;

    for (int k0 = k_begin; k0 < k_end; k0 += kGenK) {
        {
            const int grow = row0 + a_row;
            const int8_t* src = A + static_cast<size_t>(grow) * K + k0 + a_k;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                sA[a_row][a_k + i] = (grow < M && k0 + a_k + i < k_end) ? src[i] : int8_t(0);
            const int gk = k0 + w_k;
            const uint8_t* wsrc = W + static_cast<size_t>(gk) * pitch + byte0 + w_b;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                sW[w_k][w_b + i] = (gk < k_end && byte0 + w_b + i < pitch) ? wsrc[i] : uint8_t(0);
        }
        __syncthreads();

#pragma unroll 4
        for (int kk = 0; kk < kGenK; kk += 4) {
            int a4[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) a4[r] = *reinterpret_cast<const int*>(&sA[ty * 4 + r][kk]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int wb = sW[kk + q][tx];
                int w[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) w[c] = (wb << (30 - 2 * c)) >> 30;   // 00->0, 01->+1, 11->-1
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int a = (a4[r] << (24 - 8 * q)) >> 24;                 // sign-extended byte q
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[r][c] += a * w[c];
                }
            }
        }
        __syncthreads();
    }

    const int col = (byte0 + tx) * 4;
    if (col < N) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = row0 + ty * 4 + r;
            if (row < M) {
                int32_t* out = C + static_cast<size_t>(row) * ldc + col;
                if (sliced) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) atomicAdd(out + c, acc[r][c]);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) out[c] = acc[r][c];
                }
            }
        }
    }
}

}  // namespace tb200
