// Prefill-regime kernel: dense contraction on the 5th-generation tensor cores.
//
//   C[M,N] int32 = A[M,K] int8 x W[K,N] ternary (packed)      tcgen05.mma kind::i8, int32 in TMEM
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 256 or 128).  Warp roles:
//   warp 0        TMA producer: per 128-deep k-block one box of A (128 rows x 128 B, 128-byte
//                 swizzle, K-major) and one box of PACKED W (128 k-rows x BN/4 bytes).
//   warps 2..9    expanders: read packed words from shared memory, turn every 2-bit field into
//                 an int8 byte and write the B operand tile in the tensor core's N-major
//                 ("MN-major") 128-byte-swizzled layout.  One packed word (16 columns of one
//                 k-row) becomes exactly one 16-byte swizzle chunk: word j of the chunk is
//                 (w << (6-2j)) & 0xC0C0C0C0, i.e. bytes 0x00/0x40/0xC0 = 0/+64/-64.  Shift and
//                 mask only: no branch, no lookup, no dequantised tensor in global memory.
//                 Inside each 16-column chunk the tensor core therefore sees the columns in the
//                 order 0,4,8,12, 1,5,9,13, ...; the epilogue undoes that while it holds the
//                 values in registers, and shifts the 64x-scaled sums right by 6 (exact).
//   warp 1        MMA issuer: one lane issues 4 x (128 x BN x 32) MMAs per k-block into one of two
//                 TMEM accumulator buffers and commits to the barriers that free the stages.
//   warps 10..13  epilogue: tcgen05.ld the finished accumulator (its own 32-lane quadrant),
//                 >> 6, un-permute, store C.  Runs under the main loop of the next tile.
//
// Exactness: int8 x int8 products accumulated in int32, |64 * a * w| * K < 2^31 for K < 262144
// (checked by the host).  TMA zero-fills rows beyond M, k beyond K and columns beyond N, and a
// zero activation or a 00 weight code contributes nothing, so ragged edges need no special code
// in the main loop; stores are predicated.
//
// Every mbarrier wait is bounded; on a timeout the CTA stops issuing work, waits (bounded) for
// the copies and MMAs it has in flight, frees its TMEM and returns with the status word set.
#pragma once
#include <cuda.h>
#include <cstdint>
#include "ptx_sm100.cuh"

namespace tb200 {

constexpr int kTcBM = 128;
constexpr int kTcBK = 128;
constexpr int kTcStagesA = 4;          // ring of {A box, packed-W box}
constexpr int kTcStagesB = 3;          // ring of expanded B tiles
constexpr int kTcExpandWarps = 8;
constexpr int kTcFirstExpandWarp = 2;
constexpr int kTcFirstEpilogueWarp = kTcFirstExpandWarp + kTcExpandWarps;   // 10
constexpr int kTcThreads = (kTcFirstEpilogueWarp + 4) * 32;                 // 448

template <int BN>
struct TcGeom {
    static constexpr int kABytes = kTcBM * kTcBK;              // 16384
    static constexpr int kWpRowBytes = BN / 4;                 // 64 or 32
    static constexpr int kWpBytes = kTcBK * kWpRowBytes;       // 8192 or 4096
    static constexpr int kBBytes = BN * kTcBK;                 // 32768 or 16384
    static constexpr int kGroupBytes = 128 * kTcBK;            // one 128-column group of B: 16384
    static constexpr int kQuadsPerRow = BN / 64;               // 16-byte packed quads per k-row
    static constexpr int kQuads = kTcBK * kQuadsPerRow;        // 512 or 256
    static constexpr int kQuadsPerThread = kQuads / (kTcExpandWarps * 32);
    static constexpr uint32_t kTmemCols = 2 * BN;              // two accumulator buffers
    static constexpr size_t kSmemBytes = 1024 + size_t(kTcStagesA) * (kABytes + kWpBytes) +
                                         size_t(kTcStagesB) * kBBytes + 256;
    // instruction descriptor: D = s32, A = B = s8, A K-major, B MN-major, N = BN, M = 128
    static constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) |
                                       (uint32_t(BN >> 3) << 17) | (uint32_t(kTcBM >> 4) << 24);
    static_assert(kQuadsPerThread >= 1, "expand work must cover the expand warps");
};

template <int BN>
__global__ void __launch_bounds__(kTcThreads, 1)
ternary_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                       int32_t* __restrict__ C, int M, int K, int N, long long ldc, int c_vec_ok, int k_slices,
                       int32_t* __restrict__ status) {
    using G = TcGeom<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = base;                                              // [kTcStagesA][128][128]  swizzled
    uint8_t* sB = sA + kTcStagesA * G::kABytes;                      // [kTcStagesB][BN/128][128 k][128]  swizzled
    uint8_t* sWp = sB + kTcStagesB * G::kBBytes;                     // [kTcStagesA][128 k][BN/4]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sWp + kTcStagesA * G::kWpBytes);
    uint64_t* full_a = bars;                                         // TMA -> expanders + MMA
    uint64_t* empty_a = full_a + kTcStagesA;                         // expanders + MMA -> TMA
    uint64_t* full_b = empty_a + kTcStagesA;                         // expanders -> MMA
    uint64_t* empty_b = full_b + kTcStagesB;                         // MMA -> expanders
    uint64_t* tmem_full = empty_b + kTcStagesB;                      // MMA -> epilogue   [2]
    uint64_t* tmem_empty = tmem_full + 2;                            // epilogue -> MMA   [2]
    uint64_t* drain = tmem_empty + 2;                                // MMA teardown
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + kTcBM - 1) / kTcBM;
    const int n_tiles = (N + BN - 1) / BN;
    const int k_blocks = (K + kTcBK - 1) / kTcBK;
    // With few output tiles (skinny M) every tile is split along K into k_slices work items so that all SMs
    // stream weights; the items of a tile add their partial results into C (zeroed by the host): integer
    // adds are associative and every partial accumulator is an exact multiple of 64, so C stays bit-exact.
    const int slice_kb = (k_blocks + k_slices - 1) / k_slices;
    const int num_tiles = m_tiles * n_tiles * k_slices;              // work items
    const bool add_into_c = k_slices > 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStagesA; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&empty_a[s], kTcExpandWarps + 1);
        }
        for (int s = 0; s < kTcStagesB; ++s) {
            mbar_init(&full_b[s], kTcExpandWarps);
            mbar_init(&empty_b[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 4);
        }
        mbar_init(drain, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc<G::kTmemCols>(tmem_slot);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ================================================================ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_w);
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int slice = tile % k_slices, t2 = tile / k_slices;
                const int m_t = t2 % m_tiles, n_t = t2 / m_tiles;
                const int kb0 = slice * slice_kb, kb1 = kb0 + slice_kb < k_blocks ? kb0 + slice_kb : k_blocks;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % kTcStagesA;
                    if (!mbar_wait(&empty_a[s], ((it / kTcStagesA) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full_a[s], G::kABytes + G::kWpBytes);
                    tma_load_2d(sA + s * G::kABytes, &tmap_a, kb * kTcBK, m_t * kTcBM, &full_a[s]);
                    tma_load_2d(sWp + s * G::kWpBytes, &tmap_w, n_t * G::kWpRowBytes, kb * kTcBK, &full_a[s]);
                }
            }
            if (!ok) {
                // let the boxes already issued land before the CTA may exit
                const uint32_t first = it > kTcStagesA ? it - kTcStagesA : 0;
                for (uint32_t j = first; j < it; ++j)
                    mbar_drain(&full_a[j % kTcStagesA], (j / kTcStagesA) & 1);
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++lt) {
                const uint32_t acc = lt & 1;
                if (!mbar_wait(&tmem_empty[acc], ((lt >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int slice = tile % k_slices;
                const int kb0 = slice * slice_kb, kb1 = kb0 + slice_kb < k_blocks ? kb0 + slice_kb : k_blocks;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t sa = it % kTcStagesA, sb = it % kTcStagesB;
                    if (!mbar_wait(&full_a[sa], (it / kTcStagesA) & 1, abort_flag) ||
                        !mbar_wait(&full_b[sb], (it / kTcStagesB) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(sA + sa * G::kABytes);
                    const uint32_t b_addr = smem_u32(sB + sb * G::kBBytes);
#pragma unroll
                    for (int k4 = 0; k4 < kTcBK / 32; ++k4) {
                        // A: K-major, rows of 128 B, 8-row groups 1024 B apart; +32 B per 32-deep step.
                        const uint64_t da = umma_desc_sw128(a_addr + k4 * 32, 16, 1024);
                        // B: N-major, 128-column groups kGroupBytes apart (leading), 8-k-row groups
                        //    1024 B apart (stride); +32 k-rows = 4096 B per step.
                        const uint64_t db = umma_desc_sw128(b_addr + k4 * 4096, G::kGroupBytes, 1024);
                        tc_mma_i8(d_tmem, da, db, G::kIdesc, (kb != kb0 || k4 != 0) ? 1u : 0u);
                    }
                    tc_commit(&empty_a[sa]);
                    tc_commit(&empty_b[sb]);
                }
                if (ok) tc_commit(&tmem_full[acc]);
            }
            // teardown: every MMA issued by this thread must have retired before TMEM is freed
            tc_commit(drain);
            mbar_wait(drain, 0, abort_flag);
        }
    } else if (warp < kTcFirstEpilogueWarp) {
        // ================================================================ expanders
        const int e = threadIdx.x - kTcFirstExpandWarp * 32;          // 0..255
        // Per-thread constants: where each of this thread's packed quads is read, and where the
        // four 16-byte chunks it expands to are written (offsets inside a stage).
        uint32_t src_off[G::kQuadsPerThread], dst_off[G::kQuadsPerThread][4];
        bool rot[G::kQuadsPerThread];
#pragma unroll
        for (int i = 0; i < G::kQuadsPerThread; ++i) {
            const int idx = e + i * (kTcExpandWarps * 32);
            const int q = idx % G::kQuadsPerRow;               // which 64-column quad of the k-row
            const int k = idx / G::kQuadsPerRow;               // k-row inside the block
            src_off[i] = idx * 16;
            // For BN = 256 the upper two quads of a row rotate their store order by two words, so
            // that the eight lanes of a quarter-warp hit eight different 16-byte bank groups.
            rot[i] = (G::kQuadsPerRow == 4) && (q & 2);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int uu = rot[i] ? (u ^ 2) : u;           // which word of the quad is stored u-th
                const int col16 = q * 4 + uu;                  // 16-column chunk inside the tile
                const int g = col16 >> 3, c = col16 & 7;
                dst_off[i][u] = g * G::kGroupBytes + k * 128 + ((c ^ (k & 7)) << 4);
            }
        }
        const uint32_t wp_sa = smem_u32(sWp), b_sa = smem_u32(sB);
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            const int slice = tile % k_slices;
            const int kb0 = slice * slice_kb, kb1 = kb0 + slice_kb < k_blocks ? kb0 + slice_kb : k_blocks;
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t sa = it % kTcStagesA, sb = it % kTcStagesB;
                if (!mbar_wait(&full_a[sa], (it / kTcStagesA) & 1, abort_flag) ||
                    !mbar_wait(&empty_b[sb], ((it / kTcStagesB) & 1) ^ 1, abort_flag)) { ok = false; break; }
                const uint32_t wp = wp_sa + sa * G::kWpBytes;
                const uint32_t bt = b_sa + sb * G::kBBytes;
#pragma unroll
                for (int i = 0; i < G::kQuadsPerThread; ++i) {
                    uint4 v = lds_v4(wp + src_off[i]);
                    if (rot[i]) { uint32_t t0 = v.x; v.x = v.z; v.z = t0; t0 = v.y; v.y = v.w; v.w = t0; }
                    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t w = words[u];
                        uint4 o;
                        o.x = (w << 6) & 0xC0C0C0C0u;
                        o.y = (w << 4) & 0xC0C0C0C0u;
                        o.z = (w << 2) & 0xC0C0C0C0u;
                        o.w = w & 0xC0C0C0C0u;
                        sts_v4(bt + dst_off[i][u], o);
                    }
                }
                fence_proxy_async_smem();          // generic-proxy stores -> visible to the tensor core
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full_b[sb]);
                    mbar_arrive(&empty_a[sa]);
                }
            }
        }
    } else {
        // ================================================================ epilogue
        const int quad = warp & 3;                                     // TMEM lane quadrant of this warp
        uint32_t lt = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++lt) {
            const int t2 = tile / k_slices;
            const int m_t = t2 % m_tiles, n_t = t2 / m_tiles;
            const uint32_t acc = lt & 1;
            if (!mbar_wait(&tmem_full[acc], (lt >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const int row = m_t * kTcBM + quad * 32 + lane;
            int32_t* crow = C + static_cast<size_t>(row) * ldc + static_cast<size_t>(n_t) * BN;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(t_addr + c0, r);
                tmem_ld_wait();
                if (row < M && n_t * BN + c0 < N) {
                    int32_t o[32];
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            o[h * 16 + 4 * (i & 3) + (i >> 2)] = static_cast<int32_t>(r[h * 16 + i]) >> 6;
                    if (add_into_c) {
#pragma unroll
                        for (int v = 0; v < 32; ++v)
                            asm volatile("red.global.add.s32 [%0], %1;" ::"l"(crow + c0 + v), "r"(o[v]) : "memory");
                    } else if (c_vec_ok) {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            *reinterpret_cast<int4*>(crow + c0 + 4 * v) =
                                make_int4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
                    } else {
#pragma unroll
                        for (int v = 0; v < 32; ++v) crow[c0 + v] = o[v];
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        }
    }

    __syncwarp();
    if (*abort_flag && lane == 0 && status) atomicMax(status, kStatusTimeout);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<G::kTmemCols>(tmem_base);
    }
}

}  // namespace tb200
