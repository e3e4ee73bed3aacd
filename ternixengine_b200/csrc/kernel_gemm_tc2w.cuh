// Prefill-regime kernel, paired CTAs, wide tiles: 256 x 512 outputs per cluster of two CTAs.
//
// Why wider.  ternary_gemm_tc2_kernel (256 x 256 per pair) is bound by the latency of its own ring: a
// stage of A + packed W is held from TMA issue until the MMAs that read it retire, about 3,000 to 3,700
// cycles (TMA from L2, expander wake-up, expansion, remote arrive, MMA, commit), while the stages that
// fit in shared memory cover only about 2,700 cycles of tensor-core work.  With 512 columns per pair each
// byte of A feeds twice as many MACs, so the same ring covers about 4,300 cycles.  Each CTA loads its 128
// rows of A and its 256 columns of packed W per 128-deep k-block, expands them into two 128-column
// operand groups, and the leader issues two N=256 pair MMAs per 32-deep step (group h of both CTAs forms
// the B operand of MMA h).  The accumulator is 512 TMEM columns per CTA, single-buffered: the epilogue of
// a tile runs before the next tile's first MMA (about 7 % of a tile's time at K = 8192).
//
// Tail.  Tiles are dealt to the pairs round-robin, so a last, partial round would keep a few pairs busy for
// a whole tile while the rest idle (896 tiles on 74 pairs: 12.1 rounds).  When the host asks for it, the
// tiles of that partial round are split along K into slices, one slice per pair; every slice adds its
// partial result into C with red.global.add.s32 (C of those tiles is zeroed by the host beforehand).
// Integer addition is associative and each partial accumulator is an exact multiple of 64, so the result is
// bit-identical.
//
// Everything else -- decode, operand layouts, pair signalling, coalesced multi-destination epilogue,
// bounded waits -- is as in ternary_gemm_tc2_kernel.  Single product only (no problem-group tables).
#pragma once
#include <cuda.h>
#include <cstdint>
#include "kernel_gemm_tc2.cuh"

namespace tb200 {

constexpr int kTcwStagesA = 4;                                   // {A 16 KB + packed W 8 KB}
constexpr int kTcwStagesB = 3;                                   // expanded B, 2 groups x 16 KB
constexpr int kTcwTileN = 512;
constexpr int kTcwCtaN = 256;                                    // columns loaded and expanded per CTA
constexpr int kTcwGroups = 2;                                    // expander groups (k-blocks g mod 2)

struct TcwGeom {
    static constexpr int kABytes = kTcBM * kTcBK;                // 16384
    static constexpr int kWpRowBytes = kTcwCtaN / 4;             // 64
    static constexpr int kWpBytes = kTcBK * kWpRowBytes;         // 8192
    static constexpr int kGroupBytes = 128 * kTcBK;              // one 128-column operand group: 16384
    static constexpr int kBBytes = 2 * kGroupBytes;              // 32768
    static constexpr int kQuadsPerRow = kTcwCtaN / 64;           // 4
    static constexpr int kQuads = kTcBK * kQuadsPerRow;          // 512
    static constexpr int kGroupThreads = kTcExpandWarps * 32 / kTcwGroups;   // 128
    static constexpr int kGroupWarps = kTcExpandWarps / kTcwGroups;          // 4
    static constexpr int kQuadsPerThread = kQuads / kGroupThreads;           // 4
    static constexpr uint32_t kTmemCols = 512;
    static constexpr int kEpiBytes = 32 * 64 * 4;
    static constexpr size_t kSmemBytes = 1024 + size_t(kTcwStagesA) * (kABytes + kWpBytes) +
                                         size_t(kTcwStagesB) * kBBytes + 4 * kEpiBytes + 512;
    static constexpr uint32_t kIdesc = Tc2Geom::kIdesc;          // M = 256 (pair), N = 256 per instruction
};

__global__ void __launch_bounds__(kTc2Threads, 1)
ternary_gemm_tc2w_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ Tc2Dest dest, int M, int K, int N, long long ldc, int c_vec_ok,
                         int tail_slices, int32_t* __restrict__ status) {
    using G = TcwGeom;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = base;                                              // [StagesA][128][128]  swizzled
    uint8_t* sB = sA + kTcwStagesA * G::kABytes;                     // [StagesB][2 groups][128 k][128]  swizzled
    uint8_t* sWp = sB + kTcwStagesB * G::kBBytes;                    // [StagesA][128 k][64]
    uint8_t* sEpi = sWp + kTcwStagesA * G::kWpBytes;                 // [4 warps][32 rows][64 cols] int32, swizzled
    uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + 4 * G::kEpiBytes);
    uint64_t* full_a = bars;
    uint64_t* empty_a = full_a + kTcwStagesA;
    uint64_t* full_b = empty_a + kTcwStagesA;
    uint64_t* empty_b = full_b + kTcwStagesB;
    uint64_t* tmem_full = empty_b + kTcwStagesB;                     // [1]
    uint64_t* tmem_empty = tmem_full + 1;                            // [1]
    uint64_t* drain = tmem_empty + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int m_tiles = (M + 2 * kTcBM - 1) / (2 * kTcBM);
    const int n_tiles = (N + kTcwTileN - 1) / kTcwTileN;
    const int num_tiles = m_tiles * n_tiles;
    const int k_blocks = (K + kTcBK - 1) / kTcBK;
    // Work items of this pair: its whole tiles, then (tail_slices > 0) one K-slice of a tile of the last round.
    const int whole_tiles = tail_slices > 0 ? (num_tiles / num_pairs) * num_pairs : num_tiles;
    const int slice_kb = tail_slices > 0 ? (k_blocks + tail_slices - 1) / tail_slices : 0;
    const bool has_slice = tail_slices > 0 && pair < (num_tiles - whole_tiles) * tail_slices &&
                           (pair % tail_slices) * slice_kb < k_blocks;
    const int n_whole = pair < whole_tiles ? (whole_tiles - pair + num_pairs - 1) / num_pairs : 0;
    const int n_items = n_whole + (has_slice ? 1 : 0);
    // item i -> tile and k-block range
    auto item = [&](int i, int& tile, int& kb0, int& kb1) {
        if (i < n_whole) { tile = pair + i * num_pairs; kb0 = 0; kb1 = k_blocks; }
        else {
            tile = whole_tiles + pair / tail_slices;
            kb0 = (pair % tail_slices) * slice_kb;
            kb1 = kb0 + slice_kb < k_blocks ? kb0 + slice_kb : k_blocks;
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcwStagesA; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&empty_a[s], G::kGroupWarps + 1);
        }
        for (int s = 0; s < kTcwStagesB; ++s) {
            mbar_init(&full_b[s], 2 * G::kGroupWarps);
            mbar_init(&empty_b[s], 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, 8);
        mbar_init(drain, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc_pair<G::kTmemCols>(tmem_slot);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ================================================================ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_w);
            uint32_t it = 0;
            bool ok = true;
            for (int i = 0; ok && i < n_items; ++i) {
                int tile, kb0, kb1;
                item(i, tile, kb0, kb1);
                const int m_t = tile % m_tiles, n_t = tile / m_tiles;
                const int row0 = m_t * 2 * kTcBM + rank * kTcBM;
                const int wp_x = n_t * (kTcwTileN / 4) + rank * G::kWpRowBytes;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t s = it % kTcwStagesA;
                    if (!mbar_wait(&empty_a[s], ((it / kTcwStagesA) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full_a[s], G::kABytes + G::kWpBytes);
                    tma_load_2d(sA + s * G::kABytes, &tmap_a, kb * kTcBK, row0, &full_a[s]);
                    tma_load_2d(sWp + s * G::kWpBytes, &tmap_w, wp_x, kb * kTcBK, &full_a[s]);
                }
            }
            if (!ok) {
                const uint32_t first = it > kTcwStagesA ? it - kTcwStagesA : 0;
                for (uint32_t j = first; j < it; ++j) mbar_drain(&full_a[j % kTcwStagesA], (j / kTcwStagesA) & 1);
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer (leader CTA only)
        if (leader && lane == 0) {
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (int i = 0; ok && i < n_items; ++i, ++lt) {
                int tile, kb0, kb1;
                item(i, tile, kb0, kb1);
                if (!mbar_wait(tmem_empty, (lt & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const uint32_t sa = it % kTcwStagesA, sb = it % kTcwStagesB;
                    if (!mbar_wait(&full_a[sa], (it / kTcwStagesA) & 1, abort_flag) ||
                        !mbar_wait(&full_b[sb], (it / kTcwStagesB) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(sA + sa * G::kABytes);
                    const uint32_t b_addr = smem_u32(sB + sb * G::kBBytes);
#pragma unroll
                    for (int k4 = 0; k4 < kTcBK / 32; ++k4) {
                        const uint64_t da = umma_desc_sw128(a_addr + k4 * 32, 16, 1024);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint64_t db = umma_desc_sw128(b_addr + h * G::kGroupBytes + k4 * 4096, G::kGroupBytes, 1024);
                            tc_mma_i8_pair(tmem_base + h * 256, da, db, G::kIdesc, (kb != kb0 || k4 != 0) ? 1u : 0u);
                        }
                    }
                    tc_commit_pair_both(&empty_a[sa]);
                    tc_commit_pair_both(&empty_b[sb]);
                }
                if (ok) tc_commit_pair_both(tmem_full);
            }
            tc_commit_pair(drain);
            mbar_wait(drain, 0, abort_flag);
        }
    } else if (warp < kTcFirstEpilogueWarp) {
        // ================================================================ expanders: this CTA's 256 columns
        const int e = threadIdx.x - kTcFirstExpandWarp * 32;          // 0..255
        const uint32_t group = e / G::kGroupThreads;
        const int eg = e % G::kGroupThreads;
        uint32_t src_off[G::kQuadsPerThread], dst_off[G::kQuadsPerThread][4];
        bool rot[G::kQuadsPerThread];
#pragma unroll
        for (int i = 0; i < G::kQuadsPerThread; ++i) {
            const int idx = eg + i * G::kGroupThreads;
            const int q = idx % G::kQuadsPerRow, k = idx / G::kQuadsPerRow;
            src_off[i] = idx * 16;
            rot[i] = (q & 2) != 0;     // upper two quads store their words in rotated order: no bank conflicts
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int uu = rot[i] ? (u ^ 2) : u;
                const int col16 = q * 4 + uu;                          // 16-column chunk inside the 256 columns
                const int g = col16 >> 3, c = col16 & 7;
                dst_off[i][u] = g * G::kGroupBytes + k * 128 + ((c ^ (k & 7)) << 4);
            }
        }
        const uint32_t wp_sa = smem_u32(sWp), b_sa = smem_u32(sB);
        uint32_t it = 0;
        bool ok = true;
        for (int i = 0; ok && i < n_items; ++i) {
            int tile, kb0, kb1;
            item(i, tile, kb0, kb1);
            for (int kb = kb0; kb < kb1; ++kb, ++it) {
                const uint32_t sa = it % kTcwStagesA, sb = it % kTcwStagesB;
                // every expander warp observes every phase of full_a (parity waits must not skip phases)
                if (!mbar_wait(&full_a[sa], (it / kTcwStagesA) & 1, abort_flag)) { ok = false; break; }
                if (it % kTcwGroups != group) continue;
                if (!mbar_wait(&empty_b[sb], ((it / kTcwStagesB) & 1) ^ 1, abort_flag)) { ok = false; break; }
                const uint32_t wp = wp_sa + sa * G::kWpBytes;
                const uint32_t bt = b_sa + sb * G::kBBytes;
                uint4 v[G::kQuadsPerThread];
#pragma unroll
                for (int i = 0; i < G::kQuadsPerThread; ++i) v[i] = lds_v4(wp + src_off[i]);
#pragma unroll
                for (int i = 0; i < G::kQuadsPerThread; ++i) {
                    if (rot[i]) { uint32_t t0 = v[i].x; v[i].x = v[i].z; v[i].z = t0; t0 = v[i].y; v[i].y = v[i].w; v[i].w = t0; }
                    const uint32_t words[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
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
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(&full_b[sb]);
                    else mbar_arrive_remote(&full_b[sb], 0);
                    mbar_arrive(&empty_a[sa]);
                }
            }
        }
    } else {
        // ================================================================ epilogue: this CTA's 128 rows x 512 columns
        const int quad = warp & 3;
        const uint32_t stage_sa = smem_u32(sEpi) + (warp - kTcFirstEpilogueWarp) * G::kEpiBytes;
        const uint32_t my_row_sa = stage_sa + lane * 256;
        const int n_dest = dest.count;
        uint32_t lt = 0;
        bool ok = true;
        for (int i = 0; ok && i < n_items; ++i, ++lt) {
            int tile, kb0, kb1;
            item(i, tile, kb0, kb1);
            const bool add_into_c = i >= n_whole;                      // a K-slice: partial result, C was zeroed
            const int m_t = tile % m_tiles, n_t = tile / m_tiles;
            if (!mbar_wait(tmem_full, lt & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const int row_base = m_t * 2 * kTcBM + rank * kTcBM + quad * 32;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < kTcwTileN; c0 += 64) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t r[32];
                    tmem_ld_32x32(t_addr + c0 + 32 * h, r);
                    tmem_ld_wait();
                    int32_t o[32];
#pragma unroll
                    for (int g = 0; g < 2; ++g)
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            o[g * 16 + 4 * (i & 3) + (i >> 2)] = static_cast<int32_t>(r[g * 16 + i]) >> 6;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int chunk = h * 8 + j;
                        sts_v4(my_row_sa + ((chunk ^ (lane & 7)) << 4),
                               make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]));
                    }
                }
                __syncwarp();
                // TMEM column c0 = mma*256 + cta*128 + j  <->  global column n_t*512 + cta*256 + mma*128 + j
                const int col0 = n_t * kTcwTileN + ((c0 >> 7) & 1) * 256 + (c0 >> 8) * 128 + (c0 & 127);
                const int col = col0 + (lane & 15) * 4;
#pragma unroll 4
                for (int i = 0; i < 16; ++i) {
                    const int rr = 2 * i + (lane >> 4);
                    const uint4 v = lds_v4(stage_sa + rr * 256 + (((lane & 15) ^ (rr & 7)) << 4));
                    const int row = row_base + rr;
                    if (row < M && col < N && add_into_c) {
                        int32_t* out = dest.c[0] + static_cast<size_t>(row) * ldc + col;
                        asm volatile("red.global.add.s32 [%0], %1;" ::"l"(out), "r"(v.x) : "memory");
                        asm volatile("red.global.add.s32 [%0], %1;" ::"l"(out + 1), "r"(v.y) : "memory");
                        asm volatile("red.global.add.s32 [%0], %1;" ::"l"(out + 2), "r"(v.z) : "memory");
                        asm volatile("red.global.add.s32 [%0], %1;" ::"l"(out + 3), "r"(v.w) : "memory");
                    } else if (row < M && col < N) {
                        const size_t off = static_cast<size_t>(row) * ldc + col;
#pragma unroll
                        for (int d = 0; d < kTc2MaxDest; ++d) {
                            if (d >= n_dest) break;
                            int32_t* out = dest.c[d] + off;
                            if (c_vec_ok) {
                                *reinterpret_cast<uint4*>(out) = v;
                            } else {
                                out[0] = static_cast<int32_t>(v.x);
                                out[1] = static_cast<int32_t>(v.y);
                                out[2] = static_cast<int32_t>(v.z);
                                out[3] = static_cast<int32_t>(v.w);
                            }
                        }
                    }
                }
                __syncwarp();
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(tmem_empty);
                else mbar_arrive_remote(tmem_empty, 0);
            }
        }
    }

    __syncwarp();
    if (*abort_flag && lane == 0 && status) atomicMax(status, kStatusTimeout);
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair<G::kTmemCols>(tmem_base);
    }
}

}  // namespace tb200
