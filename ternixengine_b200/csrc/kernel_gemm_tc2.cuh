// Prefill-regime kernel, paired CTAs: tcgen05.mma.cta_group::2 on 256 x 256 output tiles.
//
// Why pairs.  With one CTA per tile the main loop moves about 112 KB through shared memory per
// 128-deep k-block (TMA fills, expander read + write, tensor-core operand reads) and that, not
// the tensor pipe, is what bounds ternary_gemm_tc_kernel.  Two CTAs of a cluster (the two SMs of
// a TPC) share one 256 x 256 tile: each loads its own 128 rows of A, and each loads, expands
// and serves only ITS 128 columns of W; the pair's MMA reads both halves.  Expander work and
// expanded-tile traffic per SM halve.
//
// Roles per CTA (448 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only; both
// CTAs' warp 1 allocate and free TMEM), warps 2..9 expanders, warps 10..13 epilogue.
// Cross-CTA signalling:
//   peer expanders  -> leader full_b[s]      remote mbarrier arrive (16 arrivals = 8 local + 8 remote;
//                                              a peer arrival also implies the peer's A box of that
//                                              k-block has landed, because its expanders waited on
//                                              the same TMA barrier)
//   peer epilogue   -> leader tmem_empty[a]  remote mbarrier arrive (8 arrivals)
//   leader MMA      -> empty_a / empty_b / tmem_full of BOTH CTAs: one tcgen05.commit per barrier whose
//                      arrive is delivered to the same barrier offset in both CTAs of the pair.
// TMA loads are ordinary per-CTA loads into the CTA's own shared memory.
//
// Epilogue.  Each epilogue warp turns its 32 rows x 64 columns of the accumulator into row-contiguous
// 256-byte segments through a small swizzled staging tile in shared memory, so that a warp store
// covers whole 256-byte pieces of two rows instead of 16 bytes of 32 rows.  The same segments can be
// written to several destinations: the local C and, when the weights are column-sharded over GPUs, the
// same columns of C in every peer GPU's memory (plain stores through peer-mapped pointers), which
// replaces a separate all-gather and overlaps the transfer with the next tile's main loop.
//
// Dequantising epilogue (kBf16).  The step after this product in a BitNet-style layer multiplies the integer
// result by the activation row's scale and the weight tensor's scale.  With kBf16 the epilogue does that in
// fp32 -- y = bf16_rn((float(c) * row_scale[m]) * w_scale) -- and stores bfloat16, half the bytes of int32, which
// also halves what a fused gather ships over NVLink.  The integer accumulation before it is unchanged and exact.
//
// Decode, layouts, exactness and bounded waits are those of ternary_gemm_tc_kernel.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "kernel_gemm_tc.cuh"
#include "ptx_sm100.cuh"

namespace tb200 {

#ifndef TB200_TC2_STAGES_A
#define TB200_TC2_STAGES_A 5
#endif
#ifndef TB200_TC2_STAGES_B
#define TB200_TC2_STAGES_B 5
#endif
#ifndef TB200_TC2_EXPAND_GROUPS
#define TB200_TC2_EXPAND_GROUPS 4
#endif
constexpr int kTc2StagesA = TB200_TC2_STAGES_A;     // ring of {A box, packed-W box}: 20 KB per stage
constexpr int kTc2StagesB = TB200_TC2_STAGES_B;     // ring of expanded B halves: 16 KB per stage
constexpr int kTc2Threads = (kTcFirstEpilogueWarp + 4) * 32;     // 448
constexpr int kTc2TileN = 256;                                   // pair tile: 256 rows x 256 columns
constexpr int kTc2HalfN = 128;                                   // columns expanded per CTA

struct Tc2Geom {
    static constexpr int kABytes = kTcBM * kTcBK;                // 16384: this CTA's 128 rows
    static constexpr int kWpRowBytes = kTc2HalfN / 4;            // 32
    static constexpr int kWpBytes = kTcBK * kWpRowBytes;         // 4096
    static constexpr int kBBytes = kTc2HalfN * kTcBK;            // 16384: this CTA's 128 columns
    static constexpr int kQuads = kTcBK * (kTc2HalfN / 64);      // 256 packed quads per k-block: one per expander
    static constexpr uint32_t kTmemCols = 2 * kTc2TileN;         // two accumulator buffers of 256 columns
    static constexpr int kEpiBytes = 32 * 64 * 4;                // staging tile of one epilogue warp
    static constexpr size_t kSmemBytes = 1024 + size_t(kTc2StagesA) * (kABytes + kWpBytes) +
                                         size_t(kTc2StagesB) * kBBytes + 4 * kEpiBytes + 512;
    // D = s32, A = B = s8, A K-major, B MN-major, N = 256, M = 256 (pair)
    static constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) |
                                       (uint32_t(kTc2TileN >> 3) << 17) | (uint32_t(256 >> 4) << 24);
    // The expander warps are split into groups; group g owns the k-blocks with index % kGroups == g, so the
    // latency of one expansion (load, decode, store, proxy fence, arrive) is spread over kGroups k-blocks.
    static constexpr int kGroups = TB200_TC2_EXPAND_GROUPS;
    static constexpr int kGroupThreads = kTcExpandWarps * 32 / kGroups;
    static constexpr int kGroupWarps = kTcExpandWarps / kGroups;
    static constexpr int kQuadsPerThread = kQuads / kGroupThreads;
    static_assert(kTcExpandWarps % kGroups == 0 && kQuads % kGroupThreads == 0, "expander grouping");
};

// Where the finished columns go: the local C first, then the same place in each peer's C.
constexpr int kTc2MaxDest = 8;
struct Tc2Dest {
    int32_t* c[kTc2MaxDest];
    int count;
};

// Grouped mode: one launch walks the tiles of many products (a "problem group"); descriptors and
// destinations come from tables in global memory, and every pair owns a fixed slice of the tile list.
struct alignas(64) Tc2Problem {
    CUtensorMap tmap_a;        // A: [M rows][K bytes], box 128 x 128, 128-byte swizzle
    CUtensorMap tmap_w;        // packed W: [K rows][N/4 bytes], box 32 B x 128 rows
    Tc2Dest dest;
    long long ldc;
    int M, K, N, c_vec_ok;
};
struct Tc2Tile {
    int problem, m_t, n_t, pad;
};

// The tile sequence of one CTA pair.  Every warp role constructs its own walker and sees the same sequence.
template <bool kGrouped>
struct Tc2Walk {
    const CUtensorMap* ta;
    const CUtensorMap* tw;
    const Tc2Dest* dest;
    long long ldc;
    int M, N, c_vec_ok, m_t, n_t, k_blocks;
    // single product
    int tile, num_tiles, stride, m_tiles;
    // group
    const Tc2Problem* probs;
    const Tc2Tile* tiles;
    int idx, end;

    __device__ __forceinline__ bool next() {
        if constexpr (kGrouped) {
            if (idx >= end) return false;
            const Tc2Tile t = tiles[idx++];
            const Tc2Problem* p = probs + t.problem;
            ta = &p->tmap_a; tw = &p->tmap_w; dest = &p->dest;
            ldc = p->ldc; M = p->M; N = p->N; c_vec_ok = p->c_vec_ok;
            m_t = t.m_t; n_t = t.n_t;
            k_blocks = (p->K + kTcBK - 1) / kTcBK;
            return true;
        } else {
            if (tile >= num_tiles) return false;
            m_t = tile % m_tiles; n_t = tile / m_tiles;
            tile += stride;
            return true;
        }
    }
};

// ---- cta_group::2 forms of the tcgen05 helpers
template <uint32_t kCols>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "n"(kCols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <uint32_t kCols>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(kCols) : "memory");
}
// Arrives, once the pair's MMAs issued so far have finished, on the barrier at this offset in this CTA only ...
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// ... and in both CTAs of the pair (CTA mask 0b11).
__device__ __forceinline__ void tc_commit_pair_both(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
                     "r"(smem_u32(bar)), "h"(mask)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the mbarrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(dsmem_map(smem_u32(bar), rank))
                 : "memory");
}

template <bool kGrouped, bool kBf16 = false>
__global__ void __launch_bounds__(kTc2Threads, 1)
ternary_gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                        const __grid_constant__ Tc2Dest dest, int M, int K, int N, long long ldc, int c_vec_ok,
                        const Tc2Problem* __restrict__ probs, const Tc2Tile* __restrict__ tiles,
                        const int* __restrict__ pair_first, int32_t* __restrict__ status,
                        const float* __restrict__ row_scale = nullptr, float w_scale = 1.0f) {
    static_assert(!(kGrouped && kBf16), "the dequantising epilogue is built for single products");
    using G = Tc2Geom;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = base;                                              // [StagesA][128][128]  swizzled
    uint8_t* sB = sA + kTc2StagesA * G::kABytes;                     // [StagesB][128 k][128]  swizzled
    uint8_t* sWp = sB + kTc2StagesB * G::kBBytes;                    // [StagesA][128 k][32]
    uint8_t* sEpi = sWp + kTc2StagesA * G::kWpBytes;                 // [4 warps][32 rows][64 cols] int32, swizzled
    uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + 4 * G::kEpiBytes);
    uint64_t* full_a = bars;                                         // TMA -> expanders (+ MMA in the leader)
    uint64_t* empty_a = full_a + kTc2StagesA;                        // expanders + MMA -> TMA
    uint64_t* full_b = empty_a + kTc2StagesA;                        // both CTAs' expanders -> leader MMA
    uint64_t* empty_b = full_b + kTc2StagesB;                        // MMA -> expanders
    uint64_t* tmem_full = empty_b + kTc2StagesB;                     // MMA -> epilogue  [2]
    uint64_t* tmem_empty = tmem_full + 2;                            // both CTAs' epilogues -> leader MMA [2]
    uint64_t* drain = tmem_empty + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                         // 0 = leader, 1 = peer
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    auto make_walk = [&]() {
        Tc2Walk<kGrouped> w{};
        if constexpr (kGrouped) {
            w.probs = probs; w.tiles = tiles;
            w.idx = pair_first[pair]; w.end = pair_first[pair + 1];
        } else {
            w.ta = &tmap_a; w.tw = &tmap_w; w.dest = &dest;
            w.ldc = ldc; w.M = M; w.N = N; w.c_vec_ok = c_vec_ok;
            w.k_blocks = (K + kTcBK - 1) / kTcBK;
            w.m_tiles = (M + 2 * kTcBM - 1) / (2 * kTcBM);
            w.num_tiles = w.m_tiles * ((N + kTc2TileN - 1) / kTc2TileN);
            w.tile = pair; w.stride = num_pairs;
        }
        return w;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTc2StagesA; ++s) {
            mbar_init(&full_a[s], 1);
            mbar_init(&empty_a[s], G::kGroupWarps + 1);
        }
        for (int s = 0; s < kTc2StagesB; ++s) {
            mbar_init(&full_b[s], 2 * G::kGroupWarps);
            mbar_init(&empty_b[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 8);
        }
        mbar_init(drain, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc_pair<G::kTmemCols>(tmem_slot);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();              // barriers of both CTAs are initialised before anyone arrives remotely
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ================================================================ TMA producer (each CTA for itself)
        if (lane == 0) {
            if constexpr (!kGrouped) {
                tma_prefetch_desc(&tmap_a);
                tma_prefetch_desc(&tmap_w);
            }
            uint32_t it = 0;
            bool ok = true;
            auto walk = make_walk();
            while (ok && walk.next()) {
                const int row0 = walk.m_t * 2 * kTcBM + rank * kTcBM;
                const int wp_x = walk.n_t * (kTc2TileN / 4) + rank * G::kWpRowBytes;
                for (int kb = 0; kb < walk.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % kTc2StagesA;
                    if (!mbar_wait(&empty_a[s], ((it / kTc2StagesA) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full_a[s], G::kABytes + G::kWpBytes);
                    tma_load_2d(sA + s * G::kABytes, walk.ta, kb * kTcBK, row0, &full_a[s]);
                    tma_load_2d(sWp + s * G::kWpBytes, walk.tw, wp_x, kb * kTcBK, &full_a[s]);
                }
            }
            if (!ok) {
                const uint32_t first = it > kTc2StagesA ? it - kTc2StagesA : 0;
                for (uint32_t j = first; j < it; ++j) mbar_drain(&full_a[j % kTc2StagesA], (j / kTc2StagesA) & 1);
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer (leader CTA only)
        if (leader && lane == 0) {
            uint32_t it = 0, lt = 0;
            bool ok = true;
            auto walk = make_walk();
            for (; ok && walk.next(); ++lt) {
                const uint32_t acc = lt & 1;
                if (!mbar_wait(&tmem_empty[acc], ((lt >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kTc2TileN;
                for (int kb = 0; kb < walk.k_blocks; ++kb, ++it) {
                    const uint32_t sa = it % kTc2StagesA, sb = it % kTc2StagesB;
                    if (!mbar_wait(&full_a[sa], (it / kTc2StagesA) & 1, abort_flag) ||
                        !mbar_wait(&full_b[sb], (it / kTc2StagesB) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(sA + sa * G::kABytes);
                    const uint32_t b_addr = smem_u32(sB + sb * G::kBBytes);
#pragma unroll
                    for (int k4 = 0; k4 < kTcBK / 32; ++k4) {
                        const uint64_t da = umma_desc_sw128(a_addr + k4 * 32, 16, 1024);
                        const uint64_t db = umma_desc_sw128(b_addr + k4 * 4096, G::kBBytes, 1024);
                        tc_mma_i8_pair(d_tmem, da, db, G::kIdesc, (kb | k4) != 0 ? 1u : 0u);
                    }
                    tc_commit_pair_both(&empty_a[sa]);
                    tc_commit_pair_both(&empty_b[sb]);
                }
                if (ok) tc_commit_pair_both(&tmem_full[acc]);
            }
            tc_commit_pair(drain);
            mbar_wait(drain, 0, abort_flag);
        }
    } else if (warp < kTcFirstEpilogueWarp) {
        // ================================================================ expanders: this CTA's 128 columns
        const int e = threadIdx.x - kTcFirstExpandWarp * 32;          // 0..255
        const uint32_t group = e / G::kGroupThreads;                   // which k-blocks this warp expands
        const int eg = e % G::kGroupThreads;
        uint32_t src_off[G::kQuadsPerThread], dst_off[G::kQuadsPerThread][4];
#pragma unroll
        for (int i = 0; i < G::kQuadsPerThread; ++i) {
            const int idx = eg + i * G::kGroupThreads;                 // packed quad of the k-block
            const int q = idx & 1, k = idx >> 1;                       // 64-column quad, k-row
            src_off[i] = idx * 16;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = q * 4 + u;                               // 16-column chunk inside the 128-column half
                dst_off[i][u] = k * 128 + ((c ^ (k & 7)) << 4);
            }
        }
        const uint32_t wp_sa = smem_u32(sWp), b_sa = smem_u32(sB);
        uint32_t it = 0;
        bool ok = true;
        auto walk = make_walk();
        while (ok && walk.next()) {
            for (int kb = 0; kb < walk.k_blocks; ++kb, ++it) {
                const uint32_t sa = it % kTc2StagesA, sb = it % kTc2StagesB;
                // Every expander warp observes every phase of full_a, also for k-blocks of other groups: a
                // parity wait is only meaningful for a waiter that is at most one phase behind the barrier.
                if (!mbar_wait(&full_a[sa], (it / kTc2StagesA) & 1, abort_flag)) { ok = false; break; }
                if (it % G::kGroups != group) continue;
                if (!mbar_wait(&empty_b[sb], ((it / kTc2StagesB) & 1) ^ 1, abort_flag)) { ok = false; break; }
                const uint32_t wp = wp_sa + sa * G::kWpBytes;
                const uint32_t bt = b_sa + sb * G::kBBytes;
                uint4 v[G::kQuadsPerThread];
#pragma unroll
                for (int i = 0; i < G::kQuadsPerThread; ++i) v[i] = lds_v4(wp + src_off[i]);
#pragma unroll
                for (int i = 0; i < G::kQuadsPerThread; ++i) {
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
                fence_proxy_async_smem();          // generic-proxy stores -> visible to the pair's tensor cores
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(&full_b[sb]);
                    else mbar_arrive_remote(&full_b[sb], 0);
                    mbar_arrive(&empty_a[sa]);
                }
            }
        }
    } else {
        // ================================================================ epilogue: this CTA's 128 rows x 256 columns
        const int quad = warp & 3;
        const uint32_t stage_sa = smem_u32(sEpi) + (warp - kTcFirstEpilogueWarp) * G::kEpiBytes;
        const uint32_t my_row_sa = stage_sa + lane * 256;              // this lane's accumulator row in the staging tile
        uint32_t lt = 0;
        bool ok = true;
        auto walk = make_walk();
        for (; ok && walk.next(); ++lt) {
            const int m_t = walk.m_t, n_t = walk.n_t;
            const int M = walk.M, N = walk.N, c_vec_ok = walk.c_vec_ok;
            const long long ldc = walk.ldc;
            const Tc2Dest* dst = walk.dest;
            const int n_dest = dst->count;
            const uint32_t acc = lt & 1;
            if (!mbar_wait(&tmem_full[acc], (lt >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            const int row_base = m_t * 2 * kTcBM + rank * kTcBM + quad * 32;
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kTc2TileN;
            float rs = 0.0f;                                           // scale of this lane's accumulator row
            if constexpr (kBf16) rs = (row_base + lane < M) ? row_scale[row_base + lane] : 0.0f;
#pragma unroll 1
            for (int c0 = 0; c0 < kTc2TileN; c0 += 64) {
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
                    if constexpr (kBf16) {
                        // 32 columns -> 32 bfloat16 = four 16-byte chunks of this lane's 128-byte staging row
                        uint32_t pk[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float lo = (static_cast<float>(o[2 * i]) * rs) * w_scale;
                            const float hi = (static_cast<float>(o[2 * i + 1]) * rs) * w_scale;
                            const __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                            pk[i] = *reinterpret_cast<const uint32_t*>(&b2);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int chunk = h * 4 + j;
                            sts_v4(stage_sa + lane * 128 + ((chunk ^ (lane & 7)) << 4),
                                   make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int chunk = h * 8 + j;               // 16-byte chunk of the 64-column row
                            sts_v4(my_row_sa + ((chunk ^ (lane & 7)) << 4),
                                   make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]));
                        }
                    }
                }
                __syncwarp();
                if constexpr (kBf16) {
                    // read back row-contiguous: 8 lanes cover the 128 bytes (64 bfloat16) of one row, a warp four rows
                    const int col = n_t * kTc2TileN + c0 + (lane & 7) * 8;
#pragma unroll 4
                    for (int i = 0; i < 8; ++i) {
                        const int rr = 4 * i + (lane >> 3);
                        const uint4 v = lds_v4(stage_sa + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
                        const int row = row_base + rr;
                        if (row < M && col < N) {
                            const size_t off = static_cast<size_t>(row) * ldc + col;
#pragma unroll
                            for (int d = 0; d < kTc2MaxDest; ++d) {
                                if (d >= n_dest) break;
                                uint16_t* out = reinterpret_cast<uint16_t*>(dst->c[d]) + off;
                                if (c_vec_ok) {
                                    *reinterpret_cast<uint4*>(out) = v;
                                } else {
                                    const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                                    for (int e2 = 0; e2 < 4; ++e2) {
                                        out[2 * e2] = static_cast<uint16_t>(wds[e2] & 0xFFFFu);
                                        out[2 * e2 + 1] = static_cast<uint16_t>(wds[e2] >> 16);
                                    }
                                }
                            }
                        }
                    }
                } else {
                // read back row-contiguous: 16 lanes cover the 256 bytes of one row, a warp covers two rows
                const int col = n_t * kTc2TileN + c0 + (lane & 15) * 4;
#pragma unroll 4
                for (int i = 0; i < 16; ++i) {
                    const int rr = 2 * i + (lane >> 4);
                    const uint4 v = lds_v4(stage_sa + rr * 256 + (((lane & 15) ^ (rr & 7)) << 4));
                    const int row = row_base + rr;
                    if (row < M && col < N) {
                        const size_t off = static_cast<size_t>(row) * ldc + col;
#pragma unroll
                        for (int d = 0; d < kTc2MaxDest; ++d) {
                            if (d >= n_dest) break;
                            int32_t* out = dst->c[d] + off;
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
                }
                __syncwarp();                                          // before the staging tile is rewritten
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(&tmem_empty[acc]);
                else mbar_arrive_remote(&tmem_empty[acc], 0);
            }
        }
    }

    __syncwarp();                    // the role branches above diverge inside warps; reconverge before aligned barriers
    if (*abort_flag && lane == 0 && status) atomicMax(status, kStatusTimeout);
    tc_fence_before_sync();
    cluster_sync_all();              // no CTA frees TMEM or exits while its partner may still signal or read it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair<G::kTmemCols>(tmem_base);
    }
}

}  // namespace tb200
