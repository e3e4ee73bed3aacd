// Decode regime, many projections per launch: a persistent GEMV kernel over a list of problems.
//
// One launch walks a host-built work list.  A work item is (problem, 256-column chunk, row group):
// the full K of one chunk, so there is no split-K and nothing to reduce across CTAs.  Every CTA
// owns a fixed, load-balanced slice of the list and streams the packed weights of item after
// item through the same 16-stage TMA ring without draining it between items: per SM tens of KB
// are always in flight, which is what a 4 MB GEMV launched on its own cannot do.  The per-problem
// TMA descriptors live in a table in global memory.
//
// The decode is the one of ternary_gemv_kernel (4x4 byte transpose, (T << s) & 0xC0C0C0C0, dp4a);
// activations of the next item are prefetched with a 1-D bulk copy into the second of two
// buffers while the current item is consumed; the per-item epilogue is one named barrier.
#pragma once
#include <cuda.h>
#include <cstdint>
#include "kernel_gemv.cuh"
#include "ptx_sm100.cuh"

namespace tb200 {

constexpr int kGroupWords = 16;                 // 256 output columns per item
constexpr int kGroupMaxK = 8192;                // activation bytes staged per row
constexpr int kGroupStageRows = GemvGeom<kGroupWords>::kStageRows;   // 64

struct alignas(64) GroupProblem {
    CUtensorMap tmap_w;        // packed W: [K rows][N/4 bytes], box 64 B x 64 rows
    const int8_t* A;
    int32_t* C;
    long long ldc;
    int M, K, N, pad;
};
struct GroupItem {
    int problem, chunk, row0, pad;
};

template <int MR>
constexpr size_t gemv_group_smem_bytes() {
    return 128 + size_t(kGemvStages) * kGemvStageBytes + 2 * size_t(MR) * kGroupMaxK +
           2 * size_t(MR) * 16 * (kGroupWords + 1) * 4 + (2 * kGemvStages + 4) * 8 + 16;
}

__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

template <int MR>
__global__ void __launch_bounds__(kGemvThreads)
ternary_gemv_group_kernel(const GroupProblem* __restrict__ probs, const GroupItem* __restrict__ items,
                          const int* __restrict__ cta_first, int32_t* __restrict__ status) {
    constexpr int WORDS = kGroupWords;
    constexpr int kPartInts = MR * 16 * (WORDS + 1);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t* stages = base;
    int8_t* a_buf = reinterpret_cast<int8_t*>(base + kGemvStages * kGemvStageBytes);     // [2][MR][kGroupMaxK]
    int32_t* part = reinterpret_cast<int32_t*>(a_buf + 2 * MR * kGroupMaxK);             // [2][MR][16][WORDS+1]
    uint64_t* full = reinterpret_cast<uint64_t*>(part + 2 * kPartInts);
    uint64_t* empty = full + kGemvStages;
    uint64_t* a_full = empty + kGemvStages;      // [2]
    uint64_t* a_empty = a_full + 2;              // [2]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(a_empty + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int item_lo = cta_first[blockIdx.x], item_hi = cta_first[blockIdx.x + 1];

    if (tid == 0) {
        for (int s = 0; s < kGemvStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kGemvConsumerWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&a_full[b], 1);
            mbar_init(&a_empty[b], kGemvConsumerWarps);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    for (int i = tid; i < 2 * kPartInts; i += kGemvThreads) part[i] = 0;
    __syncthreads();

    if (warp == kGemvConsumerWarps) {
        // ------------------------------------------------------------ producer lane
        if (lane == 0) {
            uint32_t t = 0;
            bool ok = true;
            for (int i = item_lo; ok && i < item_hi; ++i) {
                const GroupItem it = items[i];
                const GroupProblem* p = probs + it.problem;
                const int K = p->K;
                const uint32_t n = i - item_lo, buf = n & 1;
                int rows = p->M - it.row0;
                if (rows > MR) rows = MR;
                if (!mbar_wait(&a_empty[buf], ((n >> 1) & 1) ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&a_full[buf], static_cast<uint32_t>(rows) * K);
                for (int r = 0; r < rows; ++r)
                    bulk_copy_g2s(a_buf + (buf * MR + r) * kGroupMaxK, p->A + static_cast<size_t>(it.row0 + r) * K, K,
                                  &a_full[buf]);
                const int ntiles = (K + kGroupStageRows - 1) / kGroupStageRows;
                for (int tt = 0; tt < ntiles; ++tt, ++t) {
                    const uint32_t s = t % kGemvStages;
                    if (!mbar_wait(&empty[s], ((t / kGemvStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full[s], kGemvStageBytes);
                    tma_load_2d(stages + s * kGemvStageBytes, &p->tmap_w, it.chunk * WORDS * 4, tt * kGroupStageRows,
                                &full[s]);
                }
            }
            if (*abort_flag) {
                const uint32_t first = t > kGemvStages ? t - kGemvStages : 0;
                for (uint32_t j = first; j < t; ++j) mbar_drain(&full[j % kGemvStages], (j / kGemvStages) & 1);
                mbar_drain(&a_full[0], 0);
                mbar_drain(&a_full[1], 0);
            }
        }
    } else {
        // ------------------------------------------------------------ consumers
        const int word = lane % WORDS;
        const int kg = warp * (32 / WORDS) + lane / WORDS;     // 4-row group inside a stage
        uint32_t t = 0;
        bool ok = true;
        for (int i = item_lo; ok && i < item_hi; ++i) {
            const GroupItem it = items[i];
            const GroupProblem* p = probs + it.problem;
            const int K = p->K, M = p->M, N = p->N;
            const uint32_t n = i - item_lo, buf = n & 1;
            const int ntiles = (K + kGroupStageRows - 1) / kGroupStageRows;
            if (!mbar_wait(&a_full[buf], (n >> 1) & 1, abort_flag)) break;
            const int8_t* a_s = a_buf + buf * MR * kGroupMaxK;

            int32_t acc[MR][16];
#pragma unroll
            for (int r = 0; r < MR; ++r)
#pragma unroll
                for (int c = 0; c < 16; ++c) acc[r][c] = 0;

            for (int tt = 0; tt < ntiles; ++tt, ++t) {
                const uint32_t s = t % kGemvStages;
                if (!mbar_wait(&full[s], (t / kGemvStages) & 1, abort_flag)) { ok = false; break; }
                const uint32_t* st = reinterpret_cast<const uint32_t*>(stages + s * kGemvStageBytes);
                const uint32_t w0 = st[(kg * 4 + 0) * WORDS + word];
                const uint32_t w1 = st[(kg * 4 + 1) * WORDS + word];
                const uint32_t w2 = st[(kg * 4 + 2) * WORDS + word];
                const uint32_t w3 = st[(kg * 4 + 3) * WORDS + word];
                int a4[MR];
#pragma unroll
                for (int r = 0; r < MR; ++r)
                    a4[r] = *reinterpret_cast<const int*>(a_s + r * kGroupMaxK + tt * kGroupStageRows + kg * 4);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);

                const uint32_t lo01 = __byte_perm(w0, w1, 0x5140), hi01 = __byte_perm(w0, w1, 0x7362);
                const uint32_t lo23 = __byte_perm(w2, w3, 0x5140), hi23 = __byte_perm(w2, w3, 0x7362);
                uint32_t T[4];
                T[0] = __byte_perm(lo01, lo23, 0x5410);
                T[1] = __byte_perm(lo01, lo23, 0x7632);
                T[2] = __byte_perm(hi01, hi23, 0x5410);
                T[3] = __byte_perm(hi01, hi23, 0x7632);
#pragma unroll
                for (int b = 0; b < 4; ++b)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int x = static_cast<int>((T[b] << (6 - 2 * j)) & 0xC0C0C0C0u);
#pragma unroll
                        for (int r = 0; r < MR; ++r) acc[r][4 * b + j] = __dp4a(x, a4[r], acc[r][4 * b + j]);
                    }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_empty[buf]);           // the activation buffer may be refilled

            int32_t* pt = part + buf * kPartInts;
#pragma unroll
            for (int r = 0; r < MR; ++r)
#pragma unroll
                for (int c = 0; c < 16; ++c) atomicAdd(&pt[(r * 16 + c) * (WORDS + 1) + word], acc[r][c]);
            asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerWarps * 32) : "memory");
            // store this item's columns and leave the buffer zeroed for the item after next
            for (int idx = tid; idx < MR * WORDS * 16; idx += kGemvConsumerWarps * 32) {
                const int r = idx / (WORDS * 16), col = idx % (WORDS * 16);
                int32_t* slot = &pt[(r * 16 + (col & 15)) * (WORDS + 1) + (col >> 4)];
                const int32_t v = *slot;
                *slot = 0;
                const int grow = it.row0 + r, gcol = it.chunk * WORDS * 16 + col;
                if (grow < M && gcol < N) p->C[static_cast<size_t>(grow) * p->ldc + gcol] = v >> 6;
            }
        }
    }
    __syncthreads();
    if (tid == 0 && *abort_flag && status) atomicMax(status, kStatusTimeout);
}

}  // namespace tb200
