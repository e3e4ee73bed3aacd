// Decode regime, many projections per launch: a persistent GEMV kernel over a list of problems.
//
// One launch walks a host-built work list.  A work item is (problem, column chunk, row group): the
// full K of one chunk of 16*WORDS columns (WORDS = 32: 512 columns, 128-byte rows; WORDS = 16: 256
// columns), so there is no split-K and nothing to reduce across CTAs.  Every CTA owns a fixed,
// load-balanced slice of the list and streams the packed weights of item after item through the
// same TMA ring (8 stages of 8 KB) without draining it between items: per SM tens of KB are always in flight, which is what a 4 MB GEMV launched on
// its own cannot do.  The per-problem TMA descriptors live in a table in global memory.
//
// The decode is the leanest exact form found; with it the kernel runs at the memory system's pace while every SM
// holds its four CTAs, and what is lost is lost to the coarse items (see "Balance" below).
//   * The packed bytes of four k-rows of one byte column are brought together by the load itself:
//     ldmatrix.m16n16.x2.trans.b8 reads a block of 16 k-rows x 32 packed bytes and hands lane l four registers, each
//     holding the bytes of k-rows 4(l%4)..4(l%4)+3 of one byte column (columns l/4, l/4+8, 16+l/4, 24+l/4 of the
//     block).  The stage is loaded with the TMA swizzle that matches its row length (128 or 64 bytes) so that the
//     16-byte rows of a block fall in different banks.  A warp keeps one 128-column block of the item and walks two
//     16-row blocks of every stage; four lanes and two or four warps share each column and meet in the
//     shared-memory reduction.
//   * T ^= 0xAAAAAAAA turns every 2-bit code c in {0,1,3} into c^2 in {2,3,1} = w + 2, so a field
//     can be used IN PLACE, unsigned, with one AND and no shift or sign extension:
//     dp4a.u32.s32(T & (0x03030303 << 2j), a) adds 4^j * sum_k a_k (w_k + 2);
//   * the epilogue takes (acc >> 2j) - 2 * sum_k a_k.  The row sum of the activations is the same
//     for every column and is computed once per item by one warp (dp4a against 0x01010101 and a
//     warp-shuffle reduction).  Bound: 4^3 * 3 * 128 * K < 2^31, K <= 8192 here.
//   34 instructions per 64 weights at M = 1 (1 ldmatrix, 1 activation load, 16 LOP3, 16 dp4a).
//
// Balance.  Items are whole: a 512-column chunk over all of K.  64 projections of 2560 x 6912 are 6.05 items per SM,
// so the last third of the launch runs with two CTAs per SM instead of four.  Cutting items along K to even this out
// was tried and is slower: neighbouring CTAs then stop reading the same weight rows at the same time, and the
// 128-byte row segments of a lone CTA no longer share DRAM pages with anybody's (4.3 TB/s instead of 6.8 TB/s in the
// fully occupied phase).
//
// Prepacked weights (PRE = true, optional).  ternix_b200_prepack_k4 stores, for every group of four k-rows and
// every packed byte column, the four bytes of that column together in one 32-bit word (same size as the packed
// matrix, K rounded up to a multiple of 4), so that a lane loads its four transposed words with one 16-byte
// shared-memory load.  It predates the transposing loads above and is no faster than them; it stays for callers
// that already hold weights in that layout.
//
// Activations of the next item are prefetched with a 1-D bulk copy into the second of two
// buffers while the current item is consumed; the per-item epilogue is one named barrier.
#pragma once
#include <cuda.h>
#include <cstdint>
#include "kernel_gemv.cuh"
#include "ptx_sm100.cuh"

namespace tb200 {

constexpr int kGroupMaxK = 8192;                // activation bytes staged per row
constexpr int kGroupStageBytes = 8192;          // one TMA box
// Ring depth and resident CTAs per SM by row-group size.  The kernel is bound by instruction issue, so
// more resident warps beat a deeper ring: M = 1 runs 4 CTAs per SM with 4 stages each (measured +5 % over
// 2 CTAs x 8 stages), M = 2 runs 3, and 4-row groups (144 registers per thread) run 1 CTA with 8 stages.
constexpr int group_stages(int mr) { return mr <= 2 ? 4 : 8; }
constexpr int group_ctas_per_sm(int mr) { return mr <= 1 ? 4 : mr == 2 ? 3 : 1; }
constexpr int group_stage_rows(int words) { return kGroupStageBytes / (words * 4); }   // 128 or 64 k-rows

struct alignas(64) GroupProblem {
    CUtensorMap tmap_w;        // packed W: [K rows][N/4 bytes], box (4*WORDS) B x group_stage_rows(WORDS)
    const int8_t* A;
    int32_t* C;
    long long ldc;
    int M, K, N, pad;
};
struct GroupItem {
    int problem, chunk, row0, pad;
};

template <int MR, int WORDS>
constexpr size_t gemv_group_smem_bytes() {
    constexpr int kGroupStages = group_stages(MR);
    return 1024 + size_t(kGroupStages) * kGroupStageBytes + 2 * size_t(MR) * kGroupMaxK +
           2 * size_t(MR) * 16 * (WORDS + 1) * 4 + (2 * kGroupStages + 4) * 8 + 2 * MR * 4 + 16;
}

__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// 16 rows x 32 bytes, transposed: lanes 0-15 give the row addresses of bytes 0-15, lanes 16-31 those of bytes 16-31.
__device__ __forceinline__ void ldmatrix_x2_trans_b8(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr)
                 : "memory");
}

__device__ __forceinline__ int dp4a_u8s8(uint32_t a_unsigned, int b_signed, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
    return d;
}

// dst word [r][b] = { src[4r][b], src[4r+1][b], src[4r+2][b], src[4r+3][b] } (zero beyond K): the 4x4 byte
// transpose of the GEMV decode, done once.  src is the packed K x (N/4) matrix.
__global__ void prepack_k4_kernel(const uint8_t* __restrict__ src, uint32_t* __restrict__ dst, int K, int pitch) {
    const int k4 = (K + 3) / 4;
    const long long total = static_cast<long long>(k4) * pitch;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / pitch), b = static_cast<int>(i % pitch);
        uint32_t w = 0;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const int k = 4 * r + kk;
            if (k < K) w |= static_cast<uint32_t>(src[static_cast<size_t>(k) * pitch + b]) << (8 * kk);
        }
        dst[i] = w;
    }
}

template <int MR, int WORDS, bool PRE = false>
__global__ void __launch_bounds__(kGemvThreads)
ternary_gemv_group_kernel(const GroupProblem* __restrict__ probs, const GroupItem* __restrict__ items,
                          const int* __restrict__ cta_first, int32_t* __restrict__ status) {
    static_assert(!PRE || WORDS == 32, "prepacked weights use 512-column items");
    constexpr int kGroupStageRows = kGroupStageBytes / (WORDS * 4);
    constexpr int kGroupStages = MR <= 2 ? 4 : 8;               // = group_stages(MR)
    constexpr int kPartInts = MR * 16 * (WORDS + 1);
    constexpr bool LDM = !PRE;                          // transposing loads from a swizzled stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = base;
    int8_t* a_buf = reinterpret_cast<int8_t*>(base + kGroupStages * kGroupStageBytes);   // [2][MR][kGroupMaxK]
    int32_t* part = reinterpret_cast<int32_t*>(a_buf + 2 * MR * kGroupMaxK);             // [2][MR][16][WORDS+1]
    uint64_t* full = reinterpret_cast<uint64_t*>(part + 2 * kPartInts);
    uint64_t* empty = full + kGroupStages;
    uint64_t* a_full = empty + kGroupStages;     // [2]
    uint64_t* a_empty = a_full + 2;              // [2]
    int32_t* row_sum = reinterpret_cast<int32_t*>(a_empty + 2);                          // [2][MR]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(row_sum + 2 * MR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int item_lo = cta_first[blockIdx.x], item_hi = cta_first[blockIdx.x + 1];
    // a dependent launch (the next decode batch on the stream) may start filling SMs as this grid's CTAs retire
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (tid == 0) {
        for (int s = 0; s < kGroupStages; ++s) {
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
            auto load_tile = [&](const GroupProblem* p, const GroupItem& it, int tt) {
                const uint32_t s = t % kGroupStages;
                if (!mbar_wait(&empty[s], ((t / kGroupStages) & 1) ^ 1, abort_flag)) return false;
                mbar_arrive_expect_tx(&full[s], kGroupStageBytes);
                if constexpr (PRE)   // [K/4 rows][N/4 words]: 128 words x 16 rows = the same 64 k-rows x 512 columns
                    tma_load_2d(stages + s * kGroupStageBytes, &p->tmap_w, it.chunk * WORDS * 4, tt * (kGroupStageRows / 4),
                                &full[s]);
                else
                    tma_load_2d(stages + s * kGroupStageBytes, &p->tmap_w, it.chunk * WORDS * 4, tt * kGroupStageRows, &full[s]);
                ++t;
                return true;
            };
            for (int i = item_lo; ok && i < item_hi; ++i) {
                const GroupItem it = items[i];
                const GroupProblem* p = probs + it.problem;
                const int K = p->K;
                const uint32_t n = i - item_lo, buf = n & 1;
                int rows = p->M - it.row0;
                if (rows > MR) rows = MR;
                const int ntiles = (K + kGroupStageRows - 1) / kGroupStageRows;
                int tt = 0;
                if (i == item_lo) {
                    // Launched as a programmatic dependent of the kernel before it, this CTA may already be running
                    // while that kernel's last CTAs finish.  Weights are never written by a kernel of this library, so
                    // the first ring of weight tiles is requested right away; everything a predecessor may have
                    // produced (the activations) and every store waits for its completion.
                    for (; ok && tt < ntiles && tt < kGroupStages; ++tt) ok = load_tile(p, it, tt);
                    asm volatile("griddepcontrol.wait;" ::: "memory");
                    if (!ok) break;
                }
                if (!mbar_wait(&a_empty[buf], ((n >> 1) & 1) ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&a_full[buf], static_cast<uint32_t>(rows) * K);
                for (int r = 0; r < rows; ++r)
                    bulk_copy_g2s(a_buf + (buf * MR + r) * kGroupMaxK, p->A + static_cast<size_t>(it.row0 + r) * K, K,
                                  &a_full[buf]);
                for (; ok && tt < ntiles; ++tt) ok = load_tile(p, it, tt);
            }
            if (*abort_flag) {
                const uint32_t first = t > kGroupStages ? t - kGroupStages : 0;
                for (uint32_t j = first; j < t; ++j) mbar_drain(&full[j % kGroupStages], (j / kGroupStages) & 1);
                mbar_drain(&a_full[0], 0);
                mbar_drain(&a_full[1], 0);
            }
        }
    } else {
        // ------------------------------------------------------------ consumers
        const int kg = warp;                                   // prepacked: 4-row groups kg and kg + 8 of each stage
        // transposing loads: 128-column block `cb`, 16-row blocks `kb0` and `kb0 + (blocks per stage) / 2`; this lane's
        // row address inside the swizzled stage and its four k-rows inside a block.  128-byte rows: 4 column blocks x
        // 4 row blocks per stage, 16-byte chunk index ^= row % 8; 64-byte rows: 2 x 8, chunk index ^= (row / 2) % 4.
        constexpr int kColBlocks = WORDS / 8;
        const int cb = warp & (kColBlocks - 1), kb0 = warp / kColBlocks;
        const int ldm_row = kb0 * 16 + (lane & 15);
        const uint32_t ldm_swz = WORDS == 32 ? (ldm_row & 7) : ((ldm_row >> 1) & 3);
        const uint32_t ldm_off = ldm_row * (WORDS * 4) + (((cb * 2 + (lane >> 4)) ^ ldm_swz) << 4);
        const int ldm_k = kb0 * 16 + 4 * (lane & 3);
        const uint32_t stages_sa = smem_u32(stages), a_sa = smem_u32(a_buf), part_sa = smem_u32(part);
        uint32_t t = 0;
        bool ok = true;
        for (int i = item_lo; ok && i < item_hi; ++i) {
            const GroupItem it = items[i];
            const GroupProblem* p = probs + it.problem;
            const int K = p->K, M = p->M, N = p->N;
            const uint32_t n = i - item_lo, buf = n & 1;
            const int ntiles = (K + kGroupStageRows - 1) / kGroupStageRows;
            if (!mbar_wait(&a_full[buf], (n >> 1) & 1, abort_flag)) break;
            const int8_t* a_s = a_buf + buf * MR * kGroupMaxK;   // (row sums only; the main loop uses a_sa)

            if (warp == 0) {
                // row sums of the activations: dp4a against ones, then a warp-shuffle reduction
#pragma unroll
                for (int r = 0; r < MR; ++r) {
                    int sum = 0;
                    for (int k4 = lane; k4 < (K >> 2); k4 += 32)
                        sum = __dp4a(0x01010101, *reinterpret_cast<const int*>(a_s + r * kGroupMaxK + 4 * k4), sum);
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                    if (lane == 0) row_sum[buf * MR + r] = sum;
                }
            }

            int32_t acc[MR][16];
#pragma unroll
            for (int r = 0; r < MR; ++r)
#pragma unroll
                for (int c = 0; c < 16; ++c) acc[r][c] = 0;

            for (int tt = 0; tt < ntiles; ++tt, ++t) {
                const uint32_t s = t % kGroupStages;
                if (!mbar_wait(&full[s], (t / kGroupStages) & 1, abort_flag)) { ok = false; break; }
                const uint32_t st = stages_sa + s * kGroupStageBytes;
                uint32_t w[2][4];
                int a4[2][MR];
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    if constexpr (PRE) {
                        // row (4-k group) kg + 8g of the stage, this lane's four transposed words
                        const uint4 v = lds_v4(st + (kg + 8 * g) * (WORDS * 16) + lane * 16);
                        w[g][0] = v.x; w[g][1] = v.y; w[g][2] = v.z; w[g][3] = v.w;
                    } else {
                        ldmatrix_x2_trans_b8(w[g], st + ldm_off + g * 4096);       // second half of the stage: 4 KB on
                    }
                    const int k = LDM ? tt * kGroupStageRows + ldm_k + (kGroupStageRows / 2) * g
                                      : tt * kGroupStageRows + (kg + 8 * g) * 4;
#pragma unroll
                    for (int r = 0; r < MR; ++r) {
                        const uint32_t raw = lds_u32(a_sa + (buf * MR + r) * kGroupMaxK + k);
                        a4[g][r] = k < K ? static_cast<int>(raw) : 0;      // nothing beyond K
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);

#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const uint32_t (&T)[4] = w[g];     // four transposed words: the bytes of 4 k-rows of one byte column each
#pragma unroll
                    for (int b = 0; b < 4; ++b)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t x = (T[b] ^ 0xAAAAAAAAu) & (0x03030303u << (2 * j));   // (w + 2) * 4^j, in place
#pragma unroll
                            for (int r = 0; r < MR; ++r) acc[r][4 * b + j] = dp4a_u8s8(x, a4[g][r], acc[r][4 * b + j]);
                        }
                }
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_empty[buf]);           // the activation buffer may be refilled

            const uint32_t pt = part_sa + buf * kPartInts * 4;
#pragma unroll
            for (int r = 0; r < MR; ++r)
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    if constexpr (LDM) {
                        // register b = c / 4 holds byte column (b & 1) * 8 + (b >> 1) * 16 + lane / 4 of the block
                        const int col = cb * 128 + (((c >> 2) & 1) * 8 + (c >> 3) * 16 + (lane >> 2)) * 4 + (c & 3);
                        red_shared_add(pt + ((r * 16 + (col & 15)) * (WORDS + 1) + (col >> 4)) * 4, acc[r][c]);
                    } else {
                        red_shared_add(pt + ((r * 16 + c) * (WORDS + 1) + lane) * 4, acc[r][c]);
                    }
                }
            asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerWarps * 32) : "memory");
            // store this item's columns and leave the buffer zeroed for the item after next
            for (int idx = tid; idx < MR * WORDS * 16; idx += kGemvConsumerWarps * 32) {
                const int r = idx / (WORDS * 16), col = idx % (WORDS * 16);
                const uint32_t slot = pt + ((r * 16 + (col & 15)) * (WORDS + 1) + (col >> 4)) * 4;
                const int32_t v = static_cast<int32_t>(lds_u32(slot));
                sts_u32(slot, 0u);
                const int grow = it.row0 + r, gcol = it.chunk * WORDS * 16 + col;
                if (grow < M && gcol < N)
                    p->C[static_cast<size_t>(grow) * p->ldc + gcol] = (v >> (2 * (col & 3))) - 2 * row_sum[buf * MR + r];
            }
        }
    }
    __syncthreads();
    if (tid == 0 && *abort_flag && status) atomicMax(status, kStatusTimeout);
}

}  // namespace tb200
