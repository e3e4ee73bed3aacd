// Batched decode, a few to a few dozen rows of activations: the packed weights stream through shared memory once
// and are multiplied straight out of registers by the warp-level tensor instruction
//     mma.sync.m16n8k32 (A uint8 = decoded weights, B int8 = activations, int32 accumulators).
//
// Why this instruction and not tcgen05.  The regime is bound by HBM (a few rows of activations against megabytes of
// weights), so what has to be cheap is the path from a packed byte to a multiplier operand.  tcgen05.mma takes its
// operands from shared memory in a canonical layout, which means writing four expanded bytes per packed byte back
// to shared memory first; that expansion is what bounds the prefill kernels and is far too slow here.  mma.sync
// takes its operands from registers, and the decode below produces exactly its register layout with no data
// movement at all.  The weights are the instruction's A operand (16 rows = 16 packed byte columns), the
// activations its B operand (8 columns = 8 rows of the batch), so the result tile is C transposed:
//   * ldmatrix.m16n16.x2.trans.b8 on a block of 16 k-rows x 32 packed bytes gives lane l four registers, each the
//     bytes of k-rows 4(l%4)..4(l%4)+3 of byte column l/4 (+0, +8, +16, +24);
//   * the A fragment of m16n8k32 wants, in lane l, A[row l/4][k = 4(l%4)..+3], the same for row l/4 + 8, and both
//     again for k + 16: the registers of byte columns l/4 and l/4 + 8 of two consecutive 16-row blocks;
//   * (T ^ 0xAAAAAAAA) & (0x03030303 << 2j) leaves (w + 2) * 4^j of weight column 4 * (byte column) + j in every
//     byte, a valid unsigned operand: one LOP3 per register and field, as in the one-row kernel.
// One MMA then does 16 byte columns (one field of each) x 32 k x 8 batch rows: per 1 KB of packed weights and warp
// 32 LOP3 and 8 MMA per 8 batch rows, where the dp4a form costs 16 * M per 64 weights per lane.  The legacy tensor
// path is slow on this part (about one m16n8k32 per 31 cycles and SM sub-partition), which bounds the kernel at
// about 4.4 TB/s of packed weights for up to 8 rows and 2.2 TB/s for up to 16; it is the faster form from 3 rows up.
// The accumulators hold 4^j * sum_k a (w + 2); the epilogue takes (acc >> 2j) - 2 * sum_k a.  The row sums come
// from one more MMA per k-step with an A fragment of ones, which lands them in the lanes that need them.
// Bound: 192 * 128 * K < 2^31, K <= 65536 here.
//
// Structure: persistent CTAs of 4 consumer warps + 1 producer warp over a host-built item list, like the one-row
// kernel.  An item is (problem, 512-column chunk, row group of 8 * NG rows, k-range).  A stage is 64 k-rows: the
// chunk's 64 x 128 packed bytes (TMA, 128-byte swizzle) and 16 x 64 activation bytes (TMA, 64-byte swizzle; rows
// beyond M and columns beyond K arrive as zeros).  Each consumer warp owns one 128-column block of the chunk
// for the whole item, so there is nothing to reduce between warps and no barrier other than the ring's; its
// epilogue writes 16-byte runs of C from registers.
//
// One problem alone has too few whole-K items to fill the GPU, so the single-problem launch cuts K into slices.
// Preferred form: a thread-block cluster of 2, 4 or 8 CTAs per (chunk, row group), one slice per CTA and exactly one
// item per CTA.  Every CTA leaves its partial tile in its own shared memory (over the idle ring), the
// cluster meets at a barrier, and CTA r sums the r-th share of the tile over all CTAs through distributed shared
// memory and stores it: no atomics, no zeroing of C.  Where that does not fit (more items than resident CTAs) the
// slices add into a zeroed C with red.global.add, which the L2 retires at about 160 per ns: the count of slices is
// then chosen against that cost.
#pragma once
#include <cuda.h>
#include <cstdint>
#include "kernel_gemv.cuh"
#include "ptx_sm100.cuh"

namespace tb200 {

constexpr int kMmaConsumerWarps = 4;
constexpr int kMmaThreads = (kMmaConsumerWarps + 1) * 32;
constexpr int kMmaStages = 6;
constexpr int kMmaStageRows = 64;                 // k-rows per stage
constexpr int kMmaStageW = 8192;                  // 64 rows x 128 packed bytes
constexpr int kMmaStageA = 1024;                  // 16 rows x 64 activation bytes
constexpr int kMmaStageBytes = kMmaStageW + kMmaStageA;     // 9 KB: stages stay 1024-byte aligned
constexpr int kMmaItemCols = 512;
constexpr int kMmaBoxRows = 16;                   // rows of the activation box (a row group has 8 or 16)
constexpr int kMmaCtasPerSm = 4;
constexpr size_t kMmaSmemBytes = 1024 + size_t(kMmaStages) * kMmaStageBytes + 2 * kMmaStages * 8 + 16;

struct alignas(64) MmaProblem {
    CUtensorMap tmap_w;        // packed W [K][N/4] bytes, box 128 B x 64 rows, 128-byte swizzle
    CUtensorMap tmap_a;        // A [M][K] bytes, box 64 B x 16 rows, 64-byte swizzle
    int32_t* C;
    long long ldc;
    int M, K, N;
    int c_vec_ok;              // C and ldc allow 16-byte stores
};
struct MmaItem {
    int problem, chunk;
    int row0;                  // bits 0-15: first row of the row group; bit 16: add into C instead of storing
    int span;                  // bits 0-15: first stage; bits 16-31: number of stages (0 = all of K)
};

__device__ __forceinline__ void ldmatrix_x2_trans_b8_regs(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr)
                 : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_b16(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr)
                 : "memory");
}
// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_u8s8(int32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One problem per launch: the items are enumerated arithmetically instead of read from a table.  Item i is
// (k-slice, row group, chunk) with the chunk running fastest, and CTA b takes items b, b + grid, ...: CTAs next to
// each other read the same weight rows of neighbouring chunks at the same time, which keeps their 128-byte row
// segments in the same DRAM pages.
struct MmaSingle {
    int chunks, row_groups, slices, tiles_per_slice, total_tiles, add;
    int cluster;               // 0, or the cluster size (= slices): item of CTA b is (slice b % cluster, b / cluster)
    int group_rows;            // rows per row group: 8 * NG
};
__device__ __forceinline__ MmaItem mma_single_item(const MmaSingle& sg, int i) {
    if (sg.cluster) {
        const int sl = i % sg.cluster, rest = i / sg.cluster;
        const int chunk = rest % sg.chunks, rg = rest / sg.chunks;
        const int tile0 = sl * sg.tiles_per_slice;
        const int nt = max(0, min(sg.tiles_per_slice, sg.total_tiles - tile0));
        return MmaItem{0, chunk, rg * sg.group_rows, tile0 | (nt << 16) | (nt == 0 ? (1 << 31) : 0)};
    }
    const int chunk = i % sg.chunks, rest = i / sg.chunks;
    const int rg = rest % sg.row_groups, sl = rest / sg.row_groups;
    const int tile0 = sl * sg.tiles_per_slice;
    const int nt = min(sg.tiles_per_slice, sg.total_tiles - tile0);
    return MmaItem{0, chunk, (rg * sg.group_rows) | (sg.add << 16), tile0 | (nt << 16)};
}

// Stages of an item: bits 16-30 of span, all of K when they are zero, none when bit 31 is set (a cluster slice
// beyond the end of K).
__device__ __forceinline__ int mma_item_tiles(const MmaItem& it, int K) {
    if (it.span < 0) return 0;
    const int n = it.span >> 16;
    return n ? n : (K + kMmaStageRows - 1) / kMmaStageRows;
}

// The 16-byte group (4 columns of one batch row) that accumulator registers (ng, rr, bp, hh) of a lane make up:
// batch row 8 ng + 2 (lane % 4) + rr of the row group, byte column 16 bp + 8 hh + lane / 4 of the warp's block.
// Groups are numbered p = ((ng * 2 + rr) * 2 + bp) * 2 + hh.
template <bool kSingle, int NG>
__global__ void __launch_bounds__(kMmaThreads, kMmaCtasPerSm)
ternary_decode_mma_kernel(const __grid_constant__ MmaProblem single, const MmaSingle sg,
                          const MmaProblem* __restrict__ probs, const MmaItem* __restrict__ items,
                          const int* __restrict__ cta_first, int32_t* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* stages = base;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + kMmaStages * kMmaStageBytes);
    uint64_t* empty = full + kMmaStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMmaStages);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool clustered = kSingle && sg.cluster > 0;
    const int item_lo = kSingle ? static_cast<int>(blockIdx.x) : cta_first[blockIdx.x];
    const int item_hi = clustered ? item_lo + 1 : kSingle ? sg.chunks * sg.row_groups * sg.slices : cta_first[blockIdx.x + 1];
    const int item_step = kSingle ? static_cast<int>(gridDim.x) : 1;
    if (tid == 0) {
        for (int s = 0; s < kMmaStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kMmaConsumerWarps);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();

    if (warp == kMmaConsumerWarps) {
        // ------------------------------------------------------------ producer lane
        if (lane == 0) {
            uint32_t t = 0;
            bool ok = true;
            for (int i = item_lo; ok && i < item_hi; i += item_step) {
                const MmaItem it = kSingle ? mma_single_item(sg, i) : items[i];
                const MmaProblem* p = kSingle ? &single : probs + it.problem;
                const int tile0 = it.span & 0xffff;
                const int ntiles = mma_item_tiles(it, p->K);
                const int row0 = it.row0 & 0xffff;
                for (int tx = 0; tx < ntiles; ++tx, ++t) {
                    const uint32_t s = t % kMmaStages;
                    if (!mbar_wait(&empty[s], ((t / kMmaStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = stages + s * kMmaStageBytes;
                    const int k0 = (tile0 + tx) * kMmaStageRows;
                    mbar_arrive_expect_tx(&full[s], kMmaStageBytes);
                    tma_load_2d(st, &p->tmap_w, it.chunk * (kMmaItemCols / 4), k0, &full[s]);
                    tma_load_2d(st + kMmaStageW, &p->tmap_a, k0, row0, &full[s]);
                }
            }
            if (*abort_flag) {
                const uint32_t first = t > kMmaStages ? t - kMmaStages : 0;
                for (uint32_t j = first; j < t; ++j) mbar_drain(&full[j % kMmaStages], (j / kMmaStages) & 1);
            }
        }
    } else {
        // ------------------------------------------------------------ consumers: warp = 128-column block of the item
        const int cb = warp;
        // W: row address of this lane inside a 16-row block of the swizzled stage (16-byte chunk ^= row % 8)
        const uint32_t w_off = (lane & 15) * 128 + (((cb * 2 + (lane >> 4)) ^ (lane & 7)) << 4);
        // A: ldmatrix.x4 row addresses of the 16 x 32-byte tile of k-step 0: matrices (rows 0-7 | 8-15) x (bytes 0-15 | 16-31);
        // 64-byte swizzle: chunk ^= (row / 2) % 4.  k-step 1 is two chunks further (chunk ^ 2 after the swizzle).
        const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8;
        const uint32_t a_chunk = lane >> 4;
        const uint32_t a_swz = (a_row >> 1) & 3;
        const uint32_t a_off0 = kMmaStageW + a_row * 64 + ((a_chunk ^ a_swz) << 4);
        const uint32_t a_off1 = kMmaStageW + a_row * 64 + (((a_chunk + 2) ^ a_swz) << 4);
        const uint32_t stages_sa = smem_u32(stages);
        uint32_t t = 0;
        bool ok = true;
        for (int i = item_lo; ok && i < item_hi; i += item_step) {
            const MmaItem it = kSingle ? mma_single_item(sg, i) : items[i];
            const MmaProblem* p = kSingle ? &single : probs + it.problem;
            const int ntiles = mma_item_tiles(it, p->K);

            int32_t acc[2][4][NG][4];      // [byte-column pair bp][field j][batch-row group ng][C fragment]
            int32_t rs[NG][4];             // row sums: rs[ng][rr] for batch row 8 ng + 2 (lane % 4) + rr
#pragma unroll
            for (int ng = 0; ng < NG; ++ng) {
#pragma unroll
                for (int c = 0; c < 4; ++c) rs[ng][c] = 0;
#pragma unroll
                for (int bp = 0; bp < 2; ++bp)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[bp][j][ng][c] = 0;
            }

            for (int tx = 0; tx < ntiles; ++tx, ++t) {
                const uint32_t s = t % kMmaStages;
                if (!mbar_wait(&full[s], (t / kMmaStages) & 1, abort_flag)) { ok = false; break; }
                const uint32_t st = stages_sa + s * kMmaStageBytes;
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    // activations: a[0], a[2] = k 0-15, 16-31 of batch rows 0-7; a[1], a[3] = the same of rows 8-15
                    uint32_t a[4], r0[4], r1[4];
                    ldmatrix_x4_b16(a, st + (ks ? a_off1 : a_off0));
                    ldmatrix_x2_trans_b8_regs(r0, st + w_off + (2 * ks) * 2048);
                    ldmatrix_x2_trans_b8_regs(r1, st + w_off + (2 * ks + 1) * 2048);
#pragma unroll
                    for (int ng = 0; ng < NG; ++ng)
                        mma_u8s8(rs[ng], 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, a[ng], a[2 + ng]);
#pragma unroll
                    for (int bp = 0; bp < 2; ++bp)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t m = 0x03030303u << (2 * j);
                            const uint32_t w0 = (r0[2 * bp] ^ 0xAAAAAAAAu) & m, w1 = (r0[2 * bp + 1] ^ 0xAAAAAAAAu) & m;
                            const uint32_t w2 = (r1[2 * bp] ^ 0xAAAAAAAAu) & m, w3 = (r1[2 * bp + 1] ^ 0xAAAAAAAAu) & m;
#pragma unroll
                            for (int ng = 0; ng < NG; ++ng) mma_u8s8(acc[bp][j][ng], w0, w1, w2, w3, a[ng], a[2 + ng]);
                        }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }

            if (clustered) {
                // ---- partial results into this CTA's shared memory, over the ring (idle: this CTA has one item and
                //      every consumer warp is past its last stage).  Layout [warp][p][lane][4 columns].
                asm volatile("bar.sync 1, %0;" ::"n"(kMmaConsumerWarps * 32) : "memory");
#pragma unroll
                for (int ng = 0; ng < NG; ++ng)
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
                        for (int bp = 0; bp < 2; ++bp)
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                const int pgrp = ((ng * 2 + rr) * 2 + bp) * 2 + hh;
                                const int corr = 2 * rs[ng][rr];
                                uint4 v;
                                v.x = static_cast<uint32_t>((acc[bp][0][ng][2 * hh + rr] >> 0) - corr);
                                v.y = static_cast<uint32_t>((acc[bp][1][ng][2 * hh + rr] >> 2) - corr);
                                v.z = static_cast<uint32_t>((acc[bp][2][ng][2 * hh + rr] >> 4) - corr);
                                v.w = static_cast<uint32_t>((acc[bp][3][ng][2 * hh + rr] >> 6) - corr);
                                sts_v4(stages_sa + (((warp * (8 * NG) + pgrp) * 32 + lane) << 4), v);
                            }
                break;
            }
            if (!ok) break;

            // ---- epilogue from registers
            const int M = p->M, N = p->N;
            const bool add = (it.row0 >> 16) & 1;
            const int col_base = it.chunk * kMmaItemCols + cb * 128 + (lane >> 2) * 4;
#pragma unroll
            for (int ng = 0; ng < NG; ++ng)
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int row = (it.row0 & 0xffff) + 8 * ng + 2 * (lane & 3) + rr;
                    if (row >= M) continue;
                    const int corr = 2 * rs[ng][rr];
                    int32_t* crow = p->C + static_cast<size_t>(row) * p->ldc;
#pragma unroll
                    for (int bp = 0; bp < 2; ++bp)
#pragma unroll
                        for (int hh = 0; hh < 2; ++hh) {
                            const int col = col_base + (16 * bp + 8 * hh) * 4;
                            if (col >= N) continue;
                            int32_t v[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) v[j] = (acc[bp][j][ng][2 * hh + rr] >> (2 * j)) - corr;
                            if (add) {
#pragma unroll
                                for (int q = 0; q < 4; ++q) atomicAdd(crow + col + q, v[q]);
                            } else if (p->c_vec_ok) {
                                *reinterpret_cast<int4*>(crow + col) = make_int4(v[0], v[1], v[2], v[3]);
                            } else {
#pragma unroll
                                for (int q = 0; q < 4; ++q) crow[col + q] = v[q];
                            }
                        }
                }
        }
    }
    __syncthreads();
    if (clustered) {
        // ---- CTA r of the cluster sums groups p = r * P / S .. of every warp's tile over all CTAs and stores them
        cluster_sync_all();
        constexpr int P = 8 * NG;
        const int S = sg.cluster, rank = static_cast<int>(cluster_ctarank());
        if (warp < kMmaConsumerWarps && !*abort_flag) {
            const MmaItem it = mma_single_item(sg, blockIdx.x);
            const uint32_t stages_sa = smem_u32(stages);
            for (int pgrp = rank * P / S; pgrp < (rank + 1) * P / S; ++pgrp) {
                const int hh = pgrp & 1, bp = (pgrp >> 1) & 1, rr = (pgrp >> 2) & 1, ng = pgrp >> 3;
                const uint32_t src = stages_sa + (((warp * P + pgrp) * 32 + lane) << 4);
                int32_t v[4] = {0, 0, 0, 0};
                for (int q = 0; q < S; ++q) {
                    int4 x;
                    asm volatile("ld.shared::cluster.v4.s32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(x.x), "=r"(x.y), "=r"(x.z), "=r"(x.w)
                                 : "r"(dsmem_map(src, q)));
                    v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
                }
                const int row = (it.row0 & 0xffff) + 8 * ng + 2 * (lane & 3) + rr;
                const int col = it.chunk * kMmaItemCols + warp * 128 + (16 * bp + 8 * hh + (lane >> 2)) * 4;
                if (row < single.M && col < single.N) {
                    int32_t* dst = single.C + static_cast<size_t>(row) * single.ldc + col;
                    if (single.c_vec_ok) {
                        *reinterpret_cast<int4*>(dst) = make_int4(v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int x = 0; x < 4; ++x) dst[x] = v[x];
                    }
                }
            }
        }
        cluster_sync_all();        // nobody leaves while a peer may still read its shared memory
    }
    if (tid == 0 && *abort_flag && status) atomicMax(status, kStatusTimeout);
}

}  // namespace tb200
