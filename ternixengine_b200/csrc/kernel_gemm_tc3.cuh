// Prefill-regime kernel, paired CTAs, weights as the tensor-core A operand in tensor memory.
//
// The other tcgen05 kernels of this library expand every packed weight byte into four int8 bytes of shared
// memory, in the canonical operand layout, before the tensor core can read them; that expansion (shared-memory
// stores, proxy fences, a second ring) is what bounds them.  tcgen05.mma can also take its A operand from tensor
// memory, where row i of A sits in lane i and four K-bytes fill one 32-bit column.  So this kernel computes the
// product transposed,
//     C^T[n][m] = sum_k W[k][n] * A[m][k],
// with the weights as the A operand and the activations, untouched, as the B operand:
//   * activations: 128 rows x 256 K-bytes per CTA and stage (two boxes of 128 K-bytes), straight from TMA into the
//     K-major 128-byte-swizzle layout the B descriptor reads (the pair's two halves make the N = 256 columns of the instruction);
//   * weights: 256 k-rows x 32 packed bytes per CTA and stage (its 128 weight columns), TMA with the 32-byte
//     swizzle, through a ring of their own that runs eight k-blocks ahead (they are small and mostly come from DRAM;
//     the activations come from L2 through a ring of four; a weight slot is free as soon as the expanders have read
//     it).  An expander warp reads them with ldmatrix.m16n16.x2.trans.b8, which leaves, in lane (c, t) =
//     (lane / 4, lane % 4), the bytes of k-rows 4t..4t+3 of packed byte column c -- exactly what lane (c, t) has to
//     supply to tcgen05.st.16x128b for operand row c, columns t.  So the operand rows (tensor-memory lanes) are
//     numbered the way the load delivers them: lane l of a 32-lane quarter holds weight column 4 (l % 8) + l / 8 of
//     the quarter's 32, and no data moves between lanes.  A field is decoded without sign extension:
//     (T << (6 - 2f)) & 0xC0C0C0C0 leaves every byte as 0x00, 0x40 or 0xC0, i.e. 0, +64, -64 as int8; the
//     accumulators hold 64 x the sum and the epilogue's arithmetic shift by 6 is exact.  17 instructions per 1024
//     weights and warp (the first version, which kept the natural row order, needed eight shuffles and 45
//     instructions, and the tensor pipe waited for the expanders 11 % of the time).  Nothing expanded ever touches
//     shared memory; the rings hold 40 KB per 256-deep stage (32 KB of activations, 8 KB of packed weights) instead of 112 KB.
//   * epilogue: lane = weight column (in the expanders' numbering), tensor-memory column = activation row.  The
//     epilogue warps read their whole share of the accumulator into registers and release it at once (about 700
//     cycles from the last MMA's retirement to the first MMA of the next tile).  A step then moves 32 activation
//     rows x 128 columns into a staging buffer in shared memory, row-major as in C, and one thread hands the buffer
//     to the TMA unit as a tensor store; the stores run in the background under the next tile's MMAs, a few hundred
//     nanoseconds apart (see kTc3StorePauseNsPerStage).
//
// Tensor memory (512 columns per CTA): columns 0-255 the accumulator (128 weight columns x 256 activation rows,
// int32, single-buffered; two buffers of 128 rows in the 128-row form), columns 256-511 the A ring: 4 stages x 64
// columns (256 K-bytes per lane).
// Stages are 256 deep because every hand-over of a stage (TMA -> expanders -> leader -> tensor core -> producer)
// costs about the same whatever it carries: 128-deep stages ran 10 % slower.  A pair MMA with 128 instead of 256
// activation rows takes as long as the full one, so the 128-row form (which could double-buffer its accumulator)
// runs at two thirds of the rate and only serves products with at most 128 rows.
//
// Where the time goes (4096 x 8192 x 28672, per-CTA cycle counters): a tile of 32 stages takes 35,900 cycles for
// 32,768 cycles of MMAs.  About 800 are the hand-over of the single accumulator; most of the rest are stages that
// wait for their TMA loads in the 5,000 cycles after a tile ends, when every CTA's epilogue stores its 128 KB: the
// loads' latency doubles meanwhile (with the stores left out the tile takes 34,100 cycles and the SM clock under
// the power cap is higher as well).  A deeper shared-memory ring, L2 prefetches of the weight boxes, evict-first
// stores and stores from registers were all measured and change nothing.
//
// Roles per CTA (warps, in whole warpgroups because registers are moved between them): 0 activation producer;
// 1 MMA issuer (leader CTA only: eight M=256 N=256 K=32 pair MMAs per stage, commit -> `empty` of both CTAs);
// 2 weight producer; 3 idle; 4-11 expanders (lane quarter = warp % 4; the two warps of a quarter take the stages
// in turn; after tcgen05.wait::st they arrive on the leader's `ready`, quarter 0 only once the stage's activations
// have landed, so `ready` says that too); 12-19 epilogue, two groups of four that take alternate steps.
//
// Exactness: int8 x int8 -> int32 on weights decoded as -64/0/+64; |64 * sum| <= 64 * 128 * K < 2^31 for
// K <= 262143 (the host checks), and the shift by 6 in the epilogue restores the sum exactly.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "kernel_gemm_tc2.cuh"

namespace tb200 {

#ifndef TB200_TC3_STAGES
#define TB200_TC3_STAGES 4
#endif
constexpr int kTc3Stages = TB200_TC3_STAGES;
constexpr int kTc3TileW = 256;                    // weight columns per pair (128 per CTA)
constexpr int kTc3TileA = 256;                    // activation rows per pair (128 loaded per CTA)
#ifndef TB200_TC3_BK
#define TB200_TC3_BK 256
#endif
#ifndef TB200_TC3_EXPAND_WARPS
#define TB200_TC3_EXPAND_WARPS 8
#endif
#define TB200_TC3_EXPAND_WARPS_ TB200_TC3_EXPAND_WARPS
constexpr int kTc3BK = TB200_TC3_BK;              // K-bytes per stage: 128 or 256 (the latter as two 128-byte-swizzle boxes)
static_assert(kTc3BK == 256, "a stage is two boxes of 128 K-bytes");
constexpr int kTc3WpRowBytes = 32;
constexpr int kTc3WpBytes = kTc3BK * kTc3WpRowBytes;
constexpr uint32_t kTc3ARingCol = 256, kTc3AStageCols = kTc3BK / 4;
// Per tile form (TA = activation rows per pair instruction): the shared-memory ring of TMA stages, the accumulator
// buffers in tensor memory, and the sizes that follow.  The operand ring in tensor memory always has kTc3Stages slots.
template <int TA>
struct Tc3Geom {
    static_assert(TA == 128 || TA == 256, "activation rows per pair instruction");
    static constexpr int kRowsPerCta = TA / 2;                   // activation rows a CTA loads per stage
    static constexpr int kActBox = kRowsPerCta * 128;            // one TMA box: rows x 128 K-bytes, 128-byte swizzle
    static constexpr int kActBytes = 2 * kActBox;
    static constexpr int kStageBytes = kActBytes;                // a stage of the activation ring (the weights have a ring of their own)
    static constexpr int kAccBufs = 256 / TA;                    // accumulators of TA columns in tensor-memory columns 0-255
#ifdef TB200_TC3_SMEM_STAGES_128
    static constexpr int kSmemStages = TA == 128 ? TB200_TC3_SMEM_STAGES_128 : kTc3Stages;
#else
    static constexpr int kSmemStages = TA == 128 ? 6 : kTc3Stages;
#endif
    // an expander warp meets every phase of the barriers it waits on, and the stage whose retirement frees its operand
    // slot (kTc3Stages back) belongs to a shared-memory slot that only this same warp's next stages can complete again
    static_assert(kSmemStages >= kTc3Stages && kSmemStages % (TB200_TC3_EXPAND_WARPS_ / 4) == 0 &&
                      (kSmemStages - kTc3Stages) % (TB200_TC3_EXPAND_WARPS_ / 4) == 0,
                  "ring sizes");
};
#ifndef TB200_TC3_SLEEP_NS
#define TB200_TC3_SLEEP_NS 64
#endif
#ifndef TB200_TC3_ACC_SLEEP_NS
#define TB200_TC3_ACC_SLEEP_NS 64        // pause between the epilogue warps' probes of the "accumulator full" barrier
#endif
constexpr int kTc3ExpandWarps = TB200_TC3_EXPAND_WARPS;      // 4, 8 or 12: one, two or three warps per lane quarter
constexpr int kTc3WarpsPerQuarter = kTc3ExpandWarps / 4;     // they take the stages in turn (stage it -> warp it % n)
static_assert(TB200_TC3_STAGES % (TB200_TC3_EXPAND_WARPS / 4) == 0,
              "a warp must meet every phase of the barriers it waits on: stages a multiple of warps per quarter");
// Roles sit in whole warpgroups (4 warps) because registers are moved between them at kernel start: warps 0-3
// control (TMA producer, MMA issuer, two idle), then the expanders, then the epilogue.
constexpr int kTc3FirstExpandWarp = 4;
constexpr int kTc3FirstEpilogueWarp = kTc3FirstExpandWarp + kTc3ExpandWarps;    // 12
constexpr unsigned kTc3StorePauseNsPerStage = 40;   // pause between an epilogue group's steps, per k-stage of the tile
#ifndef TB200_TC3_EPI_GROUPS
#define TB200_TC3_EPI_GROUPS 2
#endif
constexpr int kTc3EpiGroups = TB200_TC3_EPI_GROUPS;                              // groups of 4 epilogue warps (one per lane quarter)
constexpr int kTc3Threads = (kTc3FirstEpilogueWarp + 4 * kTc3EpiGroups) * 32;     // 640
constexpr int kTc3StepsPerWarp = kTc3TileA / 32 / kTc3EpiGroups;                   // accumulator steps of 32 rows per epilogue warp
// Registers per thread after the hand-over at kernel start (setmaxnreg): an epilogue warp holds its whole share of
// the accumulator (kTc3StepsPerWarp x 32 registers) so that tensor memory is free again a few hundred cycles after
// the last MMA of a tile, long before the stores have drained.  The kernel is launched with 96 registers per thread
// (640 x 96 = 61,440), and 128 x 48 + 256 x 64 + 256 x 152 = 61,440 is exactly that.
constexpr int kTc3RegsControl = 48, kTc3RegsExpand = 64, kTc3RegsEpilogue = 152;
static_assert(kTc3EpiGroups == 2 && kTc3ExpandWarps == 8, "the register counts above are worked out for this role layout");
static_assert(128 * kTc3RegsControl + kTc3ExpandWarps * 32 * kTc3RegsExpand + kTc3EpiGroups * 128 * kTc3RegsEpilogue <=
                  kTc3Threads * 96,
              "register hand-over exceeds what the CTA owns at launch");
template <int kRegs>
__device__ __forceinline__ void warpgroup_regs_release() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void warpgroup_regs_acquire() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
#ifndef TB200_TC3_EPI_BUFS
#define TB200_TC3_EPI_BUFS 1
#endif
constexpr int kTc3EpiBufs = TB200_TC3_EPI_BUFS;   // staging buffers per epilogue group
constexpr int kTc3EpiBytes = 32 * 128 * 4;        // one step of the epilogue: 32 activation rows x 128 weight columns
#ifndef TB200_TC3_W_STAGES
#define TB200_TC3_W_STAGES 8
#endif
constexpr int kTc3WStages = TB200_TC3_W_STAGES;   // packed-weight ring: 8 KB stages, loaded up to this many k-blocks ahead (they come from DRAM)
static_assert(kTc3WStages % (TB200_TC3_EXPAND_WARPS_ / 4) == 0, "an expander warp must meet every phase of the barriers it waits on");
template <int TA>
constexpr size_t tc3_smem_bytes() {
    return 1024 + size_t(Tc3Geom<TA>::kSmemStages) * Tc3Geom<TA>::kStageBytes + size_t(kTc3WStages) * kTc3WpBytes +
           size_t(kTc3EpiGroups) * kTc3EpiBufs * kTc3EpiBytes + 512;
}
static_assert(tc3_smem_bytes<128>() <= 227 * 1024 && tc3_smem_bytes<256>() <= 227 * 1024, "shared memory: 227 KB per CTA");
constexpr size_t kTc3SmemBytes = tc3_smem_bytes<256>();

__device__ __forceinline__ void tc_mma_i8_pair_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                      uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 lanes x 8 columns: r0/r1 = rows lane/4 and lane/4 + 8 at column lane%4, r2/r3 = the same rows at column 4 + lane%4.
__device__ __forceinline__ void tmem_st_16x128_x2(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2),
                 "r"(r3)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// ldmatrix without a memory clobber: the loads of a stage are issued back to back and only ordered by their uses
// (the stage's shared memory is stable between the barrier wait before and the barrier arrive after them).
__device__ __forceinline__ void ldmatrix_x2_trans_b8_nc(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}
// Field F of every byte of T as int8 scaled by 64: codes 0, 1, 3 -> 0, +64, -64 (the two top bits of a byte ARE the
// sign-extended code once the field has been shifted there).
template <int F>
__device__ __forceinline__ uint32_t decode_field_x64(uint32_t T) {
    if constexpr (F == 3) return T & 0xC0C0C0C0u;
    else return (T << (6 - 2 * F)) & 0xC0C0C0C0u;
}

// Where the finished tiles go: the local C first, then the same place in each peer's C (fused gather over NVLink:
// one TMA tensor store per destination from the same staging buffer).
constexpr int kTc3MaxDest = 8;
struct Tc3Stores {
    CUtensorMap tmap_c[kTc3MaxDest];     // C [M][N] int32 with its row pitch, box 128 columns x 32 rows
    int count;                           // 0: C cannot be described to the TMA unit; stores from registers into `C`
};

// Grouped mode: one launch walks the tiles of many products (a "problem group"); descriptors and destinations come
// from tables in global memory, and every pair owns a fixed slice of the tile list (Tc2Tile: problem, activation
// block, weight block).
struct alignas(64) Tc3Problem {
    CUtensorMap tmap_a;        // A: [M rows][K bytes], box 128 x 128, 128-byte swizzle
    CUtensorMap tmap_w;        // packed W: [K rows][N/4 bytes], box 32 B x 128 rows, 32-byte swizzle
    Tc3Stores stores;
    int32_t* C;
    long long ldc;
    int M, K, N, pad;
};

// The tile sequence of one CTA pair.  Every warp role constructs its own walker and sees the same sequence.
template <bool kGrouped>
struct Tc3Walk {
    const CUtensorMap* ta;
    const CUtensorMap* tw;
    const Tc3Stores* st;
    int32_t* C;
    long long ldc;
    int M, N, a_t, w_t, k_blocks;
    // single product
    int tile, num_tiles, stride, a_tiles;
    // group
    const Tc3Problem* probs;
    const Tc2Tile* tiles;
    int idx, end;

    // (grouped) ask the TMA unit to fetch the operand descriptors of the tile that next() will return
    __device__ __forceinline__ void prefetch_next_maps() const {
        if (idx < end) {
            const Tc3Problem* p = probs + tiles[idx].problem;
            tma_prefetch_desc(&p->tmap_a);
            tma_prefetch_desc(&p->tmap_w);
        }
    }
    __device__ __forceinline__ void prefetch_next_store_map() const {
        if (idx < end) {
            const Tc3Problem* p = probs + tiles[idx].problem;
            if (p->stores.count > 0) tma_prefetch_desc(&p->stores.tmap_c[0]);
        }
    }
    __device__ __forceinline__ bool next() {
        if constexpr (kGrouped) {
            if (idx >= end) return false;
            const Tc2Tile t = tiles[idx++];
            const Tc3Problem* p = probs + t.problem;
            ta = &p->tmap_a; tw = &p->tmap_w; st = &p->stores;
            C = p->C; ldc = p->ldc; M = p->M; N = p->N;
            a_t = t.m_t; w_t = t.n_t;
            k_blocks = (p->K + kTc3BK - 1) / kTc3BK;
            return true;
        } else {
            if (tile >= num_tiles) return false;
            // activation block fastest: pairs that run together share few weight blocks and all of A
            a_t = tile % a_tiles; w_t = tile / a_tiles;
            tile += stride;
            return true;
        }
    }
};

__device__ __forceinline__ void sts_u16(uint32_t saddr, uint16_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(saddr), "h"(v) : "memory");
}

// kBf16: the epilogue emits bfloat16 = bf16_rn((float(c) * row_scale[m]) * w_scale) instead of int32 (the scaling
// step that follows the product in a BitNet-style layer); `stores` then describes bfloat16 tensors and `C`, `ldc`
// are the bfloat16 output and its pitch in elements.
// TA: activation rows per pair instruction (the MMA's N), 256 or 128.  With 128 each CTA loads 64 rows per stage, the
// pair's MMAs are half as long, and tensor-memory columns 0-255 hold TWO accumulators: the MMAs of the next tile run
// while the epilogue warps empty the previous one.  The shared-memory ring is then deeper than the operand ring in
// tensor memory (a stage passes in half the time, the latency of a TMA load stays what it is).
template <bool kGrouped, bool kBf16 = false, int TA = kTc3TileA>
__global__ void __launch_bounds__(kTc3Threads, 1)
ternary_gemm_tc3_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                        const __grid_constant__ Tc3Stores stores, int32_t* __restrict__ C, int M, int K, int N,
                        long long ldc, const Tc3Problem* __restrict__ probs, const Tc2Tile* __restrict__ tiles,
                        const int* __restrict__ pair_first, int32_t* __restrict__ status,
                        const float* __restrict__ row_scale = nullptr, float w_scale = 1.0f) {
    static_assert(!(kGrouped && kBf16), "the dequantising epilogue is built for single products");
    using G = Tc3Geom<TA>;
    constexpr int kRowsPerCta = G::kRowsPerCta;                            // activation rows a CTA loads per stage
    constexpr uint32_t kStageTx = G::kStageBytes;                          // bytes a stage's TMA loads deliver
    constexpr int S = G::kSmemStages;                                      // ring of TMA stages in shared memory
    constexpr int TS = kTc3Stages;                                         // ring of operand stages in tensor memory
    constexpr int BUFS = G::kAccBufs;
    constexpr int kSteps = TA / 32 / kTc3EpiGroups;                        // accumulator steps of 32 rows per epilogue warp
    constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(TA >> 3) << 17) |
                                (static_cast<uint32_t>(256 >> 4) << 24);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sAct = base;                                            // [S][2 boxes][rows][128 k]  128-byte swizzle
    constexpr int WS = kTc3WStages;
    uint8_t* sWp = sAct + S * G::kActBytes;                          // [WS][256 k][32]            32-byte swizzle
    uint8_t* sEpi = sWp + WS * kTc3WpBytes;                          // [groups][bufs][32 rows][128] int32
    uint64_t* bars = reinterpret_cast<uint64_t*>(sEpi + kTc3EpiGroups * kTc3EpiBufs * kTc3EpiBytes);
    uint64_t* full = bars;                         // [S]  this CTA's TMA bytes of a stage have landed
    uint64_t* empty = full + S;                    // [S]  the pair's MMAs on a stage have retired
    uint64_t* ready = empty + S;                   // [TS] (leader) both CTAs' operands of a stage are in place
    uint64_t* acc_full = ready + TS;               // [BUFS]
    uint64_t* acc_empty = acc_full + BUFS;         // [BUFS] (leader)
    uint64_t* w_full = acc_empty + BUFS;           // [WS] a packed-weight stage has landed
    uint64_t* w_empty = w_full + WS;               // [WS] this CTA's four lane quarters have read it
    uint64_t* drain = w_empty + WS;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    auto make_walk = [&]() {
        Tc3Walk<kGrouped> w{};
        if constexpr (kGrouped) {
            w.probs = probs; w.tiles = tiles;
            w.idx = pair_first[pair]; w.end = pair_first[pair + 1];
        } else {
            w.ta = &tmap_a; w.tw = &tmap_w; w.st = &stores;
            w.C = C; w.ldc = ldc; w.M = M; w.N = N;
            w.a_tiles = (M + TA - 1) / TA;
            w.num_tiles = w.a_tiles * ((N + kTc3TileW - 1) / kTc3TileW);
            w.k_blocks = (K + kTc3BK - 1) / kTc3BK;
            w.tile = pair; w.stride = num_pairs;
        }
        return w;
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < TS; ++s) mbar_init(&ready[s], 2 * 4);
        for (int s = 0; s < WS; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], 4);
        }
        for (int b = 0; b < BUFS; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8 * kTc3EpiGroups);
        }
        mbar_init(drain, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc_pair<512>(tmem_slot);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // Each role branch opens with its register hand-over, so that the compiler sees how many registers the code behind it may use.
    if (warp < kTc3FirstExpandWarp) {
      warpgroup_regs_release<kTc3RegsControl>();
      if (warp == 0) {
        // ================================================================ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            Tc3Walk<kGrouped> w = make_walk();
            if constexpr (!kGrouped) {
                tma_prefetch_desc(&tmap_a);
                tma_prefetch_desc(&tmap_w);
            } else {
                w.prefetch_next_maps();
            }
            while (ok && w.next()) {
                // the descriptors of the tile after this one: fetched while this tile's loads are issued, so that a
                // change of problem does not stall the ring for the latency of two descriptor reads
                if constexpr (kGrouped) w.prefetch_next_maps();
                const int row0 = w.a_t * TA + rank * kRowsPerCta;
                for (int kb = 0; kb < w.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % S;
                    if (!mbar_wait_backoff(&empty[s], ((it / S) & 1) ^ 1, abort_flag, 32)) { ok = false; break; }
                    mbar_arrive_expect_tx(&full[s], kStageTx);
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        tma_load_2d(sAct + s * G::kActBytes + j * G::kActBox, w.ta, kb * kTc3BK + j * 128, row0, &full[s]);
                }
            }
            if (!ok) {
                const uint32_t first = it > static_cast<uint32_t>(S) ? it - S : 0;
                for (uint32_t j = first; j < it; ++j) mbar_drain(&full[j % S], (j / S) & 1);
            }
        }
      } else if (warp == 1) {
        // ================================================================ MMA issuer (leader CTA only)
        if (leader && lane == 0) {
            uint32_t it = 0, lt = 0;
            bool ok = true;
            Tc3Walk<kGrouped> w = make_walk();
            for (; ok && w.next(); ++lt) {
                const uint32_t ab = lt % BUFS;
                if (!mbar_wait(&acc_empty[ab], ((lt / BUFS) & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + ab * TA;
                for (int kb = 0; kb < w.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % S, ts = it % TS;
                    if (!mbar_wait(&ready[ts], (it / TS) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t act_addr = smem_u32(sAct + s * G::kActBytes);
                    const uint32_t a_col = tmem_base + kTc3ARingCol + ts * kTc3AStageCols;
#pragma unroll
                    for (int g = 0; g < kTc3BK / 32; ++g) {
                        const uint64_t db = umma_desc_sw128(act_addr + (g >> 2) * G::kActBox + (g & 3) * 32, 16, 1024);
                        tc_mma_i8_pair_tmem_a(acc, a_col + 8 * g, db, kIdesc, (kb != 0 || g != 0) ? 1u : 0u);
                    }
                    tc_commit_pair_both(&empty[s]);
                }
                if (ok) tc_commit_pair_both(&acc_full[ab]);
            }
            tc_commit_pair(drain);
            mbar_wait(drain, 0, abort_flag);
        }
      } else if (warp == 2) {
        // ================================================================ packed weights: a ring of their own
        // The weight boxes are small (8 KB) and, unlike the activations, mostly come from DRAM, so they are requested
        // kTc3WStages k-blocks ahead instead of the activation ring's four; a slot is free again as soon as the four
        // expander quarters have read it, long before the stage's MMAs retire.
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            Tc3Walk<kGrouped> w = make_walk();
            if constexpr (kGrouped) w.prefetch_next_maps();
            else tma_prefetch_desc(&tmap_w);
            while (ok && w.next()) {
                if constexpr (kGrouped) w.prefetch_next_maps();
                const int wp_x = (w.w_t * kTc3TileW + rank * 128) / 4;
                for (int kb = 0; kb < w.k_blocks; ++kb, ++it) {
                    const uint32_t sw = it % WS;
                    if (!mbar_wait_backoff(&w_empty[sw], ((it / WS) & 1) ^ 1, abort_flag, 32)) { ok = false; break; }
                    mbar_arrive_expect_tx(&w_full[sw], kTc3WpBytes);
                    tma_load_2d(sWp + sw * kTc3WpBytes, w.tw, wp_x, kb * kTc3BK, &w_full[sw]);
                }
            }
            if (!ok) {
                const uint32_t first = it > static_cast<uint32_t>(WS) ? it - WS : 0;
                for (uint32_t j = first; j < it; ++j) mbar_drain(&w_full[j % WS], (j / WS) & 1);
            }
        }
      }     // warp 3 has nothing to do: it only fills the control warpgroup
    } else if (warp < kTc3FirstEpilogueWarp) {
        warpgroup_regs_release<kTc3RegsExpand>();
        // ================================================================ expanders: packed bytes -> int8 rows of the A operand
        // The warp of lane quarter q writes operand rows 32q .. 32q+31: packed byte columns 8q .. 8q+7 of a row, i.e.
        // half (q & 1) of the 16-byte chunk q / 2, in all four fields.
        const uint32_t q = warp & 3;
        const uint32_t slot = (warp - kTc3FirstExpandWarp) >> 2;       // this warp's turn among the warps of its quarter
        // ldmatrix.x2: matrix 0 = k 0-15, matrix 1 = k 16-31 of a 32-deep group, both of chunk q / 2; row (lane & 15),
        // 32-byte swizzle (address bit 4 ^= address bit 7, i.e. chunk ^= bit 2 of the row).
        // After the load lane (c, t) = (lane / 4, lane % 4) holds k-bytes 4t..4t+3 of byte column 8q + c (register q & 1
        // of each matrix) -- exactly what lane (c, t) has to supply to tcgen05.st.16x128b for operand row c, columns t.
        // So the operand rows are numbered the way the load delivers them: lane l of the quarter holds byte column
        // l % 8 in field l / 8, i.e. weight column 4 (l % 8) + l / 8 of the quarter's 32, and no data moves between
        // lanes.  The epilogue undoes the numbering when it writes the staging buffer.
        const uint32_t r_in = lane & 15;
        const uint32_t ld_off = (lane >> 4) * 512 + r_in * 32 + (((q >> 1) ^ ((r_in >> 2) & 1)) << 4);
        const bool odd = (q & 1) != 0;
        const uint32_t wp_sa = smem_u32(sWp);
        const uint32_t t_lane = (q * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        Tc3Walk<kGrouped> w = make_walk();
        while (ok && w.next()) {
            for (int kb = 0; kb < w.k_blocks; ++kb, ++it) {
                if (it % kTc3WarpsPerQuarter != slot) continue;
                const uint32_t s = it % S, ts = it % TS, sw = it % WS;
                if (!mbar_wait_backoff(&w_full[sw], (it / WS) & 1, abort_flag, TB200_TC3_SLEEP_NS)) { ok = false; break; }
                const uint32_t wp = wp_sa + sw * kTc3WpBytes + ld_off;
                uint32_t X[kTc3BK / 32], Y[kTc3BK / 32];
#pragma unroll
                for (int g = 0; g < kTc3BK / 32; ++g) {
                    uint32_t m[4];
                    ldmatrix_x2_trans_b8_nc(m, wp + g * 1024);
                    X[g] = odd ? m[1] : m[0];
                    Y[g] = odd ? m[3] : m[2];
                }
                {
                    // The operand slot in tensor memory is free once the MMAs of stage it - TS have retired, which is what
                    // the `empty` barrier of that stage's activation slot says.  (That barrier cannot be a phase ahead:
                    // its next completion needs stage it - TS + S >= it expanded, and this warp expands in order.)
                    if (it >= static_cast<uint32_t>(TS)) {
                        const uint32_t j = it - TS;
                        if (!mbar_wait_backoff(&empty[j % S], (j / S) & 1, abort_flag, 32)) { ok = false; break; }
                    }
                    tc_fence_after_sync();
                }
                const uint32_t a_col = tmem_base + kTc3ARingCol + ts * kTc3AStageCols + t_lane;
#pragma unroll
                for (int g = 0; g < kTc3BK / 32; ++g) {
                    tmem_st_16x128_x2(a_col + 8 * g, decode_field_x64<0>(X[g]), decode_field_x64<1>(X[g]),
                                      decode_field_x64<0>(Y[g]), decode_field_x64<1>(Y[g]));
                    tmem_st_16x128_x2(a_col + (16u << 16) + 8 * g, decode_field_x64<2>(X[g]), decode_field_x64<3>(X[g]),
                                      decode_field_x64<2>(Y[g]), decode_field_x64<3>(Y[g]));
                }
                // the stage's packed bytes have been decoded out of their registers: the weight slot is free
                __syncwarp();
                if (lane == 0) mbar_arrive(&w_empty[sw]);
                tmem_st_wait();
                tc_fence_before_sync();
                // `ready` also has to say that this CTA's activations of the stage have landed: quarter 0 answers for that
                if (q == 0 && !mbar_wait_backoff(&full[s], (it / S) & 1, abort_flag, 32)) { ok = false; break; }
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(&ready[ts]);
                    else mbar_arrive_remote(&ready[ts], 0);
                }
            }
        }
    } else {
        warpgroup_regs_acquire<kTc3RegsEpilogue>();
        // ================================================================ epilogue: 128 weight columns x 256 activation rows
        // Lane = weight column, registers = activation rows.  A step moves 32 activation rows x 128 columns from
        // tensor memory into a staging buffer in shared memory, row-major as in C (a warp writes 128 contiguous bytes
        // per row: no bank conflicts), and one thread hands the buffer to the TMA unit (cp.async.bulk.tensor store).
        // The accumulator is released as soon as it has been read: the stores to global memory, whose rate per SM is
        // what an epilogue out of registers waits for, run in the background under the next tile's MMAs.
        // Lane l of quarter q holds weight column 32q + 4 (l % 8) + l / 8 (the expanders' numbering), and 64 x the sum.
        const uint32_t q = warp & 3;
        const uint32_t colp = q * 32 + 4 * (lane & 7) + (lane >> 3);
        const int eg = (warp - kTc3FirstEpilogueWarp) >> 2;             // group: takes steps eg, eg + groups, ...
        const bool elected = ((warp - kTc3FirstEpilogueWarp) & 3) == 0 && lane == 0;
        const uint32_t epi_sa = smem_u32(sEpi);
        uint32_t lt = 0, step = 0;                                      // step: steps taken by this group so far
        bool ok = true;
        Tc3Walk<kGrouped> w = make_walk();
        if constexpr (kGrouped) {
            if (elected) w.prefetch_next_store_map();
        }
        for (; ok && w.next(); ++lt) {
            if constexpr (kGrouped) {
                if (elected) w.prefetch_next_store_map();
            }
            const int a_t = w.a_t;
            const Tc3Stores* dst = w.st;
            const int M = w.M, N = w.N;
            const long long ldc = w.ldc;
            int32_t* C = w.C;
            const uint32_t ab = lt % BUFS;
            if (!mbar_wait_backoff(&acc_full[ab], (lt / BUFS) & 1, abort_flag, TB200_TC3_ACC_SLEEP_NS)) { ok = false; break; }
            tc_fence_after_sync();
            const int col0 = w.w_t * kTc3TileW + rank * 128;
            // this warp's share of the accumulator into registers, all of it, and tensor memory is free again
            uint32_t r[kSteps][32];
#pragma unroll
            for (int i = 0; i < kSteps; ++i)
                tmem_ld_32x32(tmem_base + ((q * 32) << 16) + ab * TA + 32 * (eg + kTc3EpiGroups * i), r[i]);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(&acc_empty[ab]);
                else mbar_arrive_remote(&acc_empty[ab], 0);
            }
#pragma unroll
            for (int i = 0; i < kSteps; ++i, ++step) {
                const int c = eg + kTc3EpiGroups * i;
                const uint32_t buf = epi_sa + (eg * kTc3EpiBufs + step % kTc3EpiBufs) * kTc3EpiBytes;
                // the store that last read this buffer has finished reading
                if (elected) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kTc3EpiBufs - 1) : "memory");
                asm volatile("bar.sync %0, 128;" ::"r"(2 + eg) : "memory");
                const int row0 = a_t * TA + 32 * c;
                if constexpr (kBf16) {
                    // in place: r[i][j] becomes the bfloat16 bit pattern of the scaled value
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float rs = row0 + j < M ? __ldg(row_scale + row0 + j) : 0.0f;
                        const __nv_bfloat16 y = __float2bfloat16_rn((static_cast<float>(static_cast<int32_t>(r[i][j]) >> 6) * rs) * w_scale);
                        r[i][j] = static_cast<uint32_t>(__bfloat16_as_ushort(y));
                    }
                }
                if (dst->count > 0) {
                    if constexpr (kBf16) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) sts_u16(buf + ((j * 128 + colp) << 1), static_cast<uint16_t>(r[i][j]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            sts_u32(buf + ((j * 128 + colp) << 2), static_cast<uint32_t>(static_cast<int32_t>(r[i][j]) >> 6));
                    }
                    fence_proxy_async_smem();
                    asm volatile("bar.sync %0, 128;" ::"r"(2 + eg) : "memory");
                    if (elected) {
                        // destinations in an order that rotates with the pair and the step, so that the CTAs running
                        // together do not all store to the same peer (the same NVLink path) at the same moment
                        const int n_dst = dst->count;
                        int d = n_dst > 1 ? static_cast<int>((pair + step) % static_cast<uint32_t>(n_dst)) : 0;
                        for (int k = 0; k < n_dst; ++k) {
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                                             reinterpret_cast<uint64_t>(&dst->tmap_c[d])),
                                         "r"(col0), "r"(row0), "r"(buf)
                                         : "memory");
                            if (++d == n_dst) d = 0;
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    // Pace the group's stores: issued back to back right after a tile ends (by every CTA of the grid at
                    // about the same moment) they double the latency of the loads that refill the ring just then.
                    if (i + 1 < kSteps) __nanosleep(static_cast<unsigned>(w.k_blocks) * kTc3StorePauseNsPerStage);
                } else {
                    // C cannot be described to the TMA unit (pitch or base not 16-byte aligned): 128-byte row pieces
                    const int col = col0 + static_cast<int>(colp);
                    if (col < N) {
                        if constexpr (kBf16) {
                            uint16_t* out = reinterpret_cast<uint16_t*>(C) + static_cast<size_t>(row0) * ldc + col;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (row0 + j < M) out[static_cast<size_t>(j) * ldc] = static_cast<uint16_t>(r[i][j]);
                        } else {
                            int32_t* out = C + static_cast<size_t>(row0) * ldc + col;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (row0 + j < M) out[static_cast<size_t>(j) * ldc] = static_cast<int32_t>(r[i][j]) >> 6;
                        }
                    }
                }
            }
        }
        if (elected) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // nothing in flight when the CTA leaves
    }

    __syncwarp();
    if (*abort_flag && lane == 0 && status) atomicMax(status, kStatusTimeout);
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair<512>(tmem_base);
    }
}

}  // namespace tb200
