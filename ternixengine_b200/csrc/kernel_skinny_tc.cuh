// Batched-decode kernel on the tcgen05 tensor core: up to 128 rows of activations against a stream of packed weights.
//
// As in the paired prefill kernel the product is computed transposed, C^T[n][m] = sum_k W[k][n] * A[m][k]: the
// weights are the A operand of tcgen05.mma and live in TENSOR MEMORY (row = weight column = lane, four K-bytes per
// 32-bit column), the activations are the B operand, straight from TMA in the K-major 128-byte-swizzle layout, with
// the batch as the instruction's N (16, 32, 64 or 128).  Nothing expanded is ever written to shared memory.
//
// Where it pays, and what bounds it.  The tensor pipe is far from busy here (an N = 32 MMA occupies it for about 16
// cycles; ncu shows the pipe 20 % active): what bounds the kernel is the instruction stream of the threads that ISSUE
// the MMAs.  Measured on B200 with one issuing thread: a tcgen05.mma with N <= 64 leaves the thread every 60-90
// cycles whatever its N (N = 128: 64 cycles, N = 256: 128 cycles, the pipe's own time), a tcgen05.commit costs it
// about 180 cycles, a wait on an mbarrier that has long completed 60-150; a second issuing thread in another warp
// runs at the same rate beside the first.  With one issuer per 128-column block (two threads) a stage of 8 KB of
// packed weights took about 960 cycles, 2.4 TB/s over the GPU whatever the row count; with the stages dealt
// alternately to two such pairs (four threads, accumulators of their own, added in the epilogue) 640 cycles,
// 3.3 TB/s of packed weights.  The warp-level mma.sync kernel (kernel_decode_mma.cuh) streams 5.5 TB/s up to 8 rows and
// 3.8 TB/s up to 16, but needs one pass per 16 rows; from 17 rows up this kernel is the faster one (210 BitNet-2B
// projections: 156 us against 288 us at 32 rows, 200 us against 538 us at 64 rows), and the dispatch uses it
// there.  Group members with 65 to 128 rows run here as well (247 us at 128 rows; the paired prefill kernel pads
// them to 256-row tiles, 367 us); a single product of that size is faster on the prefill kernel.
//
// From packed bytes to the operand in 17 instructions per 1024 weights and warp:
//   * a stage is 128 k-rows x 64 packed bytes (256 weight columns), TMA with the 64-byte swizzle;
//   * ldmatrix.m16n16.x2.trans.b8 leaves, in lane (c, t) = (lane / 4, lane % 4), the bytes of k-rows 4t..4t+3 of packed
//     byte column c of a 16-byte chunk -- exactly what lane (c, t) has to supply to tcgen05.st.16x128b for operand
//     row c, columns t.  So the operand rows (tensor-memory lanes) are simply numbered the way the load delivers
//     them: lane l of a 32-lane quarter holds weight column 4 (l % 8) + l / 8 of the quarter's 32, and no data moves
//     between lanes at all.  The epilogue, which reads the accumulator lane by lane, undoes the numbering for free;
//   * a field is decoded without sign extension: (T << (6 - 2f)) & 0xC0C0C0C0 leaves every byte as 0x00, 0x40 or
//     0xC0, i.e. 0, +64, -64 as int8 (the two top bits of a byte ARE the sign-extended code).  The accumulators hold
//     64 * sum; the final arithmetic shift by 6 is exact.  Bound 64 * 128 * K < 2^31, K <= 262143.
//
// Tensor memory (512 columns): accumulators [buffer][issuer pair][128-column block] x NB columns (two buffers for
// NB <= 32, one otherwise; two issuer pairs for NB <= 64, one for NB = 128), then a ring of operand stages of
// 2 blocks x 32 columns each (6 stages for NB = 16, 4 otherwise).  Shared memory: a ring of 16 (8 for NB = 128)
// packed-weight stages (8 KB each: what is in flight from HBM) and a ring of 16 / 16 / 8 / 6 activation stages
// (NB rows x 128 bytes).  Each 128-column block has its own accumulator barriers, and the epilogue reads a whole
// batch of up to 64 rows into registers and releases the accumulator before it stores any of them, so with a single
// buffer the issuers wait for a few tcgen05.ld only.
//
// Roles (19 warps for NB <= 64, 17 for NB = 128; the last one forwards "activations landed" to the `ready` barriers,
// so that an issuer waits on one barrier per stage): 0 weight producer; 1 and 3 MMA issuers of the even stages (one per
// 128-column block), 16 and 17 those of the odd stages (NB <= 64; stages are counted over the CTA's whole walk);
// 2 activation producer; 4-11 expanders (lane quarter = warp % 4, the two warps of a quarter take the stages in
// turn); 12-15 epilogue (lane quarter = warp % 4).
//
// Work.  Grouped launches walk a host-built list of (problem, 256-column block) items over the whole of K.  One
// problem alone runs as whole-K items too whenever they occupy the machine reasonably (items of 128 columns, half a
// weight box each, when there are at most as many as SMs; items of 256 columns when those fit in one round): all
// CTAs then walk the weight rows together, which is the access pattern DRAM likes, and nothing has to be exchanged.
// Only with more blocks than SMs the (block, stage) units are dealt out as ONE contiguous range per CTA, a block
// being shared by CTAs with neighbouring indices.  Their partial sums travel through C itself: the CTA with the
// lowest stages stores its raw partial tile into C and raises a flag, the next one adds its own on top, and the CTA
// that holds the last stage shifts and stores the result.  Each CTA walks its range from the top, so the part it
// shares with its successor is done first and nobody ever waits for a CTA with a higher index; every flag wait is
// bounded like the barrier waits.  No atomics, no zeroing of C, no scratch memory beyond one flag per CTA; flags
// carry a per-launch epoch, so they never need clearing.
#pragma once
#include <cuda.h>
#include <cstdint>
#include "kernel_gemm_tc3.cuh"
#include "ptx_sm100.cuh"

namespace tb200 {

constexpr int kSkBK = 128;                        // k-rows per stage
constexpr int kSkItemCols = 256;                  // weight columns per item: two MMA blocks of 128
constexpr int kSkWpRowBytes = kSkItemCols / 4;    // 64
constexpr int kSkWpBytes = kSkBK * kSkWpRowBytes; // 8192
constexpr int kSkBaseWarps = 16;                  // + two warps per additional pair of MMA issuers (SkGeom::kThreads)
constexpr int kSkFirstExpandWarp = 4, kSkFirstEpilogueWarp = 12;
constexpr uint32_t kSkStageCols = 64;              // operand stage: 2 blocks x 128 K-bytes = 2 x 32 columns
constexpr int kSkMaxCtas = 256;                   // flags per launch slot

template <int NB>
struct SkGeom {
    static_assert(NB == 16 || NB == 32 || NB == 64 || NB == 128, "batch rows per instruction");
    static constexpr int kActBytes = NB * 128;                   // one box: NB rows x 128 K-bytes, 128-byte swizzle
    // Four MMA issuers for NB <= 64: the stages of a segment go alternately to two pairs of issuers, each pair with
    // accumulators of its own, and the epilogue adds the two.  (One thread issues a small-N MMA every 60-90 cycles and
    // spends 180 on a commit, far more than the tensor pipe needs to execute them; two threads per block double that.)
    // (Giving the second pair half of the activation rows instead, for NB = 64, was measured: every issuer then meets
    // every stage, and the stage rate is that of two issuers again.)
    // (Four pairs for NB <= 32, which leaves room for one accumulator buffer only, were measured as well: 170-176 us
    // against 158 us for the 210 projections of the header's example.)
    static constexpr int kParts = NB <= 64 ? 2 : 1;              // pairs of issuers; stage i goes to pair i % kParts
    static constexpr bool kSplitK = kParts > 1;
    static constexpr int kAccBufs = NB <= 32 ? 2 : 1;            // accumulator buffers per 128-column block and part
    static constexpr int kTStages = NB == 16 ? 6 : 4;            // operand ring (tensor memory)
    static constexpr int kForwardWarp = kSkBaseWarps + 2 * (kParts - 1);     // the warp after the last issuer
    static constexpr int kThreads = (kForwardWarp + 1) * 32;                 // 19 or 17 warps
    static constexpr int kWStages = NB == 128 ? 8 : 16;          // packed-weight ring (shared memory): what is in flight from HBM
    static constexpr int kAStages = NB == 128 ? 6 : NB == 64 ? 8 : 16;   // activation ring (shared memory)
    static constexpr uint32_t kRingCol = 2 * kParts * kAccBufs * NB;   // after the accumulators: [buffer][part][block] x NB columns
    static_assert(kRingCol + kTStages * kSkStageCols <= 512, "tensor memory: 512 columns");
    static constexpr size_t kSmemBytes = 1024 + size_t(kWStages) * kSkWpBytes + size_t(kAStages) * kActBytes + 768;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory: 227 KB per CTA");
    // D = s32, A = B = s8, both K-major, N = NB, M = 128
    static constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(NB >> 3) << 17) | (uint32_t(128 >> 4) << 24);
};

struct alignas(64) SkProblem {
    CUtensorMap tmap_w;        // packed W [K][N/4] bytes, box 64 B x 128 rows, 64-byte swizzle
    CUtensorMap tmap_a;        // A [M][K] bytes, box 128 B x NB rows, 128-byte swizzle
    int32_t* C;
    long long ldc;
    int M, K, N, pad;
};
struct SkItem {
    int problem, block;
};
// One problem per launch.  Units are (column block, stage) pairs, CTA i takes the contiguous range
// [i U / G, (i + 1) U / G).  `half_items`: a unit's column block is 128 columns wide (one half of a 256-column weight
// box) and a CTA owns whole blocks -- the form for problems with few columns, where whole-K items of 128 columns
// occupy more SMs than items of 256.  `whole_blocks`: ranges are cut at block boundaries, so no CTA shares a block.
struct SkSingle {
    int blocks, stages, whole_blocks, half_items;
};

// D[tmem] (+)= A[tmem] x B[smem desc], int8 x int8 -> int32, one CTA; the shared-memory descriptor is given as two
// 32-bit halves (no 64-bit arithmetic in the issue loop).
__device__ __forceinline__ void tc_mma_i8_tmem_a_lohi(uint32_t tmem_d, uint32_t tmem_a, uint32_t desc_lo, uint32_t desc_hi,
                                                      uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], db, %4, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32_x16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 16 lanes x 32 columns (128 K-bytes of 16 operand rows) in one instruction: registers 2i, 2i+1 are rows lane/4 and
// lane/4 + 8 at column 4i + lane%4.
__device__ __forceinline__ void tmem_st_16x128_x8(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait for another CTA's flag to show this launch's epoch.
__device__ __forceinline__ bool flag_wait(const int* flag, int epoch, volatile int* abort_flag) {
    uint64_t t0 = 0;
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (ld_acquire_gpu(flag) == epoch) return true;
        __nanosleep(64);
        if ((spin & 63u) == 63u) {
            if (*abort_flag) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) break;
        }
    }
    *abort_flag = 1;
    return false;
}

// The segments of one CTA: runs of stages [s0, s1) of one 256-column weight box, of which the 128-column blocks
// [h0, h1) are computed.  Every warp role constructs its own walker and sees the same sequence.
template <bool kGrouped>
struct SkWalk {
    const SkProblem* p;
    int block, s0, s1, h0, h1;
    bool add_prev;             // stages below s0 belong to the CTA before this one: add what it left in C
    bool last;                 // holds the block's last stage: shift and store; otherwise store raw and raise the flag
    // single problem
    int lo, hi, stages, half_items;
    // group
    const SkProblem* probs;
    const SkItem* items;
    int idx, end;

    __device__ __forceinline__ bool next() {
        if constexpr (kGrouped) {
            if (idx >= end) return false;
            const SkItem it = items[idx++];
            p = probs + it.problem;
            block = it.block;
            s0 = 0;
            s1 = (p->K + kSkBK - 1) / kSkBK;
            h0 = 0;
            h1 = (block * kSkItemCols + 128 < p->N) ? 2 : 1;      // a ragged last box may hold one block only
            add_prev = false;
            last = true;
            return true;
        } else {
            if (hi <= lo) return false;
            const int b = (hi - 1) / stages;
            const int first = max(lo, b * stages);
            s0 = first - b * stages;
            s1 = hi - b * stages;
            add_prev = s0 > 0;
            last = s1 == stages;
            hi = first;
            if (half_items) { block = b >> 1; h0 = b & 1; h1 = h0 + 1; }
            else { block = b; h0 = 0; h1 = (block * kSkItemCols + 128 < p->N) ? 2 : 1; }
            return true;
        }
    }
};

template <int NB, bool kGrouped>
__global__ void __launch_bounds__(SkGeom<NB>::kThreads, 1)
ternary_skinny_tc_kernel(const __grid_constant__ SkProblem single, const SkSingle sg,
                         const SkProblem* __restrict__ probs, const SkItem* __restrict__ items,
                         const int* __restrict__ cta_first, int* __restrict__ flags, int epoch,
                         int32_t* __restrict__ status) {
    using G = SkGeom<NB>;
    constexpr int TS = G::kTStages, AS = G::kAStages, WS = G::kWStages, BUFS = G::kAccBufs;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sW = base;                                              // [WStages][128 k][64]   64-byte swizzle
    uint8_t* sAct = sW + WS * kSkWpBytes;                    // [AS][NB rows][128 k]   128-byte swizzle
    uint64_t* bars = reinterpret_cast<uint64_t*>(sAct + AS * G::kActBytes);
    uint64_t* w_full = bars;                       // a packed-weight stage has landed
    uint64_t* w_empty = w_full + WS;       // the four quarters have read it
    uint64_t* a_full = w_empty + WS;       // an activation stage has landed
    uint64_t* a_empty = a_full + AS;               // the MMAs that read an activation stage have retired
    uint64_t* ready = a_empty + AS;                // the four quarters have written an operand stage
    uint64_t* t_free = ready + TS;                 // the MMAs that read an operand stage have retired
    uint64_t* acc_full = t_free + TS;              // [buffer][block]: that block's MMAs of a segment have retired
    uint64_t* acc_empty = acc_full + 4;            // [buffer][block]: the epilogue has read that accumulator
    uint64_t* drain = acc_empty + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* epi_count = reinterpret_cast<int*>(tmem_slot + 2);    // epilogue warps done with the one partial tile a CTA writes

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto make_walk = [&]() {
        SkWalk<kGrouped> w{};
        if constexpr (kGrouped) {
            w.probs = probs; w.items = items;
            w.idx = cta_first[blockIdx.x]; w.end = cta_first[blockIdx.x + 1];
        } else {
            w.p = &single;
            w.stages = sg.stages;
            w.half_items = sg.half_items;
            const long long g = gridDim.x, i = blockIdx.x;
            if (sg.whole_blocks) {
                w.lo = static_cast<int>(i * sg.blocks / g) * sg.stages;
                w.hi = static_cast<int>((i + 1) * sg.blocks / g) * sg.stages;
            } else {
                const long long units = static_cast<long long>(sg.blocks) * sg.stages;
                w.lo = static_cast<int>(i * units / g);
                w.hi = static_cast<int>((i + 1) * units / g);
            }
        }
        return w;
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < WS; ++s) {
            mbar_init(&w_full[s], 1);
            mbar_init(&w_empty[s], 4);
        }
        for (int s = 0; s < AS; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_empty[s], 1);
        }
        for (int s = 0; s < TS; ++s) {
            mbar_init(&ready[s], 5);                   // the four quarters and the activation forwarder
            mbar_init(&t_free[s], 2);                  // the two issuers that read the stage
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(&acc_full[b], G::kParts);      // one commit per issuer of the block
            mbar_init(&acc_empty[b], 4);
        }
        mbar_init(drain, 2 * G::kParts);
        *abort_flag = 0;
        *epi_count = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc<512>(tmem_slot);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ================================================================ packed weights: HBM -> shared memory
        if (lane == 0) {
            if constexpr (!kGrouped) tma_prefetch_desc(&single.tmap_w);
            uint32_t it = 0;
            bool ok = true;
            SkWalk<kGrouped> w = make_walk();
            while (ok && w.next()) {
                const int x = w.block * kSkWpRowBytes;
                for (int s = w.s0; s < w.s1; ++s, ++it) {
                    const uint32_t sl = it % WS;
                    if (!mbar_wait_backoff(&w_empty[sl], ((it / WS) & 1) ^ 1, abort_flag, 32)) { ok = false; break; }
                    mbar_arrive_expect_tx(&w_full[sl], kSkWpBytes);
                    tma_load_2d(sW + sl * kSkWpBytes, &w.p->tmap_w, x, s * kSkBK, &w_full[sl]);
                }
            }
            if (!ok) {
                const uint32_t first = it > WS ? it - WS : 0;
                for (uint32_t j = first; j < it; ++j) mbar_drain(&w_full[j % WS], (j / WS) & 1);
            }
        }
    } else if (warp == 2) {
        // ================================================================ activations: L2 -> shared memory
        if (lane == 0) {
            if constexpr (!kGrouped) tma_prefetch_desc(&single.tmap_a);
            uint32_t it = 0;
            bool ok = true;
            SkWalk<kGrouped> w = make_walk();
            while (ok && w.next()) {
                for (int s = w.s0; s < w.s1; ++s, ++it) {
                    const uint32_t sl = it % AS;
                    if (!mbar_wait_backoff(&a_empty[sl], ((it / AS) & 1) ^ 1, abort_flag, 32)) { ok = false; break; }
                    mbar_arrive_expect_tx(&a_full[sl], G::kActBytes);
                    tma_load_2d(sAct + sl * G::kActBytes, &w.p->tmap_a, s * kSkBK, 0, &a_full[sl]);
                }
            }
            if (!ok) {
                const uint32_t first = it > AS ? it - AS : 0;
                for (uint32_t j = first; j < it; ++j) mbar_drain(&a_full[j % AS], (j / AS) & 1);
            }
        }
    } else if (warp == 1 || warp == 3 || (warp >= 16 && 1 + ((warp - 16) >> 1) < G::kParts)) {
        // ================================================================ MMA issuers
        // One thread per 128-column block of the box and, for NB <= 64, per parity of the stage count: warps 1 and 3
        // take the even stages (counted over the CTA's whole walk), warps 16 and 17 the odd ones, each into accumulators
        // of its own, so the order between issuers never matters.  A thread's instruction stream -- waits, descriptor
        // arithmetic, 60-90 cycles per MMA, 180 per commit -- is what bounds the stage rate of this kernel, which is why
        // it is split four ways and kept short: ring positions and the descriptor's low word advance by additions.
        if (lane == 0) {
            const uint32_t hsel = warp < 16 ? (warp == 3 ? 1u : 0u) : static_cast<uint32_t>(warp & 1);
            const uint32_t part = warp < 16 ? 0u : 1u + (static_cast<uint32_t>(warp - 16) >> 1);
            uint32_t it = 0;
            const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);          // stride 1024 B, version 1, 128-byte swizzle
            const uint32_t desc_lo0 = ((smem_u32(sAct) & 0x3FFFFu) >> 4) | (1u << 16);  // start address, leading offset 16 B
            uint32_t sl = 0, ph_t = 0, al = 0, ph_a = 0, lt = 0;
            bool ok = true;
            SkWalk<kGrouped> w = make_walk();
            for (; ok && w.next(); ++lt) {
                // each issuer owns the accumulators of its block: with one buffer per block (NB = 128) the issuer of
                // block 0 can start the next segment while the epilogue still reads block 1
                const uint32_t ab = lt % BUFS, use = lt / BUFS;
                if (!mbar_wait(&acc_empty[ab * 2 + hsel], (use & 1) ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const bool mine = hsel >= static_cast<uint32_t>(w.h0) && hsel < static_cast<uint32_t>(w.h1);
                const uint32_t d = tmem_base + ((ab * G::kParts + part) * 2 + hsel) * NB;
                uint32_t acc = 0;
                for (int s = w.s0; s < w.s1; ++s, ++it) {
                    if (G::kSplitK && (it & (G::kParts - 1)) != part) {   // another pair's stage: only the ring positions move
                        if (++sl == TS) { sl = 0; ph_t ^= 1; }
                        if (++al == AS) { al = 0; ph_a ^= 1; }
                        continue;
                    }
                    // `ready` also says that the stage's activations have landed (the forwarder's arrival)
                    if (!mbar_wait(&ready[sl], ph_t, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    if (mine) {
                        const uint32_t a_col = tmem_base + G::kRingCol + sl * kSkStageCols + hsel * 32;
                        const uint32_t lo = desc_lo0 + al * (G::kActBytes >> 4);
#pragma unroll
                        for (int g = 0; g < kSkBK / 32; ++g) {
                            tc_mma_i8_tmem_a_lohi(d, a_col + 8 * g, lo + 2 * g, desc_hi, G::kIdesc, acc);
                            acc = 1;
                        }
                    }
                    tc_commit(&t_free[sl]);
                    if (++sl == TS) { sl = 0; ph_t ^= 1; }
                    if (++al == AS) { al = 0; ph_a ^= 1; }
                }
                if (ok) tc_commit(&acc_full[ab * 2 + hsel]);
            }
            tc_commit(drain);                      // both issuers: nothing of theirs is in flight when tensor memory is freed
            mbar_wait(drain, 0, abort_flag);
        }
    } else if (warp == G::kForwardWarp) {
        // ================================================================ activation forwarder
        // Passes "the activations of stage i have landed" on to the stage's `ready` barrier, so that an issuer, whose
        // instruction stream is what bounds the kernel, waits on one barrier per stage instead of two.  Like an
        // expander it may arrive for a stage only when the operand slot's previous use has retired.
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            SkWalk<kGrouped> w = make_walk();
            while (ok && w.next()) {
                for (int s = w.s0; s < w.s1; ++s, ++it) {
                    const uint32_t st = it % TS, al = it % AS;
                    if (!mbar_wait_backoff(&t_free[st], ((it / TS) & 1) ^ 1, abort_flag, 32) ||
                        !mbar_wait_backoff(&a_full[al], (it / AS) & 1, abort_flag, 32)) { ok = false; break; }
                    mbar_arrive(&ready[st]);
                }
            }
        }
    } else if (warp >= kSkFirstExpandWarp && warp < kSkFirstEpilogueWarp) {
        // ================================================================ expanders: packed bytes -> operand rows in tensor memory
        // The warp of lane quarter q writes operand rows 32q..32q+31 of both 128-column blocks: packed byte columns
        // 32h + 8q .. +7 of a row, i.e. half (q & 1) of 16-byte chunk 2h + q / 2.
        const uint32_t q = warp & 3;
        const uint32_t turn = (warp - kSkFirstExpandWarp) >> 2;
        const uint32_t r_in = lane & 15;
        // ldmatrix.x2: matrix 0 = k-rows 0-15, matrix 1 = k-rows 16-31 of a 32-deep group; 64-byte rows, 64-byte swizzle
        // (16-byte chunk ^= (row / 2) % 4)
        const uint32_t row_off = (lane >> 4) * (16 * kSkWpRowBytes) + r_in * kSkWpRowBytes;
        const uint32_t swz = (r_in >> 1) & 3;
        const uint32_t off_h[2] = {row_off + ((((q >> 1) + 0) ^ swz) << 4), row_off + ((((q >> 1) + 2) ^ swz) << 4)};
        const uint32_t w_sa = smem_u32(sW);
        const uint32_t t_lane = (q * 32) << 16;
        const bool odd = (q & 1) != 0;
        uint32_t it = 0;
        bool ok = true;
        SkWalk<kGrouped> w = make_walk();
        while (ok && w.next()) {
            for (int s = w.s0; s < w.s1; ++s, ++it) {
                if ((it & 1) != turn) continue;
                const uint32_t sw = it % WS, st = it % TS;
                if (!mbar_wait_backoff(&w_full[sw], (it / WS) & 1, abort_flag, 32)) { ok = false; break; }
                const uint32_t wp = w_sa + sw * kSkWpBytes;
                // all loads of the stage first, so that their latencies overlap
                uint32_t m[2][kSkBK / 32][4];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h < w.h0 || h >= w.h1) continue;
#pragma unroll
                    for (int g = 0; g < kSkBK / 32; ++g) ldmatrix_x2_trans_b8_nc(m[h][g], wp + g * (32 * kSkWpRowBytes) + off_h[h]);
                }
                if (!mbar_wait_backoff(&t_free[st], ((it / TS) & 1) ^ 1, abort_flag, 32)) { ok = false; break; }
                tc_fence_after_sync();
                // the MMAs of stage it - TS have retired, so its activation slot is free as well: one quarter passes that on
                // (an ordinary arrive is cheaper than a second tcgen05.commit per stage)
                if (q == 0 && lane == 0 && it >= static_cast<uint32_t>(TS)) mbar_arrive(&a_empty[(it - TS) % AS]);
                const uint32_t a_col = tmem_base + G::kRingCol + st * kSkStageCols + t_lane;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h < w.h0 || h >= w.h1) continue;
                    uint32_t lo[16], hi[16];
#pragma unroll
                    for (int g = 0; g < kSkBK / 32; ++g) {
                        const uint32_t X = odd ? m[h][g][1] : m[h][g][0], Y = odd ? m[h][g][3] : m[h][g][2];
                        lo[4 * g + 0] = decode_field_x64<0>(X); lo[4 * g + 1] = decode_field_x64<1>(X);
                        lo[4 * g + 2] = decode_field_x64<0>(Y); lo[4 * g + 3] = decode_field_x64<1>(Y);
                        hi[4 * g + 0] = decode_field_x64<2>(X); hi[4 * g + 1] = decode_field_x64<3>(X);
                        hi[4 * g + 2] = decode_field_x64<2>(Y); hi[4 * g + 3] = decode_field_x64<3>(Y);
                    }
                    tmem_st_16x128_x8(a_col + 32 * h, lo);
                    tmem_st_16x128_x8(a_col + 32 * h + (16u << 16), hi);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&w_empty[sw]);
                    mbar_arrive(&ready[st]);
                }
            }
        }
    } else if (warp >= kSkFirstEpilogueWarp && warp < kSkFirstEpilogueWarp + 4) {
        // ================================================================ epilogue
        // Thread = operand row = weight column; registers = batch rows.  Lane l of quarter q is weight column
        // 32q + 4 (l % 8) + l / 8 of its 128-column block.
        const uint32_t q = warp & 3;
        const int col_in_block = 32 * q + 4 * (lane & 7) + (lane >> 3);
        uint32_t lt = 0, it = 0;                   // it: stages before this segment (their parity says whose they were)
        bool ok = true;
        SkWalk<kGrouped> w = make_walk();
        for (; ok && w.next(); ++lt) {
            const uint32_t ab = lt % BUFS, use = lt / BUFS;
            const uint32_t n_stages = static_cast<uint32_t>(w.s1 - w.s0);
            // which issuer pairs had a stage of this segment (a pair without one left its accumulator untouched):
            // pair p took the stages i of the walk with i % kParts == p
            const uint32_t first_part = it & (G::kParts - 1);
            it += n_stages;
            const SkProblem* p = w.p;
            const int M = p->M, N = p->N;
            const long long ldc = p->ldc;
            if (w.add_prev && !flag_wait(flags + blockIdx.x - 1, epoch, abort_flag)) { ok = false; break; }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                // both issuers signal every segment, also for a block the segment does not compute
                if (!mbar_wait_backoff(&acc_full[ab * 2 + h], use & 1, abort_flag, 64)) { ok = false; break; }
                tc_fence_after_sync();
                if (h < w.h0 || h >= w.h1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[ab * 2 + h]);
                    continue;
                }
                const int col = w.block * kSkItemCols + h * 128 + col_in_block;
                int32_t* out = p->C + col;
                // A batch of up to 64 rows goes into registers (the two issuer pairs' accumulators added), and when the
                // last batch is there the accumulator is released, before any of its rows is stored: with one buffer per
                // block the issuers wait for exactly this.
                constexpr int kBatch = NB / 16 < 4 ? NB / 16 : 4;
#pragma unroll
                for (int c0 = 0; c0 < NB / 16; c0 += kBatch) {
                    uint32_t r[kBatch][16];
#pragma unroll
                    for (int c = 0; c < kBatch; ++c) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) r[c][j] = 0;
                    }
#pragma unroll
                    for (int part = 0; part < G::kParts; ++part) {
                        if (((static_cast<uint32_t>(part) - first_part) & (G::kParts - 1)) >= n_stages) continue;
#pragma unroll
                        for (int c = 0; c < kBatch; ++c) {
                            uint32_t r1[16];
                            tmem_ld_32x32_x16(tmem_base + ((q * 32) << 16) + ((ab * G::kParts + part) * 2 + h) * NB + 16 * (c0 + c), r1);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 16; ++j) r[c][j] += r1[j];
                        }
                    }
                    tmem_ld_wait();
                    if (c0 + kBatch >= NB / 16) {      // this block's accumulator has been read: its issuers may use it again
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[ab * 2 + h]);
                    }
                    if (col >= N) continue;
#pragma unroll
                    for (int c = 0; c < kBatch; ++c) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int row = 16 * (c0 + c) + j;
                            if (row < M) {
                                int32_t* dst = out + static_cast<size_t>(row) * ldc;
                                int32_t v = static_cast<int32_t>(r[c][j]);
                                if (w.add_prev) v += __ldcg(dst);
                                if (w.last) *dst = v >> 6;
                                else __stcg(dst, v);
                            }
                        }
                    }
                }
            }
            if (!ok) break;
            if (!w.last) {
                // raise this CTA's flag once all four epilogue warps have stored their part of the partial tile
                __threadfence();
                __syncwarp();
                if (lane == 0 && atomicAdd(epi_count, 1) == 3) {
                    __threadfence();
                    st_release_gpu(flags + blockIdx.x, epoch);
                }
            }
        }
    }

    __syncwarp();
    if (*abort_flag && lane == 0 && status) atomicMax(status, kStatusTimeout);
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<512>(tmem_base);
    }
}

}  // namespace tb200
