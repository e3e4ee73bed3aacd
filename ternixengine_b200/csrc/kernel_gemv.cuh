// Decode-regime kernel (M <= 16): memory-bound GEMV / skinny GEMM over the packed weights.
//
// Data path.  The packed K x (N/4) matrix is read exactly once, by TMA, in boxes of
// (4*WORDS bytes) x (KT k-rows) = 4 KB that land in a ring of shared-memory stages; one producer
// lane keeps the whole ring in flight, which is what covers the HBM latency (a CTA has tens of
// KB outstanding without spending registers on it).  No dequantised copy of W ever exists in
// global memory: fields are decoded in registers.
//
// Decode.  A thread takes the same 32-bit word (16 columns) from four consecutive k-rows and
// byte-transposes the four words with 8 PRMTs, so that every word now holds one packed byte
// from each of the four k's.  For field j, (T << (6-2j)) & 0xC0C0C0C0 leaves each byte equal
// to 0x00 / 0x40 / 0xC0 = 0 / +64 / -64 as int8: the top two bits of the byte ARE the
// sign-extended 2-bit code.  One dp4a against the four matching activation bytes then adds
// 64 * sum_k a_k w_k.  The final arithmetic shift by 6 is exact.  No branch on zero.
// Bound: 64 * 128 * K < 2^31, i.e. K < 262144 (checked by the host).
//
// Reduction.  Lanes own columns; the k-groups are spread over the 8 consumer warps, over the
// CTAs of a thread-block cluster (split-K along cluster rank) and reduced first with
// shared-memory integer adds, then across the cluster through distributed shared memory.
// Integer adds are associative, so any order gives the reference's bits.  No global scratch,
// no global atomics, C is written once.
#pragma once
#include <cuda.h>
#include <cstdint>
#include "ptx_sm100.cuh"

namespace tb200 {

constexpr int kGemvConsumerWarps = 8;
constexpr int kGemvThreads = (kGemvConsumerWarps + 1) * 32;   // + one producer warp
constexpr int kGemvStageBytes = 4096;
constexpr int kGemvStages = 16;
constexpr int kGemvMaxASlice = 32768;                         // bytes of activations staged per CTA

template <int WORDS>
struct GemvGeom {
    static constexpr int kGroupsPerWarp = 32 / WORDS;                              // 4-row k-groups per warp
    static constexpr int kStageRows = kGemvConsumerWarps * kGroupsPerWarp * 4;     // 32 or 64
    static constexpr int kCols = WORDS * 16;                                       // output columns per CTA
    static_assert(kStageRows * WORDS * 4 == kGemvStageBytes, "stage is 4 KB");
};

template <int MR, int WORDS>
constexpr size_t gemv_smem_bytes(int krange) {
    return 128 /*alignment slack*/ + size_t(kGemvStages) * kGemvStageBytes + size_t(MR) * krange +
           size_t(MR) * 16 * (WORDS + 1) * 4 + 2 * kGemvStages * 8 + 16;
}

template <int MR, int WORDS>
__global__ void __launch_bounds__(kGemvThreads)
ternary_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const int8_t* __restrict__ A,
                    int32_t* __restrict__ C, int M, int K, int N, long long ldc, int krange, int a_words_ok,
                    int32_t* __restrict__ status) {
    using G = GemvGeom<WORDS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t* stages = base;
    int8_t* a_s = reinterpret_cast<int8_t*>(base + kGemvStages * kGemvStageBytes);          // [MR][krange]
    int32_t* part = reinterpret_cast<int32_t*>(a_s + MR * krange);                          // [MR][16][WORDS+1]
    uint64_t* full = reinterpret_cast<uint64_t*>(part + MR * 16 * (WORDS + 1));
    uint64_t* empty = full + kGemvStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kGemvStages);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t nrank = cluster_nctarank();
    const int n_chunk = blockIdx.x / nrank;
    const int row0 = blockIdx.y * MR;

    const int k_begin = rank * krange;
    int k_len = K - k_begin;
    if (k_len > krange) k_len = krange;
    if (k_len < 0) k_len = 0;
    const int ntiles = (k_len + G::kStageRows - 1) / G::kStageRows;

    if (tid == 0) {
        for (int s = 0; s < kGemvStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kGemvConsumerWarps);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    for (int i = tid; i < MR * 16 * (WORDS + 1); i += kGemvThreads) part[i] = 0;
    __syncthreads();

    if (warp == kGemvConsumerWarps) {
        // ------------------------------------------------------------ producer: one lane drives TMA
        if (lane == 0) {
            tma_prefetch_desc(&tmap_w);
            int issued = 0;
            for (int t = 0; t < ntiles; ++t) {
                const int s = t % kGemvStages;
                if (t >= kGemvStages && !mbar_wait(&empty[s], ((t / kGemvStages) & 1) ^ 1, abort_flag)) break;
                mbar_arrive_expect_tx(&full[s], kGemvStageBytes);
                tma_load_2d(stages + s * kGemvStageBytes, &tmap_w, n_chunk * WORDS * 4, k_begin + t * G::kStageRows,
                            &full[s]);
                issued = t + 1;
            }
            if (*abort_flag) {
                // Teardown after a timeout: let the copies already issued land before the CTA can exit.
                const int first = issued > kGemvStages ? issued - kGemvStages : 0;
                for (int t = first; t < issued; ++t) {
                    const int s = t % kGemvStages;
                    const uint32_t ph = (t / kGemvStages) & 1;
                    mbar_drain(&full[s], ph);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ consumers
        // stage the activation slice [MR][ntiles*kStageRows], zero beyond K and beyond M
        const int a_len = ntiles * G::kStageRows;
        if (a_words_ok) {
            for (int i = tid; i < MR * (a_len >> 2); i += kGemvConsumerWarps * 32) {
                const int r = i / (a_len >> 2), kk = (i % (a_len >> 2)) * 4;
                int v = 0;
                if (row0 + r < M && k_begin + kk < K)   // K % 4 == 0 here, so a word is all-in or all-out
                    v = *reinterpret_cast<const int*>(A + static_cast<size_t>(row0 + r) * K + k_begin + kk);
                *reinterpret_cast<int*>(a_s + r * krange + kk) = v;
            }
        } else {
            for (int i = tid; i < MR * a_len; i += kGemvConsumerWarps * 32) {
                const int r = i / a_len, kk = i % a_len;
                int8_t v = 0;
                if (row0 + r < M && k_begin + kk < K) v = A[static_cast<size_t>(row0 + r) * K + k_begin + kk];
                a_s[r * krange + kk] = v;
            }
        }
        // consumer-only barrier (the producer warp is busy issuing copies)
        asm volatile("bar.sync 1, %0;" ::"n"(kGemvConsumerWarps * 32) : "memory");

        int32_t acc[MR][16];
#pragma unroll
        for (int r = 0; r < MR; ++r)
#pragma unroll
            for (int c = 0; c < 16; ++c) acc[r][c] = 0;

        const int word = lane % WORDS;
        const int kg = warp * G::kGroupsPerWarp + lane / WORDS;   // 4-row group inside a stage
        // explicit shared-window addresses: pointers derived from the dynamic-shared base are generic to the compiler
        const uint32_t stages_sa = smem_u32(stages), a_sa = smem_u32(a_s), part_sa = smem_u32(part);
        const uint32_t w_off = ((kg * 4) * WORDS + word) * 4;

        for (int t = 0; t < ntiles; ++t) {
            const int s = t % kGemvStages;
            if (!mbar_wait(&full[s], (t / kGemvStages) & 1, abort_flag)) break;
            const uint32_t st = stages_sa + s * kGemvStageBytes + w_off;
            const uint32_t w0 = lds_u32(st);
            const uint32_t w1 = lds_u32(st + WORDS * 4);
            const uint32_t w2 = lds_u32(st + 2 * WORDS * 4);
            const uint32_t w3 = lds_u32(st + 3 * WORDS * 4);
            int a4[MR];
#pragma unroll
            for (int r = 0; r < MR; ++r)
                a4[r] = static_cast<int>(lds_u32(a_sa + r * krange + t * G::kStageRows + kg * 4));
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);   // the words are in registers: release the stage early

            // 4x4 byte transpose: T[b] = { w0.byte b, w1.byte b, w2.byte b, w3.byte b }
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
                    const int x = static_cast<int>((T[b] << (6 - 2 * j)) & 0xC0C0C0C0u);   // bytes: 0, +64, -64
#pragma unroll
                    for (int r = 0; r < MR; ++r) acc[r][4 * b + j] = __dp4a(x, a4[r], acc[r][4 * b + j]);
                }
        }

        // reduce over the k-groups held by different warps (and half-warps): shared-memory integer adds
#pragma unroll
        for (int r = 0; r < MR; ++r)
#pragma unroll
            for (int c = 0; c < 16; ++c) red_shared_add(part_sa + ((r * 16 + c) * (WORDS + 1) + word) * 4, acc[r][c]);
    }

    __syncwarp();
    if (tid == 0 && *abort_flag && status) atomicMax(status, kStatusTimeout);

    // ---------------------------------------------------------------- split-K reduce across the cluster
    cluster_sync_all();
    {
        const int total = MR * G::kCols;
        const int per_rank = (total + nrank - 1) / nrank;
        const int lo = rank * per_rank;
        const int hi = lo + per_rank < total ? lo + per_rank : total;
        const uint32_t part_addr = smem_u32(part);
        for (int i = lo + tid; i < hi; i += kGemvThreads) {
            const int r = i / G::kCols, col = i % G::kCols;
            const uint32_t off = static_cast<uint32_t>(((r * 16 + (col & 15)) * (WORDS + 1) + (col >> 4)) * 4);
            // all remote loads are issued before any is used (cluster size is at most 8)
            int32_t v[8];
#pragma unroll
            for (uint32_t p = 0; p < 8; ++p) {
                v[p] = 0;
                if (p < nrank)
                    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v[p]) : "r"(dsmem_map(part_addr + off, p)));
            }
            int32_t sum = 0;
#pragma unroll
            for (uint32_t p = 0; p < 8; ++p) sum += v[p];
            const int grow = row0 + r, gcol = n_chunk * G::kCols + col;
            if (grow < M && gcol < N) C[static_cast<size_t>(grow) * ldc + gcol] = sum >> 6;
        }
    }
    cluster_sync_all();   // nobody leaves while a peer may still read its shared memory
}

}  // namespace tb200
