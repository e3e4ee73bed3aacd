// C ABI of the B200 ternary matrix product: shape checks, kernel choice, TMA descriptors, launches.
// Declared in include/ternix_b200.h.  No CPU fallback: device entry points need a GPU.
#include "ternix_b200.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <mutex>
#include <new>
#include <queue>
#include <vector>

#include "kernel_gemm_tc.cuh"
#include "kernel_gemm_tc2.cuh"
#include "kernel_gemm_tc3.cuh"
#include "kernel_gemv.cuh"
#include "kernel_decode_mma.cuh"
#include "kernel_gemv_group.cuh"
#include "kernel_generic.cuh"
#include "kernel_skinny_tc.cuh"

namespace {

thread_local int g_last_cuda_error = 0;
thread_local int g_last_launched = 0;      // TERNIX_B200_LAUNCHED_* of the calling thread's last single-product launch

int cuda_fail(cudaError_t e) {
    g_last_cuda_error = static_cast<int>(e);
    return TERNIX_B200_ERR_CUDA;
}
#define TB_CUDA(call)                                            \
    do {                                                         \
        cudaError_t e_ = (call);                                 \
        if (e_ != cudaSuccess) return cuda_fail(e_);             \
    } while (0)

// The scaled accumulators of the fast kernels hold 64 * sum; 64 * 128 * K must stay below 2^31.
constexpr int kMaxScaledK = 262143;

// ---------------------------------------------------------------- driver entry point for TMA maps
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q{};
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 2-D byte tensor [rows][row_bytes] with `pitch` bytes between rows; box = box_rows x box_bytes.
int make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t row_bytes, uint64_t rows, uint64_t pitch,
                 uint32_t box_bytes, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return cuda_fail(cudaErrorNotSupported);
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
    return TERNIX_B200_OK;
}

// 2-D tensor of 32-bit words [rows][row_words] with `pitch` bytes between rows; box = box_rows x box_words.
int make_tmap_2d_u32(CUtensorMap* out, const void* ptr, uint64_t row_words, uint64_t rows, uint64_t pitch,
                     uint32_t box_words, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return cuda_fail(cudaErrorNotSupported);
    const cuuint64_t dims[2] = {row_words, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_words, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
    return TERNIX_B200_OK;
}

// 2-D tensor of 16-bit elements [rows][row_elems] with `pitch` bytes between rows; box = box_rows x box_elems.
int make_tmap_2d_u16(CUtensorMap* out, const void* ptr, uint64_t row_elems, uint64_t rows, uint64_t pitch,
                     uint32_t box_elems, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return cuda_fail(cudaErrorNotSupported);
    const cuuint64_t dims[2] = {row_elems, rows};
    const cuuint64_t strides[1] = {pitch};
    const cuuint32_t box[2] = {box_elems, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cuda_fail(cudaErrorInvalidValue);
    return TERNIX_B200_OK;
}

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

constexpr int kMaxDevices = 64;

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    return dev;
}

// SM count of the current device (cached per device).
int sm_count() {
    static std::atomic<int> cache[kMaxDevices] = {};
    const int dev = current_device();
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cache[dev].store(v, std::memory_order_relaxed);
    return v;
}

// Opt-in to more than 48 KB of dynamic shared memory.  The attribute belongs to the (kernel, device) pair, so it is
// set once per device, with that device current; the state is per kernel because the kernel is a template argument.
template <auto Kern>
int ensure_smem_attr(size_t bytes) {
    static std::mutex mu;
    static unsigned char done[kMaxDevices] = {};
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(mu);
    if (done[dev]) return TERNIX_B200_OK;
    const cudaError_t e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e != cudaSuccess) return cuda_fail(e);
    done[dev] = 1;
    return TERNIX_B200_OK;
}

// ---------------------------------------------------------------- tuning options
// Defaults are the measured best; the tests force the other paths.  Read once from the environment
// (TERNIX_B200_<NAME>) when the library is first used and changed afterwards only through ternix_b200_set_option;
// the launch path reads plain fields.
struct Options {
    int tc_tile_rows = 0;              // activation rows per pair instruction of the tensor-memory GEMM: 0 = by shape, 128, 256
    int tc3 = 1;                       // 0: the kernels that expand weights into shared memory instead of tensor memory
    int tc_bn = 0;                     // 128 | 256: single-CTA tiles of that width; 2: paired CTAs; 0: by shape
    int tc_ksplit = 1;                 // 0: no K split in the single-CTA kernel
    int gemv_words = 0, gemv_split = 0;   // plan of the one-row kernel ("words,ksplit"), 0 = heuristic
    int group_words = 0;               // 16 | 32: item width of the grouped one-row kernel, 0 = by membership
    int gemv_pdl = -1;                 // decode batches as programmatic dependents: 0 never, 1 always, -1 for short launches
    int mma_lo = 2, mma_hi = 64;       // rows served by the mma.sync decode kernel when skinny_hi < rows
    int mma_slices = 0;                // K slices of a single mma.sync decode problem, 0 = cost model
    int mma_cluster = -1;              // 0 | 2 | 4 | 8: cluster form of the same, -1 = largest that fits
    int skinny_lo = 33, skinny_hi = 64; // rows of a single product served by the tensor-memory decode kernel (0,0 = never)
    int skinny_group_lo = 17, skinny_group_hi = 128;   // the same for members of a problem group (one launch serves many products there)
    int skinny_split = 1;              // 0: never share a block between CTAs; 1: only when blocks outnumber SMs; 2: whenever it evens the load
    int host_slab = -1;                // slab extent of the pipelined host-pointer call; 0 = off, -1 = plan
    bool host_slab_rows = false;
};
Options g_opt;
std::mutex g_opt_mutex;

int apply_option(const char* name, const char* value) {
    const Options def;
    const bool reset = !value || !*value;
    auto num = [&](int d) { return reset ? d : std::atoi(value); };
    if (!std::strcmp(name, "tc3")) g_opt.tc3 = num(def.tc3);
    else if (!std::strcmp(name, "tc_tile_rows")) g_opt.tc_tile_rows = num(def.tc_tile_rows);
    else if (!std::strcmp(name, "tc_bn")) g_opt.tc_bn = num(def.tc_bn);
    else if (!std::strcmp(name, "tc_ksplit")) g_opt.tc_ksplit = num(def.tc_ksplit);
    else if (!std::strcmp(name, "group_words")) g_opt.group_words = num(def.group_words);
    else if (!std::strcmp(name, "gemv_pdl")) g_opt.gemv_pdl = num(def.gemv_pdl);
    else if (!std::strcmp(name, "mma_slices")) g_opt.mma_slices = num(def.mma_slices);
    else if (!std::strcmp(name, "mma_cluster")) g_opt.mma_cluster = num(def.mma_cluster);
    else if (!std::strcmp(name, "skinny_split")) g_opt.skinny_split = num(def.skinny_split);
    else if (!std::strcmp(name, "gemv_plan")) {
        g_opt.gemv_words = def.gemv_words; g_opt.gemv_split = def.gemv_split;
        if (!reset) std::sscanf(value, "%d,%d", &g_opt.gemv_words, &g_opt.gemv_split);
    } else if (!std::strcmp(name, "mma_rows")) {
        g_opt.mma_lo = def.mma_lo; g_opt.mma_hi = def.mma_hi;
        if (!reset) std::sscanf(value, "%d,%d", &g_opt.mma_lo, &g_opt.mma_hi);
    } else if (!std::strcmp(name, "skinny_rows")) {
        g_opt.skinny_lo = def.skinny_lo; g_opt.skinny_hi = def.skinny_hi;
        if (!reset) std::sscanf(value, "%d,%d", &g_opt.skinny_lo, &g_opt.skinny_hi);
    } else if (!std::strcmp(name, "skinny_group_rows")) {
        g_opt.skinny_group_lo = def.skinny_group_lo; g_opt.skinny_group_hi = def.skinny_group_hi;
        if (!reset && std::sscanf(value, "%d,%d", &g_opt.skinny_group_lo, &g_opt.skinny_group_hi) == 1)
            g_opt.skinny_group_hi = def.skinny_group_hi;
    } else if (!std::strcmp(name, "host_slab")) {
        g_opt.host_slab = def.host_slab; g_opt.host_slab_rows = false;
        if (!reset) {
            g_opt.host_slab_rows = value[0] == 'r';
            g_opt.host_slab = std::atoi(value + (g_opt.host_slab_rows ? 1 : 0));
        }
    } else return TERNIX_B200_ERR_INVALID_ARG;
    return TERNIX_B200_OK;
}

const Options& options() {
    static std::once_flag once;
    std::call_once(once, [] {
        static const char* const names[] = {"tc3", "tc_tile_rows", "tc_bn", "tc_ksplit", "gemv_plan", "group_words", "gemv_pdl", "mma_rows", "mma_slices",
                                            "mma_cluster", "skinny_rows", "skinny_group_rows", "skinny_split", "host_slab"};
        std::lock_guard<std::mutex> lock(g_opt_mutex);
        for (const char* n : names) {
            char env[64] = "TERNIX_B200_";
            size_t len = std::strlen(env);
            for (const char* c = n; *c && len + 1 < sizeof env; ++c) env[len++] = static_cast<char>(std::toupper(*c));
            env[len] = 0;
            if (const char* v = std::getenv(env)) apply_option(n, v);
        }
    });
    return g_opt;
}

// Stream-ordered memory pool of the host-pointer entry point, one per device, created on first use.  Freed blocks
// stay in the pool up to kPoolKeepBytes so that repeated calls skip the driver allocation; what is above that goes
// back to the driver at the next synchronisation, and ternix_b200_release_cached_memory() returns all of it.
constexpr unsigned long long kPoolKeepBytes = 1ull << 30;
std::mutex g_pool_mutex;
cudaMemPool_t g_pools[kMaxDevices] = {};

int host_call_pool(cudaMemPool_t* out) {
    int dev = 0;
    TB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return TERNIX_B200_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    if (!g_pools[dev]) {
        cudaMemPoolProps props{};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t p = nullptr;
        TB_CUDA(cudaMemPoolCreate(&p, &props));
        unsigned long long keep = kPoolKeepBytes;
        TB_CUDA(cudaMemPoolSetAttribute(p, cudaMemPoolAttrReleaseThreshold, &keep));
        g_pools[dev] = p;
    }
    *out = g_pools[dev];
    return TERNIX_B200_OK;
}

// ---------------------------------------------------------------- kernel eligibility
bool gemv_ok(const void* dW, int M, int K, int N) {
    return M <= 16 && (N % 64) == 0 && aligned(dW, 16) && K <= kMaxScaledK && K <= 8 * (tb200::kGemvMaxASlice / 4);
}
bool gemm_tc_ok(const void* dA, const void* dW, int K, int N) {
    return (N % 64) == 0 && (K % 16) == 0 && aligned(dA, 16) && aligned(dW, 16) && K <= kMaxScaledK;
}

// Members of a problem group with this many rows go to the mma.sync decode kernel (one row: the dp4a kernel;
// more: tcgen05 tiles).  Measured on 210 BitNet-2B projections per launch: 2 rows 116 us with dp4a row groups
// against 97 us here, 16 rows 732 us against 148 us.
constexpr int kGroupMmaMinRows = 2, kGroupMmaMaxRows = 64;

// Batched decode on the warp-level tensor instruction: row groups of 8 or 16, any M >= 1.
bool decode_mma_ok(const void* dA, const void* dW, int M, int K, int N) {
    return M >= 1 && (N % 64) == 0 && (K % 16) == 0 && K >= 16 && K <= 65536 && aligned(dA, 16) && aligned(dW, 16);
}
// Tensor-memory decode kernel (kernel_skinny_tc.cuh): up to 128 rows.
bool skinny_ok(const void* dA, const void* dW, int M, int K, int N) {
    return M >= 1 && M <= 128 && (N % 64) == 0 && (K % 16) == 0 && K >= 16 && K <= kMaxScaledK && aligned(dA, 16) &&
           aligned(dW, 16);
}

bool gemm_tc2_ok(const void* dA, const void* dW, int M, int K, int N) {
    return gemm_tc_ok(dA, dW, K, N) && M > 128 && N >= 256;
}

int select_kernel(const void* dA, const void* dW, int M, int K, int N) {
    const Options& o = options();
    if (M >= o.skinny_lo && M <= o.skinny_hi && skinny_ok(dA, dW, M, K, N)) return TERNIX_B200_KERNEL_SKINNY_TC;
    if (M >= o.mma_lo && M <= o.mma_hi && decode_mma_ok(dA, dW, M, K, N)) return TERNIX_B200_KERNEL_DECODE_MMA;
    if (gemv_ok(dW, M, K, N)) return TERNIX_B200_KERNEL_GEMV;
    if (gemm_tc_ok(dA, dW, K, N)) return TERNIX_B200_KERNEL_GEMM_TC;
    return TERNIX_B200_KERNEL_GENERIC;
}

// ---------------------------------------------------------------- launches
int launch_generic(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                   cudaStream_t st) {
    const int pitch = N / 4;
    dim3 grid((pitch + tb200::kGenBytes - 1) / tb200::kGenBytes, (M + tb200::kGenRows - 1) / tb200::kGenRows);
    if (grid.y > 65535) return TERNIX_B200_ERR_INVALID_SHAPE;
    // Few output tiles: cut K into slices (two CTAs per SM in all) that add into a zeroed C.
    const long tiles = static_cast<long>(grid.x) * grid.y;
    const int slabs = (K + tb200::kGenK - 1) / tb200::kGenK;
    int k_per_slice = K;
    if (tiles < sm_count() && slabs >= 8) {
        const int slices = static_cast<int>(std::min<long>(slabs, (2L * sm_count() + tiles - 1) / tiles));
        const int slabs_per_slice = (slabs + slices - 1) / slices;
        k_per_slice = slabs_per_slice * tb200::kGenK;
        grid.z = static_cast<unsigned>((slabs + slabs_per_slice - 1) / slabs_per_slice);
        if (grid.z > 1) TB_CUDA(cudaMemset2DAsync(dC, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(N) * 4, M, st));
    }
    tb200::ternary_generic_kernel<<<grid, tb200::kGenThreads, 0, st>>>(dA, dW, dC, M, K, N, ldc, k_per_slice);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

// Split-K plan of the GEMV: words per CTA row (32 -> 512 columns, 16 -> 256 columns) and cluster size.
struct GemvPlan {
    int words, ksplit, krange;
};

GemvPlan plan_gemv_with(int M, int K, int N, int force_words, int force_split) {
    const int row_groups = (M + 3) / 4;
    const int target = 2 * sm_count();
    GemvPlan best{0, 0, 0};
    long best_score = -1;
    for (int words : {16, 32}) {
        if (force_words && words != force_words) continue;
        const int stage_rows = 8 * (32 / words) * 4;
        const int chunks = (N + words * 16 - 1) / (words * 16);
        for (int ks : {1, 2, 4, 8}) {
            if (force_split && ks != force_split) continue;
            int krange = (K + ks - 1) / ks;
            krange = (krange + stage_rows - 1) / stage_rows * stage_rows;
            if (krange * 4 > tb200::kGemvMaxASlice) continue;
            if (ks > 1 && static_cast<long>(krange) * (ks - 1) >= K) continue;   // a rank would be idle
            const long ctas = static_cast<long>(chunks) * ks * row_groups;
            // closest to two resident CTAs per SM without exceeding it much; prefer wider tiles on ties
            long score = ctas <= target ? ctas * 1000 : (static_cast<long>(target) * 1000 - (ctas - target) * 200);
            score += words;
            if (score > best_score) { best_score = score; best = {words, ks, krange}; }
        }
    }
    return best;
}

GemvPlan plan_gemv(int M, int K, int N) {
    const Options& o = options();      // option gemv_plan = "words,ksplit" overrides the heuristic where feasible
    if (o.gemv_words || o.gemv_split) {
        const GemvPlan p = plan_gemv_with(M, K, N, o.gemv_words, o.gemv_split);
        if (p.words) return p;
    }
    return plan_gemv_with(M, K, N, 0, 0);
}

template <int MR, int WORDS>
int launch_gemv_t(const CUtensorMap& tmap, const int8_t* dA, int32_t* dC, int M, int K, int N, long long ldc,
                  const GemvPlan& p, int32_t* d_status, cudaStream_t st) {
    auto kern = tb200::ternary_gemv_kernel<MR, WORDS>;
    const size_t smem = tb200::gemv_smem_bytes<MR, WORDS>(p.krange);
    if (const int rc = ensure_smem_attr<tb200::ternary_gemv_kernel<MR, WORDS>>(
            tb200::gemv_smem_bytes<MR, WORDS>(tb200::kGemvMaxASlice / MR)))
        return rc;
    const int chunks = (N + WORDS * 16 - 1) / (WORDS * 16);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(chunks * p.ksplit, (M + MR - 1) / MR, 1);
    cfg.blockDim = dim3(tb200::kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int a_words_ok = (K % 4 == 0) && aligned(dA, 4);
    TB_CUDA(cudaLaunchKernelEx(&cfg, kern, tmap, dA, dC, M, K, N, ldc, p.krange, a_words_ok, d_status));
    return TERNIX_B200_OK;
}

int launch_gemv(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                int32_t* d_status, cudaStream_t st) {
    const GemvPlan p = plan_gemv(M, K, N);
    if (p.words == 0) return TERNIX_B200_ERR_UNSUPPORTED;
    const int stage_rows = 8 * (32 / p.words) * 4;
    CUtensorMap tmap;
    const int rc = make_tmap_2d(&tmap, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K),
                                static_cast<uint64_t>(N / 4), p.words * 4, stage_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
#define TB_GEMV(MR_, W_) launch_gemv_t<MR_, W_>(tmap, dA, dC, M, K, N, ldc, p, d_status, st)
    if (p.words == 32) {
        if (M == 1) return TB_GEMV(1, 32);
        if (M == 2) return TB_GEMV(2, 32);
        return TB_GEMV(4, 32);
    }
    if (M == 1) return TB_GEMV(1, 16);
    if (M == 2) return TB_GEMV(2, 16);
    return TB_GEMV(4, 16);
#undef TB_GEMV
}


// ---------------------------------------------------------------- batched decode on mma.sync (kernel_decode_mma.cuh)
int make_mma_problem(tb200::MmaProblem* out, const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N,
                     long long ldc) {
    *out = tb200::MmaProblem{};
    int rc = make_tmap_2d(&out->tmap_w, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K),
                          static_cast<uint64_t>(N / 4), tb200::kMmaItemCols / 4, tb200::kMmaStageRows,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&out->tmap_a, dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), 64,
                      tb200::kMmaBoxRows, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    out->C = dC;
    out->ldc = ldc;
    out->M = M;
    out->K = K;
    out->N = N;
    out->c_vec_ok = (ldc % 4 == 0) && aligned(dC, 16);
    return TERNIX_B200_OK;
}

template <bool kSingle, int NG>
int decode_mma_attr() {
    return ensure_smem_attr<tb200::ternary_decode_mma_kernel<kSingle, NG>>(tb200::kMmaSmemBytes);
}

// One problem: items enumerated in the kernel.  When whole-K items would leave most of the GPU idle the K range is
// cut into slices that add into a zeroed C.
template <int NG>
int launch_decode_mma_t(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                        int32_t* d_status, cudaStream_t st) {
    tb200::MmaProblem prob;
    int rc = make_mma_problem(&prob, dA, dW, dC, M, K, N, ldc);
    if (rc) return rc;
    if ((rc = decode_mma_attr<true, NG>())) return rc;
    auto kern = tb200::ternary_decode_mma_kernel<true, NG>;
    tb200::MmaSingle sg{};
    sg.group_rows = 8 * NG;
    sg.chunks = (N + tb200::kMmaItemCols - 1) / tb200::kMmaItemCols;
    sg.row_groups = (M + sg.group_rows - 1) / sg.group_rows;
    sg.total_tiles = (K + tb200::kMmaStageRows - 1) / tb200::kMmaStageRows;
    const int resident = sm_count() * tb200::kMmaCtasPerSm;
    const int base_items = sg.chunks * sg.row_groups;
    // Slices of K buy parallelism (a lone CTA streams about 23 GB/s) and cost one red.global.add per output and
    // slice (the L2 retires about 160 of them per ns), plus the zeroing of C.  Take the count with the smallest sum
    // (option mma_slices forces the count).
    int slices = 1;
    {
        const double w_bytes = static_cast<double>(K) * (N / 4) * sg.row_groups;
        double best = 0;
        const int max_slices = std::max(1, std::min(sg.total_tiles / 2, resident / std::max(1, base_items)));
        for (int sl = 1; sl <= max_slices; ++sl) {
            const int ctas = std::min(resident, base_items * sl);
            const double stream_ns = std::max(w_bytes / (ctas * 23.0), w_bytes / 6000.0);
            const double add_ns = sl > 1 ? 2000.0 + static_cast<double>(M) * N * sl / 160.0 : 0.0;
            const double total = stream_ns + add_ns;
            if (sl == 1 || total < best) { best = total; slices = sl; }
        }
    }
    const Options& o = options();
    if (o.mma_slices > 0) slices = std::max(1, std::min(o.mma_slices, sg.total_tiles));
    // Cluster form: the largest cluster that still leaves one item per resident CTA (option mma_cluster = 0|2|4|8
    // overrides; a forced slice count switches the cluster form off).
    int cluster = 0;
    for (int c : {8, 4, 2})
        if (base_items * c <= resident && sg.total_tiles >= 2 * c) { cluster = c; break; }
    if (o.mma_cluster >= 0) {
        const int c = o.mma_cluster;
        cluster = ((c == 2 || c == 4 || c == 8) && base_items * c <= resident) ? c : 0;
    } else if (o.mma_slices > 0) {
        cluster = 0;
    }
    if (cluster) {
        sg.cluster = cluster;
        sg.slices = cluster;
        sg.tiles_per_slice = (sg.total_tiles + cluster - 1) / cluster;
        sg.add = 0;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(base_items * cluster));
        cfg.blockDim = dim3(tb200::kMmaThreads);
        cfg.dynamicSmemBytes = tb200::kMmaSmemBytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const tb200::MmaProblem* no_probs = nullptr;
        const tb200::MmaItem* no_items = nullptr;
        const int* no_first = nullptr;
        TB_CUDA(cudaLaunchKernelEx(&cfg, kern, prob, sg, no_probs, no_items, no_first, d_status));
        return TERNIX_B200_OK;
    }
    sg.tiles_per_slice = (sg.total_tiles + slices - 1) / slices;
    sg.slices = (sg.total_tiles + sg.tiles_per_slice - 1) / sg.tiles_per_slice;
    sg.add = sg.slices > 1;
    if (sg.add) TB_CUDA(cudaMemset2DAsync(dC, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(N) * 4, M, st));
    const int grid = std::min(resident, base_items * sg.slices);
    kern<<<grid, tb200::kMmaThreads, tb200::kMmaSmemBytes, st>>>(prob, sg, nullptr, nullptr, nullptr, d_status);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

// Row groups of 8 up to 8 rows (half the tensor instructions), of 16 beyond.
int launch_decode_mma(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                      int32_t* d_status, cudaStream_t st) {
    if (M <= 8) return launch_decode_mma_t<1>(dA, dW, dC, M, K, N, ldc, d_status, st);
    return launch_decode_mma_t<2>(dA, dW, dC, M, K, N, ldc, d_status, st);
}

template <int BN>
int launch_gemm_tc_t(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                     int32_t* d_status, cudaStream_t st) {
    using G = tb200::TcGeom<BN>;
    auto kern = tb200::ternary_gemm_tc_kernel<BN>;
    if (const int arc = ensure_smem_attr<tb200::ternary_gemm_tc_kernel<BN>>(G::kSmemBytes)) return arc;
    CUtensorMap tmap_a, tmap_w;
    int rc = make_tmap_2d(&tmap_a, dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K),
                          tb200::kTcBK, tb200::kTcBM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmap_w, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K),
                      static_cast<uint64_t>(N / 4), G::kWpRowBytes, tb200::kTcBK, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const long tiles = static_cast<long>((M + tb200::kTcBM - 1) / tb200::kTcBM) * ((N + BN - 1) / BN);
    // Skinny problems: split K so that every SM gets a work item; partial results are added into a zeroed C.
    int k_slices = 1;
    const int k_blocks = (K + tb200::kTcBK - 1) / tb200::kTcBK;
    if (tiles * 2 <= sm_count() && k_blocks >= 8) k_slices = static_cast<int>(std::min<long>(sm_count() / tiles, k_blocks / 4));
    if (!options().tc_ksplit) k_slices = 1;
    if (k_slices > 1)
        TB_CUDA(cudaMemset2DAsync(dC, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(N) * 4, M, st));
    const long items = tiles * k_slices;
    const int grid = static_cast<int>(items < sm_count() ? items : sm_count());
    const int c_vec_ok = (ldc % 4 == 0) && aligned(dC, 16);
    kern<<<grid, tb200::kTcThreads, G::kSmemBytes, st>>>(tmap_a, tmap_w, dC, M, K, N, ldc, c_vec_ok, k_slices, d_status);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

// Paired-CTA kernel that expands the weights into shared memory: clusters of two CTAs, one 256 x 256 tile per
// cluster at a time.  Serves outputs the TMA unit cannot describe (and option tc3 = 0).
int launch_gemm_tc2_expand(const int8_t* dA, const uint8_t* dW, int32_t* const* dC_list, int n_dest, int M, int K, int N,
                           long long ldc, int32_t* d_status, cudaStream_t st) {
    constexpr size_t smem = tb200::Tc2Geom::kSmemBytes;
    if (const int arc = ensure_smem_attr<tb200::ternary_gemm_tc2_kernel<false>>(smem)) return arc;
    CUtensorMap tmap_a, tmap_w;
    int rc = make_tmap_2d(&tmap_a, dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K),
                          tb200::kTcBK, tb200::kTcBM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmap_w, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K),
                      static_cast<uint64_t>(N / 4), tb200::Tc2Geom::kWpRowBytes, tb200::kTcBK, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const long tiles = static_cast<long>((M + 255) / 256) * ((N + tb200::kTc2TileN - 1) / tb200::kTc2TileN);
    const long max_pairs = sm_count() / 2;
    const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    tb200::Tc2Dest dest{};
    dest.count = n_dest;
    int c_vec_ok = (ldc % 4 == 0);
    for (int d = 0; d < n_dest; ++d) {
        dest.c[d] = dC_list[d];
        c_vec_ok = c_vec_ok && aligned(dC_list[d], 16);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(tb200::kTc2Threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TB_CUDA(cudaLaunchKernelEx(&cfg, tb200::ternary_gemm_tc2_kernel<false>, tmap_a, tmap_w, dest, M, K, N, ldc,
                               c_vec_ok, static_cast<const tb200::Tc2Problem*>(nullptr),
                               static_cast<const tb200::Tc2Tile*>(nullptr), static_cast<const int*>(nullptr), d_status,
                               static_cast<const float*>(nullptr), 1.0f));
    return TERNIX_B200_OK;
}

// Paired CTAs with the weights as the A operand in tensor memory (kernel_gemm_tc3.cuh).  Several destinations need
// every C to be describable to the TMA unit (16-byte aligned base and pitch); ERR_UNSUPPORTED otherwise.
// Activation rows per pair instruction: the 128-row form for products that have no more rows than that.
int tc3_tile_rows(int M) {
    const int forced = options().tc_tile_rows;
    if (forced == 128 || forced == 256) return forced;
    return M <= 128 ? 128 : 256;
}

int make_tc3_act_map(CUtensorMap* out, const int8_t* dA, int M, int K, int tile_rows = 256) {
    return make_tmap_2d(out, dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), tb200::kTcBK,
                        tile_rows / 2, CU_TENSOR_MAP_SWIZZLE_128B);
}
int make_tc3_weight_map(CUtensorMap* out, const uint8_t* dW, int K, int N) {
    return make_tmap_2d(out, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K), static_cast<uint64_t>(N / 4),
                        tb200::kTc3WpRowBytes, tb200::kTc3BK, CU_TENSOR_MAP_SWIZZLE_32B);
}
int make_tc3_store_map(CUtensorMap* out, int32_t* dC, int M, int N, long long ldc) {
    return make_tmap_2d_u32(out, dC, static_cast<uint64_t>(N), static_cast<uint64_t>(M), static_cast<uint64_t>(ldc) * 4, 128, 32);
}

template <int TA>
int launch_gemm_tc3_maps_t(const CUtensorMap& tmap_a, const CUtensorMap& tmap_w, const tb200::Tc3Stores& stores, int32_t* dC0,
                           int M, int K, int N, long long ldc, int32_t* d_status, cudaStream_t st) {
    if (const int arc = ensure_smem_attr<tb200::ternary_gemm_tc3_kernel<false, false, TA>>(tb200::tc3_smem_bytes<TA>())) return arc;
    const long tiles = static_cast<long>((M + TA - 1) / TA) * ((N + tb200::kTc3TileW - 1) / tb200::kTc3TileW);
    const long max_pairs = sm_count() / 2;
    const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(tb200::kTc3Threads, 1, 1);
    cfg.dynamicSmemBytes = tb200::tc3_smem_bytes<TA>();
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const tb200::Tc3Problem* no_probs = nullptr;
    const tb200::Tc2Tile* no_tiles = nullptr;
    const int* no_first = nullptr;
    TB_CUDA(cudaLaunchKernelEx(&cfg, tb200::ternary_gemm_tc3_kernel<false, false, TA>, tmap_a, tmap_w, stores, dC0, M, K, N, ldc,
                               no_probs, no_tiles, no_first, d_status, static_cast<const float*>(nullptr), 1.0f));
    return TERNIX_B200_OK;
}

// tmap_a must have been made for tc3_tile_rows(M).
int launch_gemm_tc3_maps(const CUtensorMap& tmap_a, const CUtensorMap& tmap_w, const tb200::Tc3Stores& stores, int32_t* dC0,
                         int M, int K, int N, long long ldc, int32_t* d_status, cudaStream_t st) {
    if (tc3_tile_rows(M) == 128)
        return launch_gemm_tc3_maps_t<128>(tmap_a, tmap_w, stores, dC0, M, K, N, ldc, d_status, st);
    return launch_gemm_tc3_maps_t<256>(tmap_a, tmap_w, stores, dC0, M, K, N, ldc, d_status, st);
}

int launch_gemm_tc3(const int8_t* dA, const uint8_t* dW, int32_t* const* dC_list, int n_dest, int M, int K, int N,
                    long long ldc, int32_t* d_status, cudaStream_t st) {
    if (n_dest < 1 || n_dest > tb200::kTc3MaxDest) return TERNIX_B200_ERR_UNSUPPORTED;
    bool tma_ok = (ldc % 4 == 0);
    for (int d = 0; d < n_dest; ++d) tma_ok = tma_ok && aligned(dC_list[d], 16);
    if (!tma_ok && n_dest > 1) return TERNIX_B200_ERR_UNSUPPORTED;
    CUtensorMap tmap_a, tmap_w;
    int rc = make_tc3_act_map(&tmap_a, dA, M, K, tc3_tile_rows(M));
    if (rc) return rc;
    rc = make_tc3_weight_map(&tmap_w, dW, K, N);
    if (rc) return rc;
    tb200::Tc3Stores stores{};
    stores.count = tma_ok ? n_dest : 0;
    for (int d = 0; d < stores.count; ++d)
        if ((rc = make_tc3_store_map(&stores.tmap_c[d], dC_list[d], M, N, ldc))) return rc;
    return launch_gemm_tc3_maps(tmap_a, tmap_w, stores, dC_list[0], M, K, N, ldc, d_status, st);
}

int launch_gemm_tc2(const int8_t* dA, const uint8_t* dW, int32_t* const* dC_list, int n_dest, int M, int K, int N,
                    long long ldc, int32_t* d_status, cudaStream_t st, int* used = nullptr) {
    // The kernel that keeps the decoded weights in tensor memory, unless option tc3 = 0 asks for the kernel that
    // expands them into shared memory or a C among several destinations has no TMA view.
    if (options().tc3) {
        const int rc = launch_gemm_tc3(dA, dW, dC_list, n_dest, M, K, N, ldc, d_status, st);
        if (rc != TERNIX_B200_ERR_UNSUPPORTED) {
            if (used) *used = TERNIX_B200_LAUNCHED_GEMM_TC3;
            return rc;
        }
    }
    if (used) *used = TERNIX_B200_LAUNCHED_GEMM_TC2;
    return launch_gemm_tc2_expand(dA, dW, dC_list, n_dest, M, K, N, ldc, d_status, st);
}

int launch_gemm_tc(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                   int32_t* d_status, cudaStream_t st, int* used = nullptr) {
    // Option tc_bn = 128|256 forces the single-CTA kernel at that tile width, tc_bn = 2 the paired-CTA kernels.
    // Default: pairs from 65 rows up.  The tensor-memory kernel pads a half-empty activation tile for nothing (rows
    // beyond M arrive as zeros from TMA) and still beats the single-CTA tiles; with tc3 = 0 the limit is 128 rows.
    const Options& o = options();
    int bn = o.tc_bn;
    const int pair_min_rows = o.tc3 ? 64 : 128;
    if (bn == 2 || (bn == 0 && M > pair_min_rows && N >= 256))
        return launch_gemm_tc2(dA, dW, &dC, 1, M, K, N, ldc, d_status, st, used);
    if (bn != 128 && bn != 256) {
        const long m_tiles = (M + tb200::kTcBM - 1) / tb200::kTcBM;
        const long tiles256 = m_tiles * ((N + 255) / 256);
        const long tiles128 = m_tiles * ((N + 127) / 128);
        // 256-wide tiles when they fill the machine, or when 128-wide tiles neither fill it nor leave room for a
        // K-split while 256-wide tiles do (skinny M: 43 tiles x 3 K-slices beat 86 unsplit tiles)
        const bool fill256 = tiles256 >= sm_count();
        const bool split256 = tiles128 * 2 > sm_count() && tiles256 * 2 <= sm_count() && K >= 1024;
        bn = (N % 256 == 0 || N > 256) && (fill256 || split256) ? 256 : 128;
    }
    if (used) *used = TERNIX_B200_LAUNCHED_GEMM_TC1;
    if (bn == 256) return launch_gemm_tc_t<256>(dA, dW, dC, M, K, N, ldc, d_status, st);
    return launch_gemm_tc_t<128>(dA, dW, dC, M, K, N, ldc, d_status, st);
}

// ---------------------------------------------------------------- tensor-memory decode kernel (kernel_skinny_tc.cuh)
// CTAs of one launch that share a 256-column block hand their partial sums on through C and signal each other with
// one flag per CTA.  The flags live in a file-scope device array (no allocation); a launch gets the slot of its
// (device, stream) pair, because launches on one stream run one after the other and launches on different streams
// may overlap.  When all slots of a device are taken by other streams the launch falls back to whole blocks per CTA,
// which needs no flags.  Flags carry the launch's epoch, so nothing is ever cleared.
constexpr int kSkFlagSlots = 32;
__device__ int g_sk_flags[kSkFlagSlots * tb200::kSkMaxCtas];
std::mutex g_sk_mutex;
int* g_sk_flags_dev[kMaxDevices] = {};
cudaStream_t g_sk_slot_stream[kMaxDevices][kSkFlagSlots] = {};
bool g_sk_slot_used[kMaxDevices][kSkFlagSlots] = {};
std::atomic<unsigned> g_sk_epoch{0};

// Device address of the flag slot for (current device, stream); *out = nullptr when every slot belongs to another stream.
int skinny_flag_slot(cudaStream_t st, int** out) {
    *out = nullptr;
    const int dev = current_device();
    std::lock_guard<std::mutex> lock(g_sk_mutex);
    if (!g_sk_flags_dev[dev]) {
        void* p = nullptr;
        TB_CUDA(cudaGetSymbolAddress(&p, g_sk_flags));      // with this device current: the symbol's copy on it
        g_sk_flags_dev[dev] = static_cast<int*>(p);
    }
    int free_slot = -1;
    for (int i = 0; i < kSkFlagSlots; ++i) {
        if (g_sk_slot_used[dev][i] && g_sk_slot_stream[dev][i] == st) { *out = g_sk_flags_dev[dev] + i * tb200::kSkMaxCtas; return TERNIX_B200_OK; }
        if (!g_sk_slot_used[dev][i] && free_slot < 0) free_slot = i;
    }
    if (free_slot >= 0) {
        g_sk_slot_used[dev][free_slot] = true;
        g_sk_slot_stream[dev][free_slot] = st;
        *out = g_sk_flags_dev[dev] + free_slot * tb200::kSkMaxCtas;
    }
    return TERNIX_B200_OK;
}

int next_skinny_epoch() {
    unsigned e = ++g_sk_epoch;
    if ((e & 0x7fffffffu) == 0) e = ++g_sk_epoch;          // never 0: that is what fresh flags hold
    return static_cast<int>(e & 0x7fffffffu);
}

int skinny_rows_class(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128; }

int make_skinny_problem(tb200::SkProblem* out, const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N,
                        long long ldc) {
    *out = tb200::SkProblem{};
    int rc = make_tmap_2d(&out->tmap_w, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K),
                          static_cast<uint64_t>(N / 4), tb200::kSkWpRowBytes, tb200::kSkBK, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    rc = make_tmap_2d(&out->tmap_a, dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), 128,
                      skinny_rows_class(M), CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    out->C = dC;
    out->ldc = ldc;
    out->M = M;
    out->K = K;
    out->N = N;
    return TERNIX_B200_OK;
}

template <int NB, bool kGrouped>
int launch_skinny_t(const tb200::SkProblem& single, const tb200::SkSingle& sg, const tb200::SkProblem* d_probs,
                    const tb200::SkItem* d_items, const int* d_first, int grid, int* d_flags, int epoch,
                    int32_t* d_status, cudaStream_t st) {
    if (const int arc = ensure_smem_attr<tb200::ternary_skinny_tc_kernel<NB, kGrouped>>(tb200::SkGeom<NB>::kSmemBytes))
        return arc;
    tb200::ternary_skinny_tc_kernel<NB, kGrouped><<<grid, tb200::SkGeom<NB>::kThreads, tb200::SkGeom<NB>::kSmemBytes, st>>>(
        single, sg, d_probs, d_items, d_first, d_flags, epoch, d_status);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

// The plan of one problem.  Whole-K items keep all CTAs on the same weight rows at the same time (the matrix streams
// row by row, which is what DRAM likes) and need no exchange of partial sums, so they are taken whenever they occupy
// the machine reasonably: items of 128 columns when there are at most as many as SMs, items of 256 columns when
// those fit in one round.  Otherwise (more 256-column blocks than SMs, or option skinny_split = 2) the
// (block, stage) units are dealt out as one contiguous range per CTA, a block being shared by at most a few CTAs
// with neighbouring indices; that form needs a flag slot.
void plan_skinny(int K, int N, bool can_split, int split_mode, tb200::SkSingle* sg, int* grid) {
    const int blocks256 = (N + tb200::kSkItemCols - 1) / tb200::kSkItemCols, blocks128 = (N + 127) / 128;
    sg->stages = (K + tb200::kSkBK - 1) / tb200::kSkBK;
    const int sms = std::min(sm_count(), tb200::kSkMaxCtas);
    sg->half_items = 0;
    sg->whole_blocks = 1;
    if (blocks128 <= sms && split_mode < 2) {
        sg->half_items = 1;
        sg->blocks = blocks128;
        *grid = blocks128;
        return;
    }
    sg->blocks = blocks256;
    const bool want_split = can_split && (split_mode >= 2 || blocks256 > sms);
    const long long units = static_cast<long long>(blocks256) * sg->stages;
    const int min_units = std::max(2, (sg->stages + 1) / 2);       // at most three CTAs share a block
    const int g = static_cast<int>(std::max<long long>(1, std::min<long long>(sms, units / min_units)));
    if (want_split && !(g <= blocks256 && blocks256 % g == 0)) {
        sg->whole_blocks = 0;
        *grid = g;
    } else {
        *grid = std::min(sms, blocks256);
    }
}

int launch_skinny_problem(const tb200::SkProblem& prob, int32_t* d_status, cudaStream_t st) {
    tb200::SkSingle sg{};
    int grid = 0;
    int* d_flags = nullptr;
    const int split_mode = options().skinny_split;
    if (split_mode) {
        const int rc = skinny_flag_slot(st, &d_flags);
        if (rc) return rc;
    }
    plan_skinny(prob.K, prob.N, d_flags != nullptr, split_mode, &sg, &grid);
    const int epoch = sg.whole_blocks ? 0 : next_skinny_epoch();
    switch (skinny_rows_class(prob.M)) {
        case 16: return launch_skinny_t<16, false>(prob, sg, nullptr, nullptr, nullptr, grid, d_flags, epoch, d_status, st);
        case 32: return launch_skinny_t<32, false>(prob, sg, nullptr, nullptr, nullptr, grid, d_flags, epoch, d_status, st);
        case 64: return launch_skinny_t<64, false>(prob, sg, nullptr, nullptr, nullptr, grid, d_flags, epoch, d_status, st);
        default: return launch_skinny_t<128, false>(prob, sg, nullptr, nullptr, nullptr, grid, d_flags, epoch, d_status, st);
    }
}

int launch_skinny(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                  int32_t* d_status, cudaStream_t st) {
    tb200::SkProblem prob;
    const int rc = make_skinny_problem(&prob, dA, dW, dC, M, K, N, ldc);
    if (rc) return rc;
    return launch_skinny_problem(prob, d_status, st);
}

// ---------------------------------------------------------------- self-test of the bounded waits
// What every kernel of this library does when a wait runs out, in isolation and with a short limit: warp 0 waits
// for a shared-memory barrier that nobody will ever arrive on; when the limit ends it raises the CTA's abort flag;
// warp 1, waiting on a second barrier, sees the flag and leaves too; the "copy in flight" is drained with the same
// bounded helper; the CTA reports TERNIX_B200_ERR_TIMEOUT through the status word and returns.  No TMA, no tensor
// memory, nothing that faults: the context stays usable.
__global__ void wait_timeout_selftest_kernel(unsigned long long limit_ns, int32_t* __restrict__ status,
                                             unsigned long long* __restrict__ waited_ns) {
    __shared__ uint64_t bars[2];
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        tb200::mbar_init(&bars[0], 1);
        tb200::mbar_init(&bars[1], 1);
        abort_flag = 0;
        tb200::mbar_init_fence();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint64_t t0 = tb200::global_timer_ns();
    bool ok = true;
    if (lane == 0) {
        if (warp == 0) ok = tb200::mbar_wait(&bars[0], 0, &abort_flag, limit_ns);
        else ok = tb200::mbar_wait_backoff(&bars[1], 0, &abort_flag, 64);       // leaves through the abort flag
        if (!ok && warp == 0) tb200::mbar_drain(&bars[1], 0, limit_ns);         // teardown path, bounded as well
    }
    __syncwarp();
    if (abort_flag && lane == 0 && status) atomicMax(status, tb200::kStatusTimeout);
    __syncthreads();
    if (threadIdx.x == 0 && waited_ns) *waited_ns = tb200::global_timer_ns() - t0;
}

// Barrier between the GPUs of a sharded product, on a stream: thread t tells rank t that this rank has arrived (a
// release store, at system scope, of the barrier's epoch into slot `rank` of rank t's flag array) and then waits until
// rank t's epoch shows in slot t of this rank's own array.  Stream order puts the kernel behind this rank's GEMM, so
// the release also covers the GEMM's stores into the peers' C; the acquire on the other side makes them visible to
// what the peer runs next.  Epochs only grow, so a rank that is a barrier ahead does no harm.  The wait is bounded
// like every other wait of this library (status word, no trap).
constexpr int kPeerBarrierMaxRanks = 32;
struct PeerFlags {
    unsigned* flags[kPeerBarrierMaxRanks];     // flags[r]: rank r's array of `world` slots (own rank: the local array)
};
__global__ void peer_barrier_kernel(const __grid_constant__ PeerFlags pf, int world, int rank, unsigned epoch,
                                    unsigned long long limit_ns, int32_t* __restrict__ status) {
    const int t = threadIdx.x;
    if (t >= world || t == rank) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.flags[t] + rank), "r"(epoch) : "memory");
    const unsigned* mine = pf.flags[rank] + t;
    const uint64_t t0 = tb200::global_timer_ns();
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if (static_cast<int>(v - epoch) >= 0) break;
        if (tb200::global_timer_ns() - t0 > limit_ns) {
            if (status) atomicMax(status, tb200::kStatusTimeout);
            break;
        }
        __nanosleep(100);
    }
}

// Device-side packer: four consecutive int8 weights -> one byte, the arithmetic of the host packer
// (code = 1 for +1, 3 for -1, else 0; field j in bits 2j..2j+1).  One thread packs 16 weights into 4 bytes.
__global__ void pack_ternary_kernel(const int8_t* __restrict__ w, uint8_t* __restrict__ packed, size_t n_bytes) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    const size_t n_words = n_bytes / 4;
    auto code4 = [](uint32_t v) {      // four int8 in a word -> four 2-bit codes in the low byte
        uint32_t out = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int8_t x = static_cast<int8_t>(v >> (8 * j));
            out |= (x == 1 ? 1u : x == -1 ? 3u : 0u) << (2 * j);
        }
        return out;
    };
    const bool vec = (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(packed) & 3) == 0;
    if (vec) {
        for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_words; i += stride) {
            const uint4 v = reinterpret_cast<const uint4*>(w)[i];
            reinterpret_cast<uint32_t*>(packed)[i] = code4(v.x) | (code4(v.y) << 8) | (code4(v.z) << 16) | (code4(v.w) << 24);
        }
    }
    // tail bytes (and everything, when the pointers are not aligned for the vector path)
    const size_t first = vec ? n_words * 4 : 0;
    for (size_t b = first + blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; b < n_bytes; b += stride) {
        uint32_t v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) v |= static_cast<uint32_t>(static_cast<uint8_t>(w[4 * b + j])) << (8 * j);
        packed[b] = static_cast<uint8_t>(code4(v));
    }
}

// Rank-major gather buffer -> row-major C.
__global__ void unpack_gathered_kernel(const int32_t* __restrict__ g, int32_t* __restrict__ C, int M, int N,
                                       long long ldc, int world, int granule, int n_pad) {
    const int granules = (N + granule - 1) / granule;
    const int base = granules / world, extra = granules % world;
    const long long total = static_cast<long long>(M) * N;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / N), col = static_cast<int>(i % N);
        const int gi = col / granule;
        // ranks [0, extra) own base+1 granules, the rest own base
        int rank, first;
        if (gi < extra * (base + 1)) { rank = gi / (base + 1); first = rank * (base + 1); }
        else { rank = extra + (base ? (gi - extra * (base + 1)) / base : 0); first = extra * (base + 1) + (rank - extra) * base; }
        const int local = col - first * granule;
        C[static_cast<long long>(row) * ldc + col] =
            g[(static_cast<long long>(rank) * M + row) * n_pad + local];
    }
}

// ---------------------------------------------------------------- problem groups (many projections per launch)
bool group_gemv_ok(const ternix_b200_problem& q) {
    return q.M >= 1 && q.M <= 16 && q.K >= 1 && q.K <= tb200::kGroupMaxK && (q.K % 16) == 0 && (q.N % 64) == 0 &&
           q.N >= 64 && aligned(q.dA, 16) && aligned(q.dW, 16) && q.ldc >= q.N;
}

// Launch of the persistent one-row decode kernel.  A short launch (at most four items per CTA) is made a programmatic
// dependent of the kernel before it on the stream: when that kernel is another decode batch of this library (the
// only kernels here that release their dependents early), the new grid's CTAs move onto SMs as the old grid's CTAs
// retire and request their first weight tiles while the old grid finishes; they read activations and write C only
// after it has completed (griddepcontrol.wait).  Behind any other kernel or copy the launch waits for full completion
// as usual.  Measured: 64 x config 1 per launch 51.6 -> 48.7 us.  Long launches lose by it (256 x config 1: 182 -> 192
// us): CTAs that start one by one no longer walk the same weight rows as their neighbours at the same time, which
// costs more DRAM efficiency than the filled ramp gains.  Option gemv_pdl = 0 | 1 forces the choice.
template <class Kern>
int launch_decode_batch(Kern kern, int grid, size_t smem, cudaStream_t st, const tb200::GroupProblem* d_probs,
                        const tb200::GroupItem* d_items, const int* d_first, int32_t* d_status, bool short_launch) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(tb200::kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    const int pdl = options().gemv_pdl;
    cfg.numAttrs = (pdl > 0 || (pdl < 0 && short_launch)) ? 1 : 0;
    TB_CUDA(cudaLaunchKernelEx(&cfg, kern, d_probs, d_items, d_first, d_status));
    return TERNIX_B200_OK;
}

template <int MR, int WORDS, bool PRE = false>
int launch_gemv_group_t(const ternix_b200_group* g, int32_t* d_status, cudaStream_t st);

}  // namespace

struct ternix_b200_group {
    std::vector<ternix_b200_problem> singles;   // problems launched one by one
    void* d_blob = nullptr;                     // [GroupProblem[] | GroupItem[] | int cta_first[]]
    const tb200::GroupProblem* d_probs = nullptr;
    const tb200::GroupItem* d_items = nullptr;
    const int* d_cta_first = nullptr;
    int grid = 0, mr = 0, words = 0, device = 0;
    bool short_launch = false;                  // at most four items per CTA: launched as a programmatic dependent
    bool prepacked = false;                     // dW of every member is in the ternix_b200_prepack_k4 layout
    size_t grouped = 0;
    // prefill-regime members: one launch of the paired-CTA GEMM over all their tiles
    void* d_tc_blob = nullptr;                  // [Tc2Problem[] | Tc2Tile[] | int pair_first[]]
    const tb200::Tc2Problem* d_tc_probs = nullptr;
    const tb200::Tc3Problem* d_tc3_probs = nullptr;   // set instead of d_tc_probs when the tensor-memory kernel takes them
    const tb200::Tc2Tile* d_tc_tiles = nullptr;
    const int* d_tc_first = nullptr;
    int tc_pairs = 0;
    size_t tc_grouped = 0;
    // batched-decode members (3 to 64 rows): one launch of the mma.sync kernel per row-group size (8, 16)
    struct MmaTables {
        void* d_blob = nullptr;                 // [MmaProblem[] | MmaItem[] | int cta_first[]]
        const tb200::MmaProblem* d_probs = nullptr;
        const tb200::MmaItem* d_items = nullptr;
        const int* d_first = nullptr;
        int grid = 0;
    } mma[2];
    size_t mma_grouped = 0;
    // batched-decode members served by the tensor-memory kernel: one launch per batch class (16, 32, 64, 128 rows)
    struct SkTables {
        void* d_blob = nullptr;                 // [SkProblem[] | SkItem[] | int cta_first[]]
        const tb200::SkProblem* d_probs = nullptr;
        const tb200::SkItem* d_items = nullptr;
        const int* d_first = nullptr;
        int grid = 0;
    } sk[4];
    size_t sk_grouped = 0;
    // members the grouped kernels could not take but that have peer destinations: copied after their launch
    struct PeerCopy { ternix_b200_problem q; std::vector<int32_t*> peers; };
    std::vector<PeerCopy> single_peers;
};

// A weight matrix with its TMA descriptors encoded once (ternix_b200_weights_create).  A single-product launch
// otherwise spends more host time in cuTensorMapEncodeTiled than the decode kernels run for; with the handle a
// launch encodes nothing for operands it has seen before.
struct ternix_b200_weights {
    const uint8_t* dW = nullptr;
    int K = 0, N = 0, device = 0;
    bool fast = false;                 // N % 64 == 0, K % 16 == 0, 16-byte aligned: the TMA kernels apply
    CUtensorMap tmap_w_skinny{}, tmap_w_tc3{};
    std::mutex mu;                     // guards the one-entry caches below
    // last activation operand seen per kernel family, and last output
    const int8_t* a_ptr[2] = {nullptr, nullptr};
    int a_rows[2] = {0, 0};
    int a_tile_rows = 0;               // tile form the prefill kernel's activation map was made for
    CUtensorMap tmap_a[2] = {};
    int32_t* c_ptr = nullptr;
    int c_rows = 0;
    long long c_ld = 0;
    CUtensorMap tmap_c{};
};

namespace {

template <int MR, int WORDS, bool PRE>
int launch_gemv_group_t(const ternix_b200_group* g, int32_t* d_status, cudaStream_t st) {
    auto kern = tb200::ternary_gemv_group_kernel<MR, WORDS, PRE>;
    constexpr size_t smem = tb200::gemv_group_smem_bytes<MR, WORDS>();
    if (const int arc = ensure_smem_attr<tb200::ternary_gemv_group_kernel<MR, WORDS, PRE>>(smem)) return arc;
    return launch_decode_batch(kern, g->grid, smem, st, g->d_probs, g->d_items, g->d_cta_first, d_status, g->short_launch);
}

int launch_gemm_tc3_group(const ternix_b200_group* g, int32_t* d_status, cudaStream_t st) {
    auto kern = tb200::ternary_gemm_tc3_kernel<true>;
    if (const int arc = ensure_smem_attr<tb200::ternary_gemm_tc3_kernel<true>>(tb200::kTc3SmemBytes)) return arc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * g->tc_pairs, 1, 1);
    cfg.blockDim = dim3(tb200::kTc3Threads, 1, 1);
    cfg.dynamicSmemBytes = tb200::kTc3SmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CUtensorMap unused{};
    tb200::Tc3Stores none{};
    int32_t* no_c = nullptr;
    TB_CUDA(cudaLaunchKernelEx(&cfg, kern, unused, unused, none, no_c, 0, 0, 0, 0LL, g->d_tc3_probs, g->d_tc_tiles,
                               g->d_tc_first, d_status, static_cast<const float*>(nullptr), 1.0f));
    return TERNIX_B200_OK;
}

int launch_gemm_tc2_group(const ternix_b200_group* g, int32_t* d_status, cudaStream_t st) {
    if (g->d_tc3_probs) return launch_gemm_tc3_group(g, d_status, st);
    using G = tb200::Tc2Geom;
    auto kern = tb200::ternary_gemm_tc2_kernel<true>;
    if (const int arc = ensure_smem_attr<tb200::ternary_gemm_tc2_kernel<true>>(G::kSmemBytes)) return arc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * g->tc_pairs, 1, 1);
    cfg.blockDim = dim3(tb200::kTc2Threads, 1, 1);
    cfg.dynamicSmemBytes = G::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CUtensorMap unused{};
    tb200::Tc2Dest no_dest{};
    TB_CUDA(cudaLaunchKernelEx(&cfg, kern, unused, unused, no_dest, 0, 0, 0, 0LL, 0, g->d_tc_probs, g->d_tc_tiles,
                               g->d_tc_first, d_status, static_cast<const float*>(nullptr), 1.0f));
    return TERNIX_B200_OK;
}

// ---------------------------------------------------------------- the steps either side of the product
// Per-row absmax quantisation of activations (BitNet b1.58's activation quantiser): one CTA per row.
//   absmax = max_k |x|;  s = 127 / absmax;  q = rint(x * s) in [-127, 127];  row_scale = absmax / 127.
// An all-zero row gets q = 0 and row_scale = 1.  fp32 arithmetic, round-to-nearest-even.
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const T* __restrict__ X, long long ldx, int8_t* __restrict__ A, float* __restrict__ row_scale,
                     int M, int K) {
    __shared__ float s_max[8];
    const int row = blockIdx.x;
    const T* x = X + static_cast<size_t>(row) * ldx;
    float m = 0.0f;
    for (int k = threadIdx.x; k < K; k += 256) m = fmaxf(m, fabsf(to_f32<T>(x[k])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
    __syncthreads();
    m = s_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s_max[w]);
    const float s = m > 0.0f ? 127.0f / m : 0.0f;
    if (threadIdx.x == 0) row_scale[row] = m > 0.0f ? m / 127.0f : 1.0f;
    int8_t* a = A + static_cast<size_t>(row) * K;
    for (int k = threadIdx.x; k < K; k += 256) {
        int q = __float2int_rn(to_f32<T>(x[k]) * s);
        q = q > 127 ? 127 : q < -127 ? -127 : q;
        a[k] = static_cast<int8_t>(q);
    }
}

// y = bf16_rn((float(c) * row_scale[m]) * w_scale), from an int32 C to up to 8 bfloat16 destinations: the
// unfused form of the dequantising epilogue, for problems the paired-CTA kernel does not take.
__global__ void dequant_rows_kernel(const int32_t* __restrict__ C, long long ldc, tb200::Tc2Dest dest, long long ldy,
                                    const float* __restrict__ row_scale, float w_scale, int M, int N) {
    const long long total = static_cast<long long>(M) * N;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / N), col = static_cast<int>(i % N);
        const float v = (static_cast<float>(C[static_cast<size_t>(row) * ldc + col]) * row_scale[row]) * w_scale;
        const __nv_bfloat16 b = __float2bfloat16_rn(v);
        for (int d = 0; d < dest.count; ++d)
            reinterpret_cast<__nv_bfloat16*>(dest.c[d])[static_cast<size_t>(row) * ldy + col] = b;
    }
}

// The same product with the dequantising epilogue of the tensor-memory kernel (bfloat16 out, one TMA store per
// destination).  ERR_UNSUPPORTED when an output has no TMA view and there are several of them.
int launch_gemm_tc3_bf16(const int8_t* dA, const uint8_t* dW, void* const* dY_list, int n_dest, const float* row_scale,
                         float w_scale, int M, int K, int N, long long ldy, int32_t* d_status, cudaStream_t st) {
    auto kern = tb200::ternary_gemm_tc3_kernel<false, true>;
    if (const int arc = ensure_smem_attr<tb200::ternary_gemm_tc3_kernel<false, true>>(tb200::kTc3SmemBytes)) return arc;
    if (n_dest < 1 || n_dest > tb200::kTc3MaxDest) return TERNIX_B200_ERR_UNSUPPORTED;
    bool tma_ok = (ldy % 8 == 0);
    for (int d = 0; d < n_dest; ++d) tma_ok = tma_ok && aligned(dY_list[d], 16);
    if (!tma_ok && n_dest > 1) return TERNIX_B200_ERR_UNSUPPORTED;
    CUtensorMap tmap_a, tmap_w;
    int rc = make_tmap_2d(&tmap_a, dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), 128,
                          128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmap_w, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K), static_cast<uint64_t>(N / 4),
                      tb200::kTc3WpRowBytes, tb200::kTc3BK, CU_TENSOR_MAP_SWIZZLE_32B);
    if (rc) return rc;
    tb200::Tc3Stores stores{};
    stores.count = tma_ok ? n_dest : 0;
    for (int d = 0; d < stores.count; ++d) {
        rc = make_tmap_2d_u16(&stores.tmap_c[d], dY_list[d], static_cast<uint64_t>(N), static_cast<uint64_t>(M),
                              static_cast<uint64_t>(ldy) * 2, 128, 32);
        if (rc) return rc;
    }
    const long tiles = static_cast<long>((M + tb200::kTc3TileA - 1) / tb200::kTc3TileA) *
                       ((N + tb200::kTc3TileW - 1) / tb200::kTc3TileW);
    const long max_pairs = sm_count() / 2;
    const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(tb200::kTc3Threads, 1, 1);
    cfg.dynamicSmemBytes = tb200::kTc3SmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TB_CUDA(cudaLaunchKernelEx(&cfg, kern, tmap_a, tmap_w, stores, static_cast<int32_t*>(dY_list[0]), M, K, N, ldy,
                               static_cast<const tb200::Tc3Problem*>(nullptr), static_cast<const tb200::Tc2Tile*>(nullptr),
                               static_cast<const int*>(nullptr), d_status, row_scale, w_scale));
    return TERNIX_B200_OK;
}

int launch_gemm_tc2_bf16(const int8_t* dA, const uint8_t* dW, void* const* dY_list, int n_dest, const float* row_scale,
                         float w_scale, int M, int K, int N, long long ldy, int32_t* d_status, cudaStream_t st) {
    if (options().tc3) {
        const int rc3 = launch_gemm_tc3_bf16(dA, dW, dY_list, n_dest, row_scale, w_scale, M, K, N, ldy, d_status, st);
        if (rc3 != TERNIX_B200_ERR_UNSUPPORTED) return rc3;
    }
    using G = tb200::Tc2Geom;
    auto kern = tb200::ternary_gemm_tc2_kernel<false, true>;
    if (const int arc = ensure_smem_attr<tb200::ternary_gemm_tc2_kernel<false, true>>(G::kSmemBytes)) return arc;
    CUtensorMap tmap_a, tmap_w;
    int rc = make_tmap_2d(&tmap_a, dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K),
                          tb200::kTcBK, tb200::kTcBM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap_2d(&tmap_w, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K),
                      static_cast<uint64_t>(N / 4), G::kWpRowBytes, tb200::kTcBK, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    const long tiles = static_cast<long>((M + 255) / 256) * ((N + 255) / 256);
    const long max_pairs = sm_count() / 2;
    const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
    tb200::Tc2Dest dest{};
    dest.count = n_dest;
    int vec_ok = (ldy % 8 == 0);
    for (int d = 0; d < n_dest; ++d) {
        dest.c[d] = static_cast<int32_t*>(dY_list[d]);
        vec_ok = vec_ok && aligned(dY_list[d], 16);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(tb200::kTc2Threads, 1, 1);
    cfg.dynamicSmemBytes = G::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TB_CUDA(cudaLaunchKernelEx(&cfg, kern, tmap_a, tmap_w, dest, M, K, N, ldy, vec_ok,
                               static_cast<const tb200::Tc2Problem*>(nullptr), static_cast<const tb200::Tc2Tile*>(nullptr),
                               static_cast<const int*>(nullptr), d_status, row_scale, w_scale));
    return TERNIX_B200_OK;
}

// ---------------------------------------------------------------- decode batch without any allocation
// Scratch of ternix_b200_gemv_batch_noalloc: the tables the persistent GEMV kernel reads (per-problem TMA
// descriptors, the work list and each CTA's slice of it) live in this file-scope device array instead of a
// cudaMalloc'ed block.  Every GPU that loads the library carries it until the process exits.
constexpr int kNoAllocMaxProblems = 256;
constexpr int kNoAllocMaxItems = 4096;
constexpr int kNoAllocMaxCtas = 640;          // 148 SMs x 4 resident CTAs of the one-row kernel, with room
constexpr size_t kNoAllocProbBytes = size_t(kNoAllocMaxProblems) * sizeof(tb200::GroupProblem);
constexpr size_t kNoAllocItemBytes = size_t(kNoAllocMaxItems) * sizeof(tb200::GroupItem);
constexpr size_t kNoAllocFirstBytes = ((size_t(kNoAllocMaxCtas) + 1) * sizeof(int) + 255) & ~size_t(255);
constexpr size_t kNoAllocBytes = kNoAllocProbBytes + kNoAllocItemBytes + kNoAllocFirstBytes;   // 117,504 bytes
static_assert(kNoAllocProbBytes % 256 == 0 && kNoAllocItemBytes % 256 == 0, "sub-tables stay 256-byte aligned");

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// In host code `g_noalloc_scratch` is only a stand-in for the symbol, not a device address.  The address is
// looked up once per device, with that device current, and cached here.
constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_dev_ptr[kNoAllocMaxDevices] = {};

int noalloc_scratch_for_current_device(unsigned char** out) {
    int dev = 0;
    TB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kNoAllocMaxDevices) return TERNIX_B200_ERR_UNSUPPORTED;
    if (!g_noalloc_dev_ptr[dev]) {
        void* p = nullptr;
        TB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_noalloc_dev_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_noalloc_dev_ptr[dev];
    return TERNIX_B200_OK;
}

// Host-side staging of the same tables: fixed size, no heap.
struct NoAllocHostTables {
    tb200::GroupProblem probs[kNoAllocMaxProblems];
    tb200::GroupItem items[kNoAllocMaxItems];       // in CTA order
    tb200::GroupItem pending[kNoAllocMaxItems];     // before assignment, heaviest first
    unsigned short cta_of[kNoAllocMaxItems];
    int first[kNoAllocMaxCtas + 1];
    long load[kNoAllocMaxCtas];
};
NoAllocHostTables g_noalloc_host;

template <int MR, int WORDS>
int launch_gemv_group_tables(const tb200::GroupProblem* d_probs, const tb200::GroupItem* d_items, const int* d_first,
                             int grid, int32_t* d_status, cudaStream_t st, bool short_launch) {
    auto kern = tb200::ternary_gemv_group_kernel<MR, WORDS>;
    constexpr size_t smem = tb200::gemv_group_smem_bytes<MR, WORDS>();
    if (const int arc = ensure_smem_attr<tb200::ternary_gemv_group_kernel<MR, WORDS>>(smem)) return arc;
    return launch_decode_batch(kern, grid, smem, st, d_probs, d_items, d_first, d_status, short_launch);
}

}  // namespace

extern "C" {

const char* ternix_b200_status_string(int status) {
    switch (status) {
        case TERNIX_B200_OK: return "ok";
        case TERNIX_B200_ERR_INVALID_SHAPE: return "invalid shape (need M,K,N >= 0, N % 4 == 0, sizes within int32)";
        case TERNIX_B200_ERR_INVALID_ARG: return "invalid argument (null pointer, bad selector or pitch)";
        case TERNIX_B200_ERR_CUDA: return "CUDA error (see ternix_b200_last_cuda_error)";
        case TERNIX_B200_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        case TERNIX_B200_ERR_UNSUPPORTED: return "the requested kernel cannot take this problem";
        case TERNIX_B200_ERR_TOO_LARGE: return "the request exceeds the fixed capacity of this entry point";
        default: return "unknown status";
    }
}

int ternix_b200_last_cuda_error(void) { return g_last_cuda_error; }
const char* ternix_b200_cuda_error_string(int cuda_error) {
    return cudaGetErrorString(static_cast<cudaError_t>(cuda_error));
}
int ternix_b200_version(void) { return 200; }

int ternix_b200_set_option(const char* name, const char* value) {
    if (!name) return TERNIX_B200_ERR_INVALID_ARG;
    options();                                   // the environment is read first, once
    std::lock_guard<std::mutex> lock(g_opt_mutex);
    return apply_option(name, value);
}

int ternix_b200_last_launched_kernel(void) { return g_last_launched; }
const char* ternix_b200_launched_kernel_name(int id) {
    switch (id) {
        case TERNIX_B200_LAUNCHED_GENERIC: return "ternary_generic_kernel";
        case TERNIX_B200_LAUNCHED_GEMV: return "ternary_gemv_kernel";
        case TERNIX_B200_LAUNCHED_GEMM_TC1: return "ternary_gemm_tc_kernel";
        case TERNIX_B200_LAUNCHED_DECODE_MMA: return "ternary_decode_mma_kernel";
        case TERNIX_B200_LAUNCHED_SKINNY_TC: return "ternary_skinny_tc_kernel";
        case TERNIX_B200_LAUNCHED_GEMM_TC2: return "ternary_gemm_tc2_kernel";
        case TERNIX_B200_LAUNCHED_GEMM_TC3: return "ternary_gemm_tc3_kernel";
        default: return "none";
    }
}

int ternix_b200_release_cached_memory(void) {
    std::lock_guard<std::mutex> lock(g_pool_mutex);
    for (int dev = 0; dev < kMaxDevices; ++dev)
        if (g_pools[dev]) TB_CUDA(cudaMemPoolTrimTo(g_pools[dev], 0));
    return TERNIX_B200_OK;
}

int ternix_b200_select_kernel(const void* dA, const void* dW, const void* dC, int M, int K, int N, long long ldc) {
    (void)dC;
    (void)ldc;
    if (M < 0 || K < 0 || N < 0 || (N % 4) != 0) return -TERNIX_B200_ERR_INVALID_SHAPE;
    return select_kernel(dA, dW, M, K, N);
}

int ternix_b200_matmul_ex(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, long long ldc,
                          int kernel, int32_t* d_status, void* stream) {
    // Shape first, before any pointer is looked at (the reference's wrappers promise the same,
    // tests/test_cuda_matmul.cu:41-43).
    if (M < 0 || K < 0 || N < 0 || (N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (ldc < N) return TERNIX_B200_ERR_INVALID_ARG;
    if (kernel < TERNIX_B200_KERNEL_AUTO || kernel > TERNIX_B200_KERNEL_SKINNY_TC) return TERNIX_B200_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return TERNIX_B200_OK;
    if (!dC || (K > 0 && (!dA || !dW))) return TERNIX_B200_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K == 0) {   // empty sum: C = 0
        TB_CUDA(cudaMemset2DAsync(dC, static_cast<size_t>(ldc) * 4, 0, static_cast<size_t>(N) * 4, M, st));
        return TERNIX_B200_OK;
    }
    if (kernel == TERNIX_B200_KERNEL_AUTO) kernel = select_kernel(dA, dW, M, K, N);
    switch (kernel) {
        case TERNIX_B200_KERNEL_GEMV:
            if (!gemv_ok(dW, M, K, N)) return TERNIX_B200_ERR_UNSUPPORTED;
            g_last_launched = TERNIX_B200_LAUNCHED_GEMV;
            return launch_gemv(dA, dW, dC, M, K, N, ldc, d_status, st);
        case TERNIX_B200_KERNEL_GEMM_TC:
            if (!gemm_tc_ok(dA, dW, K, N)) return TERNIX_B200_ERR_UNSUPPORTED;
            return launch_gemm_tc(dA, dW, dC, M, K, N, ldc, d_status, st, &g_last_launched);
        case TERNIX_B200_KERNEL_DECODE_MMA:
            if (!decode_mma_ok(dA, dW, M, K, N)) return TERNIX_B200_ERR_UNSUPPORTED;
            g_last_launched = TERNIX_B200_LAUNCHED_DECODE_MMA;
            return launch_decode_mma(dA, dW, dC, M, K, N, ldc, d_status, st);
        case TERNIX_B200_KERNEL_SKINNY_TC:
            if (!skinny_ok(dA, dW, M, K, N)) return TERNIX_B200_ERR_UNSUPPORTED;
            g_last_launched = TERNIX_B200_LAUNCHED_SKINNY_TC;
            return launch_skinny(dA, dW, dC, M, K, N, ldc, d_status, st);
        default:
            g_last_launched = TERNIX_B200_LAUNCHED_GENERIC;
            return launch_generic(dA, dW, dC, M, K, N, ldc, st);
    }
}

int ternix_b200_matmul(const int8_t* dA, const uint8_t* dW, int32_t* dC, int M, int K, int N, void* stream) {
    return ternix_b200_matmul_ex(dA, dW, dC, M, K, N, N, TERNIX_B200_KERNEL_AUTO, nullptr, stream);
}

}  // extern "C"

namespace {
// Streams and events of the pipelined host-pointer call, one set per device, created on first use.  The call holds
// `mu` from start to end: two host threads on one device run one after the other.
struct HostPipe {
    std::mutex mu;
    bool ready = false;
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
    static constexpr int kMaxSlabs = 16;
    cudaEvent_t ev_alloc = nullptr, ev_a = nullptr, ev_done = nullptr, ev_w[kMaxSlabs] = {}, ev_c[kMaxSlabs] = {};
};
int host_pipe(HostPipe** out) {
    static std::mutex mu;
    static HostPipe* pipes[64] = {};
    int dev = 0;
    TB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return TERNIX_B200_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(mu);
    if (!pipes[dev]) pipes[dev] = new HostPipe();
    HostPipe* p = pipes[dev];
    if (!p->ready) {
        TB_CUDA(cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking));
        TB_CUDA(cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking));
        TB_CUDA(cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking));
        cudaEvent_t* singles[] = {&p->ev_alloc, &p->ev_a, &p->ev_done};
        for (cudaEvent_t* e : singles) TB_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
        for (int i = 0; i < HostPipe::kMaxSlabs; ++i) {
            TB_CUDA(cudaEventCreateWithFlags(&p->ev_w[i], cudaEventDisableTiming));
            TB_CUDA(cudaEventCreateWithFlags(&p->ev_c[i], cudaEventDisableTiming));
        }
        p->ready = true;
    }
    *out = p;
    return TERNIX_B200_OK;
}

// Large products through host pointers are bound by the device-to-host copy of C (4 bytes per output against one
// byte per 4 weights in).  This path cuts C into slabs and runs three streams: the inputs of slab j+1 go up while
// slab j is computed and slab j-1 comes down, so that the link carries C from shortly after the shared operand has
// arrived.  Column slabs (by_rows == false) share A and take W slab by slab; W and C of a slab are compact on the
// device and the copies are pitched on the host side.  Row slabs share W and take A slab by slab; every copy is
// contiguous.
// d_w_resident: the packed weights are on the device already (row slabs only): nothing is uploaded but A.
int matmul_host_pipelined(const int8_t* A, const uint8_t* Wp, int32_t* C, int M, int K, int N, int kernel, int slab,
                          bool by_rows, const uint8_t* d_w_resident = nullptr) {
    if (d_w_resident && !by_rows) return TERNIX_B200_ERR_INVALID_ARG;
    HostPipe* hp = nullptr;
    int rc = host_pipe(&hp);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(hp->mu);
    const int extent = by_rows ? M : N;
    // With resident weights nothing but the first slab's activations stands before the first product, so a short first
    // slab (256 rows) lets the download start a few hundred microseconds earlier.
    const int first = (d_w_resident && extent > slab && slab > 256) ? 256 : slab;
    const int n_slabs = 1 + (extent > first ? (extent - first + slab - 1) / slab : 0);
    if (n_slabs > HostPipe::kMaxSlabs) return TERNIX_B200_ERR_INVALID_ARG;
    int start[HostPipe::kMaxSlabs], ext_of[HostPipe::kMaxSlabs];
    for (int j = 0; j < n_slabs; ++j) {
        start[j] = j == 0 ? 0 : first + (j - 1) * slab;
        ext_of[j] = j == 0 ? std::min(first, extent) : std::min(slab, extent - start[j]);
    }
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    // [status | shared operand | per slab: its input, its C]
    const size_t shared_bytes = d_w_resident ? 0 : by_rows ? static_cast<size_t>(K) * (N / 4) : static_cast<size_t>(M) * K;
    size_t off_in[HostPipe::kMaxSlabs], off_c[HostPipe::kMaxSlabs];
    size_t total = 256 + up(shared_bytes);
    for (int j = 0; j < n_slabs; ++j) {
        const size_t ext = static_cast<size_t>(ext_of[j]);
        off_in[j] = total;
        total += up(by_rows ? ext * K : static_cast<size_t>(K) * (ext / 4));
        off_c[j] = total;
        total += up((by_rows ? ext * N : static_cast<size_t>(M) * ext) * sizeof(int32_t));
    }
    cudaMemPool_t pool = nullptr;
    rc = host_call_pool(&pool);
    if (rc) return rc;
    uint8_t* blob = nullptr;
    cudaError_t e = cudaMallocFromPoolAsync(reinterpret_cast<void**>(&blob), total, pool, hp->s_run);
    if (e != cudaSuccess) return cuda_fail(e);
    int32_t* dS = reinterpret_cast<int32_t*>(blob);
    const uint8_t* d_shared = d_w_resident ? d_w_resident : blob + 256;
    int32_t h_status = 0;
    do {
        if ((e = cudaMemsetAsync(dS, 0, 4, hp->s_run)) != cudaSuccess) break;
        if ((e = cudaEventRecord(hp->ev_alloc, hp->s_run)) != cudaSuccess) break;
        if ((e = cudaStreamWaitEvent(hp->s_in, hp->ev_alloc, 0)) != cudaSuccess) break;
        if ((e = cudaStreamWaitEvent(hp->s_out, hp->ev_alloc, 0)) != cudaSuccess) break;
        // up: the first slab's own input, then the shared operand, then the other slabs
        for (int j = 0; j < n_slabs && e == cudaSuccess; ++j) {
            const int x0 = start[j], ext = ext_of[j];
            if (by_rows)
                e = cudaMemcpyAsync(blob + off_in[j], A + static_cast<size_t>(x0) * K, static_cast<size_t>(ext) * K,
                                    cudaMemcpyHostToDevice, hp->s_in);
            else
                e = cudaMemcpy2DAsync(blob + off_in[j], ext / 4, Wp + x0 / 4, N / 4, ext / 4, K, cudaMemcpyHostToDevice,
                                      hp->s_in);
            if (e == cudaSuccess) e = cudaEventRecord(hp->ev_w[j], hp->s_in);
            if (j == 0 && e == cudaSuccess) {
                if (!d_w_resident)
                    e = cudaMemcpyAsync(blob + 256, by_rows ? static_cast<const void*>(Wp) : static_cast<const void*>(A),
                                        shared_bytes, cudaMemcpyHostToDevice, hp->s_in);
                if (e == cudaSuccess) e = cudaEventRecord(hp->ev_a, hp->s_in);
            }
        }
        if (e != cudaSuccess) break;
        if ((e = cudaStreamWaitEvent(hp->s_run, hp->ev_a, 0)) != cudaSuccess) break;
        for (int j = 0; j < n_slabs; ++j) {
            const int x0 = start[j], ext = ext_of[j];
            int32_t* dCj = reinterpret_cast<int32_t*>(blob + off_c[j]);
            if ((e = cudaStreamWaitEvent(hp->s_run, hp->ev_w[j], 0)) != cudaSuccess) break;
            if (by_rows)
                rc = ternix_b200_matmul_ex(reinterpret_cast<const int8_t*>(blob + off_in[j]), d_shared, dCj, ext, K, N, N,
                                           kernel, dS, hp->s_run);
            else
                rc = ternix_b200_matmul_ex(reinterpret_cast<const int8_t*>(blob + 256), blob + off_in[j], dCj, M, K, ext,
                                           ext, kernel, dS, hp->s_run);
            if (rc) break;
            if ((e = cudaEventRecord(hp->ev_c[j], hp->s_run)) != cudaSuccess) break;
            if ((e = cudaStreamWaitEvent(hp->s_out, hp->ev_c[j], 0)) != cudaSuccess) break;
            if (by_rows)
                e = cudaMemcpyAsync(C + static_cast<size_t>(x0) * N, dCj, static_cast<size_t>(ext) * N * 4,
                                    cudaMemcpyDeviceToHost, hp->s_out);
            else
                e = cudaMemcpy2DAsync(C + x0, static_cast<size_t>(N) * 4, dCj, static_cast<size_t>(ext) * 4,
                                      static_cast<size_t>(ext) * 4, M, cudaMemcpyDeviceToHost, hp->s_out);
            if (e != cudaSuccess) break;
        }
        if (e != cudaSuccess || rc) break;
        e = cudaMemcpyAsync(&h_status, dS, 4, cudaMemcpyDeviceToHost, hp->s_out);
    } while (false);
    // Whatever happened above, everything queued so far ends before the block goes back to the pool.
    const cudaError_t e_in = cudaStreamSynchronize(hp->s_in);
    const cudaError_t e_out = cudaStreamSynchronize(hp->s_out);
    cudaFreeAsync(blob, hp->s_run);
    const cudaError_t e_run = cudaStreamSynchronize(hp->s_run);
    if (e == cudaSuccess) e = e_in;
    if (e == cudaSuccess) e = e_out;
    if (e == cudaSuccess) e = e_run;
    if (e != cudaSuccess) return cuda_fail(e);
    if (rc) return rc;
    return h_status ? h_status : TERNIX_B200_OK;
}

// Slab plan of a host-pointer product: the slab extent (0 = single-shot path) and whether slabs are rows.  About
// 64 MB of C per slab, at most 16 slabs.  Column slabs (multiples of 512 columns, at least 4096 wide so that the
// pitched copy of C keeps long rows) are taken when A is the smaller operand to wait for; row slabs (multiples of
// 256 rows) otherwise.  Option host_slab = <columns>, or r<rows>, overrides; 0 switches the pipeline off.
int host_slab_plan(int M, int K, int N, bool* by_rows) {
    *by_rows = false;
    if (K <= 0 || (N % 64) != 0) return 0;
    auto fit = [](long long extent, long long want, long long unit) {
        long long v = std::max(unit, (want + unit - 1) / unit * unit);
        while ((extent + v - 1) / v > HostPipe::kMaxSlabs) v += unit;
        return v >= extent ? 0ll : v;
    };
    const Options& o = options();
    if (o.host_slab >= 0) {
        *by_rows = o.host_slab_rows;
        if (o.host_slab == 0) return 0;
        return static_cast<int>(*by_rows ? fit(M, o.host_slab, 256) : fit(N, o.host_slab, 512));
    }
    const size_t c_bytes = static_cast<size_t>(M) * N * sizeof(int32_t);
    if (c_bytes < (size_t(64) << 20)) return 0;
    const long long slabs = std::min<long long>(HostPipe::kMaxSlabs, std::max<long long>(2, c_bytes / (size_t(64) << 20)));
    const bool a_smaller = static_cast<size_t>(M) * K <= static_cast<size_t>(K) * (N / 4);
    if (a_smaller && N >= 8192) return static_cast<int>(fit(N, std::max<long long>(4096, (N + slabs - 1) / slabs), 512));
    *by_rows = true;
    return static_cast<int>(fit(M, (M + slabs - 1) / slabs, 256));
}
}  // namespace

extern "C" {

int ternix_b200_matmul_host(const int8_t* A, const uint8_t* Wp, int32_t* C, int M, int K, int N, int kernel) {
    if (M < 0 || K < 0 || N < 0 || (N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (kernel < TERNIX_B200_KERNEL_AUTO || kernel > TERNIX_B200_KERNEL_SKINNY_TC) return TERNIX_B200_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return TERNIX_B200_OK;
    if (!C || (K > 0 && (!A || !Wp))) return TERNIX_B200_ERR_INVALID_ARG;
    bool by_rows = false;
    if (const int slab = host_slab_plan(M, K, N, &by_rows)) return matmul_host_pipelined(A, Wp, C, M, K, N, kernel, slab, by_rows);
    const size_t a_bytes = static_cast<size_t>(M) * K, w_bytes = static_cast<size_t>(K) * (N / 4),
                 c_bytes = static_cast<size_t>(M) * N * sizeof(int32_t);
    int8_t* dA = nullptr;
    uint8_t* dW = nullptr;
    int32_t* dC = nullptr;
    int32_t* dS = nullptr;
    int rc = TERNIX_B200_OK;
    cudaError_t e = cudaSuccess;
    int32_t h_status = 0;
    // One allocation for everything: [status | A | W | C], each part 256-byte aligned.  It comes from a
    // stream-ordered pool owned by this library and goes back to it before the call returns; the pool keeps
    // the pages, so repeated calls do not pay the driver's allocation cost again.
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    uint8_t* blob = nullptr;
    const size_t total = 256 + up(a_bytes) + up(w_bytes) + up(c_bytes);
    cudaMemPool_t pool = nullptr;
    rc = host_call_pool(&pool);
    if (rc) return rc;
    if ((e = cudaMallocFromPoolAsync(reinterpret_cast<void**>(&blob), total, pool, 0)) != cudaSuccess) return cuda_fail(e);
    dS = reinterpret_cast<int32_t*>(blob);
    dA = reinterpret_cast<int8_t*>(blob + 256);
    dW = reinterpret_cast<uint8_t*>(blob + 256 + up(a_bytes));
    dC = reinterpret_cast<int32_t*>(blob + 256 + up(a_bytes) + up(w_bytes));
    do {
        if ((e = cudaMemsetAsync(dS, 0, 4, 0)) != cudaSuccess) break;
        if (K > 0) {
            if ((e = cudaMemcpyAsync(dA, A, a_bytes, cudaMemcpyHostToDevice, 0)) != cudaSuccess) break;
            if ((e = cudaMemcpyAsync(dW, Wp, w_bytes, cudaMemcpyHostToDevice, 0)) != cudaSuccess) break;
        }
        rc = ternix_b200_matmul_ex(dA, dW, dC, M, K, N, N, kernel, dS, nullptr);
        if (rc) break;
        if ((e = cudaMemcpyAsync(C, dC, c_bytes, cudaMemcpyDeviceToHost, 0)) != cudaSuccess) break;
        if ((e = cudaMemcpyAsync(&h_status, dS, 4, cudaMemcpyDeviceToHost, 0)) != cudaSuccess) break;
    } while (false);
    cudaFreeAsync(blob, 0);
    const cudaError_t e_sync = cudaStreamSynchronize(0);
    if (e == cudaSuccess) e = e_sync;
    if (e != cudaSuccess) return cuda_fail(e);
    if (rc) return rc;
    return h_status ? h_status : TERNIX_B200_OK;
}

int ternix_b200_shard_columns(int N, int world, int rank, int granule, int* n0, int* n_cols) {
    if (N < 0 || (N % 4) != 0 || world < 1 || rank < 0 || rank >= world || granule < 4 || (granule % 4) != 0 ||
        !n0 || !n_cols)
        return TERNIX_B200_ERR_INVALID_ARG;
    const int granules = (N + granule - 1) / granule;
    const int base = granules / world, extra = granules % world;
    const int first = rank < extra ? rank * (base + 1) : extra * (base + 1) + (rank - extra) * base;
    const int count = rank < extra ? base + 1 : base;
    long long c0 = static_cast<long long>(first) * granule, c1 = static_cast<long long>(first + count) * granule;
    if (c0 > N) c0 = N;
    if (c1 > N) c1 = N;
    *n0 = static_cast<int>(c0);
    *n_cols = static_cast<int>(c1 - c0);
    return TERNIX_B200_OK;
}

int ternix_b200_unpack_gathered(const int32_t* d_gathered, int32_t* dC, int M, int N, long long ldc, int world,
                                int granule, int n_pad, void* stream) {
    if (M < 0 || N < 0 || (N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (world < 1 || granule < 4 || (granule % 4) != 0 || ldc < N || n_pad < 0) return TERNIX_B200_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return TERNIX_B200_OK;
    if (!d_gathered || !dC) return TERNIX_B200_ERR_INVALID_ARG;
    const long long total = static_cast<long long>(M) * N;
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    unpack_gathered_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        d_gathered, dC, M, N, ldc, world, granule, n_pad);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

static int group_create_impl(ternix_b200_group** out, const ternix_b200_problem* problems, int count,
                             int32_t* const* peer_dC, int n_peers, bool prepacked) {
    if (!out || count < 0 || (count > 0 && !problems)) return TERNIX_B200_ERR_INVALID_ARG;
    if (n_peers < 0 || n_peers >= tb200::kTc2MaxDest || (n_peers > 0 && !peer_dC)) return TERNIX_B200_ERR_INVALID_ARG;
    *out = nullptr;
    for (int i = 0; i < count; ++i) {
        const ternix_b200_problem& q = problems[i];
        if (q.M < 0 || q.K < 0 || q.N < 0 || (q.N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
        if (q.ldc < q.N) return TERNIX_B200_ERR_INVALID_ARG;
        if (q.M > 0 && q.N > 0 && (!q.dC || (q.K > 0 && (!q.dA || !q.dW)))) return TERNIX_B200_ERR_INVALID_ARG;
    }
    ternix_b200_group* g = new (std::nothrow) ternix_b200_group();
    if (!g) return TERNIX_B200_ERR_INVALID_ARG;
    if (cudaGetDevice(&g->device) != cudaSuccess) g->device = 0;

    // Item width: 256 columns (64-byte rows) when every decode member has one row: the finer items balance better
    // over the SMs (measured +1..4 %); 512 columns (128-byte rows) for row groups, where the wider item wins.
    // Option group_words = 16|32 overrides.
    g->prepacked = prepacked;
    const Options& opt = options();
    // rows below this stay with the dp4a kernel: the batched-decode kernels take over from their first row count
    const int decode_rows_end = opt.skinny_group_lo > 0 ? std::min(kGroupMmaMinRows, opt.skinny_group_lo) : kGroupMmaMinRows;
    int decode_max_m = 0;
    for (int i = 0; i < count; ++i)
        if (problems[i].M > 0 && problems[i].N > 0 && group_gemv_ok(problems[i]) &&
            !(problems[i].K > 0 && gemm_tc2_ok(problems[i].dA, problems[i].dW, problems[i].M, problems[i].K, problems[i].N)))
            if (prepacked || problems[i].M < decode_rows_end) decode_max_m = std::max(decode_max_m, problems[i].M);
    g->words = (!prepacked && decode_max_m == 1) ? 16 : 32;
    if (options().group_words) g->words = (!prepacked && options().group_words == 16) ? 16 : 32;
    const int item_cols = g->words * 16;
    std::vector<tb200::Tc2Problem> tc_probs;
    std::vector<tb200::Tc3Problem> tc3_probs;
    bool tc3_group = options().tc3 != 0;                  // option tc3 = 0: the expanding kernel
    std::vector<tb200::MmaProblem> mma_probs[2];          // row groups of 8, of 16
    std::vector<tb200::SkProblem> sk_probs[4];            // batch classes 16, 32, 64, 128
    std::vector<tb200::GroupProblem> probs;
    struct HostItem { tb200::GroupItem item; long cost; };
    std::vector<HostItem> items;
    int max_m = 0;
    for (int i = 0; i < count; ++i) {
        const ternix_b200_problem& q = problems[i];
        if (q.M == 0 || q.N == 0) continue;
        if (prepacked && !group_gemv_ok(q)) { delete g; return TERNIX_B200_ERR_UNSUPPORTED; }   // decode members only
        if (!prepacked && q.K > 0 && gemm_tc2_ok(q.dA, q.dW, q.M, q.K, q.N)) {
            tb200::Tc2Problem tp{};
            int rc = make_tmap_2d(&tp.tmap_a, q.dA, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.M),
                                  static_cast<uint64_t>(q.K), tb200::kTcBK, tb200::kTcBM, CU_TENSOR_MAP_SWIZZLE_128B);
            if (!rc)
                rc = make_tmap_2d(&tp.tmap_w, q.dW, static_cast<uint64_t>(q.N / 4), static_cast<uint64_t>(q.K),
                                  static_cast<uint64_t>(q.N / 4), tb200::Tc2Geom::kWpRowBytes, tb200::kTcBK,
                                  CU_TENSOR_MAP_SWIZZLE_NONE);
            if (rc) { delete g; return rc; }
            tp.dest.count = 1 + n_peers;
            tp.dest.c[0] = q.dC;
            tp.c_vec_ok = (q.ldc % 4 == 0) && aligned(q.dC, 16);
            for (int j = 0; j < n_peers; ++j) {
                int32_t* p = peer_dC[static_cast<size_t>(i) * n_peers + j];
                if (!p) { delete g; return TERNIX_B200_ERR_INVALID_ARG; }
                tp.dest.c[1 + j] = p;
                tp.c_vec_ok = tp.c_vec_ok && aligned(p, 16);
            }
            tp.ldc = q.ldc; tp.M = q.M; tp.K = q.K; tp.N = q.N;
            tc_probs.push_back(tp);
            // the same member for the kernel that keeps decoded weights in tensor memory (needs TMA views of every C)
            if (tc3_group && tp.c_vec_ok) {
                tb200::Tc3Problem t3{};
                rc = make_tmap_2d(&t3.tmap_a, q.dA, static_cast<uint64_t>(q.K), static_cast<uint64_t>(q.M),
                                  static_cast<uint64_t>(q.K), tb200::kTcBK, 128, CU_TENSOR_MAP_SWIZZLE_128B);
                if (!rc)
                    rc = make_tmap_2d(&t3.tmap_w, q.dW, static_cast<uint64_t>(q.N / 4), static_cast<uint64_t>(q.K),
                                      static_cast<uint64_t>(q.N / 4), tb200::kTc3WpRowBytes, tb200::kTc3BK,
                                      CU_TENSOR_MAP_SWIZZLE_32B);
                t3.stores.count = tp.dest.count;
                for (int d = 0; !rc && d < tp.dest.count; ++d)
                    rc = make_tmap_2d_u32(&t3.stores.tmap_c[d], tp.dest.c[d], static_cast<uint64_t>(q.N),
                                          static_cast<uint64_t>(q.M), static_cast<uint64_t>(q.ldc) * 4, 128, 32);
                if (rc) { delete g; return rc; }
                t3.C = q.dC; t3.ldc = q.ldc; t3.M = q.M; t3.K = q.K; t3.N = q.N;
                tc3_probs.push_back(t3);
            } else {
                tc3_group = false;
            }
            ++g->tc_grouped;
            continue;
        }
        if (n_peers > 0) {           // not a paired-GEMM member: run it as usual, then copy its C to the peers
            ternix_b200_group::PeerCopy pc{q, {}};
            for (int j = 0; j < n_peers; ++j) pc.peers.push_back(peer_dC[static_cast<size_t>(i) * n_peers + j]);
            g->single_peers.push_back(pc);
        }
        if (!prepacked && opt.skinny_group_lo > 0 && q.M >= opt.skinny_group_lo && q.M <= opt.skinny_group_hi && q.K > 0 &&
            skinny_ok(q.dA, q.dW, q.M, q.K, q.N)) {
            tb200::SkProblem sp;
            const int rc = make_skinny_problem(&sp, q.dA, q.dW, q.dC, q.M, q.K, q.N, q.ldc);
            if (rc) { delete g; return rc; }
            sk_probs[q.M <= 16 ? 0 : q.M <= 32 ? 1 : q.M <= 64 ? 2 : 3].push_back(sp);
            ++g->sk_grouped;
            continue;
        }
        if (!prepacked && q.M >= kGroupMmaMinRows && q.M <= kGroupMmaMaxRows && q.K > 0 && q.ldc >= q.N &&
            decode_mma_ok(q.dA, q.dW, q.M, q.K, q.N)) {
            tb200::MmaProblem mp;
            const int rc = make_mma_problem(&mp, q.dA, q.dW, q.dC, q.M, q.K, q.N, q.ldc);
            if (rc) { delete g; return rc; }
            mma_probs[q.M <= 8 ? 0 : 1].push_back(mp);
            ++g->mma_grouped;
            continue;
        }
        if (!group_gemv_ok(q)) { g->singles.push_back(q); continue; }
        tb200::GroupProblem gp{};
        const int rc = prepacked
            ? make_tmap_2d_u32(&gp.tmap_w, q.dW, static_cast<uint64_t>(q.N / 4), static_cast<uint64_t>((q.K + 3) / 4),
                               static_cast<uint64_t>(q.N), 128, tb200::group_stage_rows(32) / 4)
            : make_tmap_2d(&gp.tmap_w, q.dW, static_cast<uint64_t>(q.N / 4), static_cast<uint64_t>(q.K),
                           static_cast<uint64_t>(q.N / 4), g->words * 4, tb200::group_stage_rows(g->words),
                           g->words == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
        if (rc) { delete g; return rc; }
        gp.A = q.dA; gp.C = q.dC; gp.ldc = q.ldc; gp.M = q.M; gp.K = q.K; gp.N = q.N;
        const int pi = static_cast<int>(probs.size());
        probs.push_back(gp);
        max_m = std::max(max_m, q.M);
        ++g->grouped;
    }
    g->mr = max_m <= 1 ? 1 : max_m <= 2 ? 2 : 4;
    for (int pi = 0; pi < static_cast<int>(probs.size()); ++pi) {
        const tb200::GroupProblem& gp = probs[pi];
        const int chunks = (gp.N + item_cols - 1) / item_cols;
        for (int row0 = 0; row0 < gp.M; row0 += g->mr)
            for (int c = 0; c < chunks; ++c) items.push_back({{pi, c, row0, 0}, static_cast<long>(gp.K) + 256});
    }
    if (!items.empty()) {
        // longest-processing-time-first: heaviest items first, each to the least-loaded CTA
        const int per_sm = tb200::group_ctas_per_sm(g->mr);
        const int ctas = static_cast<int>(std::min<size_t>(items.size(), static_cast<size_t>(sm_count()) * per_sm));
        std::stable_sort(items.begin(), items.end(), [](const HostItem& a, const HostItem& b) { return a.cost > b.cost; });
        using Load = std::pair<long, int>;
        std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
        for (int c = 0; c < ctas; ++c) heap.push({0, c});
        std::vector<std::vector<tb200::GroupItem>> per_cta(ctas);
        for (const HostItem& h : items) {
            Load l = heap.top();
            heap.pop();
            per_cta[l.second].push_back(h.item);
            heap.push({l.first + h.cost, l.second});
        }
        std::vector<tb200::GroupItem> flat;
        std::vector<int> first(ctas + 1, 0);
        for (int c = 0; c < ctas; ++c) {
            first[c] = static_cast<int>(flat.size());
            flat.insert(flat.end(), per_cta[c].begin(), per_cta[c].end());
        }
        first[ctas] = static_cast<int>(flat.size());
        const size_t b_probs = probs.size() * sizeof(tb200::GroupProblem);
        const size_t b_items = (flat.size() * sizeof(tb200::GroupItem) + 63) & ~size_t(63);
        const size_t b_first = first.size() * sizeof(int);
        cudaError_t e = cudaMalloc(&g->d_blob, b_probs + b_items + b_first);
        if (e != cudaSuccess) { delete g; return cuda_fail(e); }
        uint8_t* d = static_cast<uint8_t*>(g->d_blob);
        if ((e = cudaMemcpy(d, probs.data(), b_probs, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(d + b_probs, flat.data(), flat.size() * sizeof(tb200::GroupItem), cudaMemcpyHostToDevice)) !=
                cudaSuccess ||
            (e = cudaMemcpy(d + b_probs + b_items, first.data(), b_first, cudaMemcpyHostToDevice)) != cudaSuccess) {
            cudaFree(g->d_blob);
            delete g;
            return cuda_fail(e);
        }
        g->d_probs = reinterpret_cast<const tb200::GroupProblem*>(d);
        g->d_items = reinterpret_cast<const tb200::GroupItem*>(d + b_probs);
        g->d_cta_first = reinterpret_cast<const int*>(d + b_probs + b_items);
        g->grid = ctas;
        g->short_launch = flat.size() <= static_cast<size_t>(4) * ctas;
    }
    if (!tc_probs.empty()) {
        // tiles of all prefill members, heaviest (deepest K) first, each to the least-loaded CTA pair
        struct HostTile { tb200::Tc2Tile tile; long cost; };
        std::vector<HostTile> tl;
        for (int pi = 0; pi < static_cast<int>(tc_probs.size()); ++pi) {
            const tb200::Tc2Problem& tp = tc_probs[pi];
            const int m_tiles = (tp.M + 255) / 256, n_tiles = (tp.N + 255) / 256;
            const long kb = (tp.K + tb200::kTcBK - 1) / tb200::kTcBK;
            for (int n_t = 0; n_t < n_tiles; ++n_t)
                for (int m_t = 0; m_t < m_tiles; ++m_t) tl.push_back({{pi, m_t, n_t, 0}, kb + 2});
        }
        const int pairs = static_cast<int>(std::min<size_t>(tl.size(), static_cast<size_t>(sm_count() / 2)));
        std::stable_sort(tl.begin(), tl.end(), [](const HostTile& a, const HostTile& b) { return a.cost > b.cost; });
        using Load = std::pair<long, int>;
        std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
        for (int c = 0; c < pairs; ++c) heap.push({0, c});
        std::vector<std::vector<tb200::Tc2Tile>> per_pair(pairs);
        for (const HostTile& h : tl) {
            Load l = heap.top();
            heap.pop();
            per_pair[l.second].push_back(h.tile);
            heap.push({l.first + h.cost, l.second});
        }
        std::vector<tb200::Tc2Tile> flat;
        std::vector<int> first(pairs + 1, 0);
        for (int c = 0; c < pairs; ++c) {
            first[c] = static_cast<int>(flat.size());
            flat.insert(flat.end(), per_pair[c].begin(), per_pair[c].end());
        }
        first[pairs] = static_cast<int>(flat.size());
        const bool use_tc3 = tc3_group && tc3_probs.size() == tc_probs.size();
        const size_t b_probs = use_tc3 ? tc3_probs.size() * sizeof(tb200::Tc3Problem) : tc_probs.size() * sizeof(tb200::Tc2Problem);
        const void* h_probs = use_tc3 ? static_cast<const void*>(tc3_probs.data()) : static_cast<const void*>(tc_probs.data());
        const size_t b_tiles = (flat.size() * sizeof(tb200::Tc2Tile) + 63) & ~size_t(63);
        const size_t b_first = first.size() * sizeof(int);
        cudaError_t e = cudaMalloc(&g->d_tc_blob, b_probs + b_tiles + b_first);
        if (e != cudaSuccess) { ternix_b200_group_destroy(g); return cuda_fail(e); }
        uint8_t* d = static_cast<uint8_t*>(g->d_tc_blob);
        if ((e = cudaMemcpy(d, h_probs, b_probs, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(d + b_probs, flat.data(), flat.size() * sizeof(tb200::Tc2Tile), cudaMemcpyHostToDevice)) !=
                cudaSuccess ||
            (e = cudaMemcpy(d + b_probs + b_tiles, first.data(), b_first, cudaMemcpyHostToDevice)) != cudaSuccess) {
            ternix_b200_group_destroy(g);
            return cuda_fail(e);
        }
        if (use_tc3) g->d_tc3_probs = reinterpret_cast<const tb200::Tc3Problem*>(d);
        else g->d_tc_probs = reinterpret_cast<const tb200::Tc2Problem*>(d);
        g->d_tc_tiles = reinterpret_cast<const tb200::Tc2Tile*>(d + b_probs);
        g->d_tc_first = reinterpret_cast<const int*>(d + b_probs + b_tiles);
        g->tc_pairs = pairs;
    }
    for (int v = 0; v < 2; ++v) {
        if (mma_probs[v].empty()) continue;
        // whole-K items, deepest K first, each to the least-loaded CTA: with equal costs this deals the items out in
        // order, so that neighbouring CTAs read the same weight rows of neighbouring chunks at the same time
        const int group_rows = v == 0 ? 8 : 16;
        struct HostMmaItem { tb200::MmaItem item; long cost; };
        std::vector<HostMmaItem> hi;
        for (int pi = 0; pi < static_cast<int>(mma_probs[v].size()); ++pi) {
            const tb200::MmaProblem& mp = mma_probs[v][pi];
            const int chunks = (mp.N + tb200::kMmaItemCols - 1) / tb200::kMmaItemCols;
            for (int row0 = 0; row0 < mp.M; row0 += group_rows)
                for (int c = 0; c < chunks; ++c) hi.push_back({{pi, c, row0, 0}, static_cast<long>(mp.K) + 256});
        }
        const int ctas = static_cast<int>(std::min<size_t>(hi.size(), static_cast<size_t>(sm_count()) * tb200::kMmaCtasPerSm));
        std::stable_sort(hi.begin(), hi.end(), [](const HostMmaItem& a, const HostMmaItem& b) { return a.cost > b.cost; });
        using Load = std::pair<long, int>;
        std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
        for (int c = 0; c < ctas; ++c) heap.push({0, c});
        std::vector<std::vector<tb200::MmaItem>> per_cta(ctas);
        for (const HostMmaItem& h : hi) {
            Load l = heap.top();
            heap.pop();
            per_cta[l.second].push_back(h.item);
            heap.push({l.first + h.cost, l.second});
        }
        std::vector<tb200::MmaItem> flat;
        std::vector<int> first(ctas + 1, 0);
        for (int c = 0; c < ctas; ++c) {
            first[c] = static_cast<int>(flat.size());
            flat.insert(flat.end(), per_cta[c].begin(), per_cta[c].end());
        }
        first[ctas] = static_cast<int>(flat.size());
        const size_t b_probs = mma_probs[v].size() * sizeof(tb200::MmaProblem);
        const size_t b_items = (flat.size() * sizeof(tb200::MmaItem) + 63) & ~size_t(63);
        const size_t b_first = first.size() * sizeof(int);
        auto& mt = g->mma[v];
        cudaError_t e = cudaMalloc(&mt.d_blob, b_probs + b_items + b_first);
        if (e != cudaSuccess) { ternix_b200_group_destroy(g); return cuda_fail(e); }
        uint8_t* d = static_cast<uint8_t*>(mt.d_blob);
        if ((e = cudaMemcpy(d, mma_probs[v].data(), b_probs, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(d + b_probs, flat.data(), flat.size() * sizeof(tb200::MmaItem), cudaMemcpyHostToDevice)) !=
                cudaSuccess ||
            (e = cudaMemcpy(d + b_probs + b_items, first.data(), b_first, cudaMemcpyHostToDevice)) != cudaSuccess) {
            ternix_b200_group_destroy(g);
            return cuda_fail(e);
        }
        mt.d_probs = reinterpret_cast<const tb200::MmaProblem*>(d);
        mt.d_items = reinterpret_cast<const tb200::MmaItem*>(d + b_probs);
        mt.d_first = reinterpret_cast<const int*>(d + b_probs + b_items);
        mt.grid = ctas;
    }
    for (int v = 0; v < 4; ++v) {
        if (sk_probs[v].empty()) continue;
        // whole-K items of 256 columns in (problem, block) order, dealt out to the least-loaded CTA: with equal costs
        // neighbouring CTAs stream neighbouring blocks of the same weight rows at the same time
        struct HostSkItem { tb200::SkItem item; long cost; };
        std::vector<HostSkItem> hi;
        for (int pi = 0; pi < static_cast<int>(sk_probs[v].size()); ++pi) {
            const tb200::SkProblem& sp = sk_probs[v][pi];
            const int blocks = (sp.N + tb200::kSkItemCols - 1) / tb200::kSkItemCols;
            for (int b = 0; b < blocks; ++b) hi.push_back({{pi, b}, static_cast<long>(sp.K) + 256});
        }
        const int ctas = static_cast<int>(std::min<size_t>(hi.size(), static_cast<size_t>(sm_count())));
        std::stable_sort(hi.begin(), hi.end(), [](const HostSkItem& a, const HostSkItem& b) { return a.cost > b.cost; });
        using Load = std::pair<long, int>;
        std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
        for (int c = 0; c < ctas; ++c) heap.push({0, c});
        std::vector<std::vector<tb200::SkItem>> per_cta(ctas);
        for (const HostSkItem& h : hi) {
            Load l = heap.top();
            heap.pop();
            per_cta[l.second].push_back(h.item);
            heap.push({l.first + h.cost, l.second});
        }
        std::vector<tb200::SkItem> flat;
        std::vector<int> first(ctas + 1, 0);
        for (int c = 0; c < ctas; ++c) {
            first[c] = static_cast<int>(flat.size());
            flat.insert(flat.end(), per_cta[c].begin(), per_cta[c].end());
        }
        first[ctas] = static_cast<int>(flat.size());
        const size_t b_probs = sk_probs[v].size() * sizeof(tb200::SkProblem);
        const size_t b_items = (flat.size() * sizeof(tb200::SkItem) + 63) & ~size_t(63);
        const size_t b_first = first.size() * sizeof(int);
        auto& t = g->sk[v];
        cudaError_t e = cudaMalloc(&t.d_blob, b_probs + b_items + b_first);
        if (e != cudaSuccess) { ternix_b200_group_destroy(g); return cuda_fail(e); }
        uint8_t* d = static_cast<uint8_t*>(t.d_blob);
        if ((e = cudaMemcpy(d, sk_probs[v].data(), b_probs, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(d + b_probs, flat.data(), flat.size() * sizeof(tb200::SkItem), cudaMemcpyHostToDevice)) !=
                cudaSuccess ||
            (e = cudaMemcpy(d + b_probs + b_items, first.data(), b_first, cudaMemcpyHostToDevice)) != cudaSuccess) {
            ternix_b200_group_destroy(g);
            return cuda_fail(e);
        }
        t.d_probs = reinterpret_cast<const tb200::SkProblem*>(d);
        t.d_items = reinterpret_cast<const tb200::SkItem*>(d + b_probs);
        t.d_first = reinterpret_cast<const int*>(d + b_probs + b_items);
        t.grid = ctas;
    }
    *out = g;
    return TERNIX_B200_OK;
}

int ternix_b200_group_create_ex(ternix_b200_group** out, const ternix_b200_problem* problems, int count,
                                int32_t* const* peer_dC, int n_peers) {
    return group_create_impl(out, problems, count, peer_dC, n_peers, false);
}

int ternix_b200_group_create(ternix_b200_group** out, const ternix_b200_problem* problems, int count) {
    return group_create_impl(out, problems, count, nullptr, 0, false);
}

int ternix_b200_group_create_prepacked(ternix_b200_group** out, const ternix_b200_problem* problems, int count) {
    return group_create_impl(out, problems, count, nullptr, 0, true);
}

size_t ternix_b200_prepack_k4_bytes(int K, int N) {
    if (K < 0 || N < 0 || (N % 4) != 0) return 0;
    return static_cast<size_t>((K + 3) / 4) * static_cast<size_t>(N);
}

int ternix_b200_prepack_k4(const uint8_t* dW, uint8_t* dW_prepacked, int K, int N, void* stream) {
    if (K < 0 || N < 0 || (N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (K == 0 || N == 0) return TERNIX_B200_OK;
    if (!dW || !dW_prepacked || !aligned(dW_prepacked, 16)) return TERNIX_B200_ERR_INVALID_ARG;
    const long long total = static_cast<long long>((K + 3) / 4) * (N / 4);
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    tb200::prepack_k4_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        dW, reinterpret_cast<uint32_t*>(dW_prepacked), K, N / 4);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}



int ternix_b200_group_run(const ternix_b200_group* g, int32_t* d_status, void* stream) {
    if (!g) return TERNIX_B200_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g->grid > 0) {
        int rc;
        if (g->prepacked) {
            if (g->mr == 1) rc = launch_gemv_group_t<1, 32, true>(g, d_status, st);
            else if (g->mr == 2) rc = launch_gemv_group_t<2, 32, true>(g, d_status, st);
            else rc = launch_gemv_group_t<4, 32, true>(g, d_status, st);
        } else if (g->words == 32) {
            if (g->mr == 1) rc = launch_gemv_group_t<1, 32>(g, d_status, st);
            else if (g->mr == 2) rc = launch_gemv_group_t<2, 32>(g, d_status, st);
            else rc = launch_gemv_group_t<4, 32>(g, d_status, st);
        } else {
            if (g->mr == 1) rc = launch_gemv_group_t<1, 16>(g, d_status, st);
            else if (g->mr == 2) rc = launch_gemv_group_t<2, 16>(g, d_status, st);
            else rc = launch_gemv_group_t<4, 16>(g, d_status, st);
        }
        if (rc) return rc;
    }
    if (g->tc_pairs > 0) {
        const int rc = launch_gemm_tc2_group(g, d_status, st);
        if (rc) return rc;
    }
    for (int v = 0; v < 2; ++v) {
        const auto& mt = g->mma[v];
        if (mt.grid == 0) continue;
        int rc = v == 0 ? decode_mma_attr<false, 1>() : decode_mma_attr<false, 2>();
        if (rc) return rc;
        const tb200::MmaProblem none{};
        const tb200::MmaSingle sg{};
        if (v == 0)
            tb200::ternary_decode_mma_kernel<false, 1><<<mt.grid, tb200::kMmaThreads, tb200::kMmaSmemBytes, st>>>(
                none, sg, mt.d_probs, mt.d_items, mt.d_first, d_status);
        else
            tb200::ternary_decode_mma_kernel<false, 2><<<mt.grid, tb200::kMmaThreads, tb200::kMmaSmemBytes, st>>>(
                none, sg, mt.d_probs, mt.d_items, mt.d_first, d_status);
        TB_CUDA(cudaGetLastError());
    }
    for (int v = 0; v < 4; ++v) {
        const auto& t = g->sk[v];
        if (t.grid == 0) continue;
        const tb200::SkProblem none{};
        const tb200::SkSingle sg{};
        int rc;
        if (v == 0) rc = launch_skinny_t<16, true>(none, sg, t.d_probs, t.d_items, t.d_first, t.grid, nullptr, 0, d_status, st);
        else if (v == 1) rc = launch_skinny_t<32, true>(none, sg, t.d_probs, t.d_items, t.d_first, t.grid, nullptr, 0, d_status, st);
        else if (v == 2) rc = launch_skinny_t<64, true>(none, sg, t.d_probs, t.d_items, t.d_first, t.grid, nullptr, 0, d_status, st);
        else rc = launch_skinny_t<128, true>(none, sg, t.d_probs, t.d_items, t.d_first, t.grid, nullptr, 0, d_status, st);
        if (rc) return rc;
    }
    for (const ternix_b200_problem& q : g->singles) {
        const int rc = ternix_b200_matmul_ex(q.dA, q.dW, q.dC, q.M, q.K, q.N, q.ldc, TERNIX_B200_KERNEL_AUTO, d_status,
                                             stream);
        if (rc) return rc;
    }
    for (const auto& pc : g->single_peers)
        for (int32_t* peer : pc.peers)
            TB_CUDA(cudaMemcpy2DAsync(peer, static_cast<size_t>(pc.q.ldc) * 4, pc.q.dC, static_cast<size_t>(pc.q.ldc) * 4,
                                      static_cast<size_t>(pc.q.N) * 4, pc.q.M, cudaMemcpyDefault, st));
    return TERNIX_B200_OK;
}

int ternix_b200_group_launches(const ternix_b200_group* g) {
    if (!g) return 0;
    int n = (g->grid > 0 ? 1 : 0) + (g->tc_pairs > 0 ? 1 : 0) + static_cast<int>(g->singles.size());
    for (const auto& mt : g->mma) n += mt.grid > 0 ? 1 : 0;
    for (const auto& t : g->sk) n += t.grid > 0 ? 1 : 0;
    return n;
}

void ternix_b200_group_destroy(ternix_b200_group* g) {
    if (!g) return;
    if (g->d_blob) cudaFree(g->d_blob);
    if (g->d_tc_blob) cudaFree(g->d_tc_blob);
    for (auto& mt : g->mma)
        if (mt.d_blob) cudaFree(mt.d_blob);
    for (auto& t : g->sk)
        if (t.d_blob) cudaFree(t.d_blob);
    delete g;
}

int ternix_b200_matmul_bcast(const int8_t* dA, const uint8_t* dW, int32_t* const* dC_list, int n_dest, int M, int K,
                             int N, long long ldc, int32_t* d_status, void* stream) {
    if (M < 0 || K < 0 || N < 0 || (N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (ldc < N || n_dest < 1 || n_dest > tb200::kTc2MaxDest || !dC_list) return TERNIX_B200_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return TERNIX_B200_OK;
    for (int d = 0; d < n_dest; ++d)
        if (!dC_list[d]) return TERNIX_B200_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K > 0 && dA && dW && gemm_tc2_ok(dA, dW, M, K, N))
        return launch_gemm_tc2(dA, dW, dC_list, n_dest, M, K, N, ldc, d_status, st, &g_last_launched);
    // Any other problem: compute into the first destination, then copy it to the others.
    const int rc = ternix_b200_matmul_ex(dA, dW, dC_list[0], M, K, N, ldc, TERNIX_B200_KERNEL_AUTO, d_status, stream);
    if (rc) return rc;
    for (int d = 1; d < n_dest; ++d)
        TB_CUDA(cudaMemcpy2DAsync(dC_list[d], static_cast<size_t>(ldc) * 4, dC_list[0], static_cast<size_t>(ldc) * 4,
                                  static_cast<size_t>(N) * 4, M, cudaMemcpyDefault, st));
    return TERNIX_B200_OK;
}

int ternix_b200_peer_alloc(void** dptr, size_t bytes) {
    if (!dptr) return TERNIX_B200_ERR_INVALID_ARG;
    TB_CUDA(cudaMalloc(dptr, bytes ? bytes : 1));
    return TERNIX_B200_OK;
}
int ternix_b200_peer_free(void* dptr) {
    TB_CUDA(cudaFree(dptr));
    return TERNIX_B200_OK;
}
int ternix_b200_peer_export(void* dptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!dptr || !handle) return TERNIX_B200_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    TB_CUDA(cudaIpcGetMemHandle(&h, dptr));
    std::memcpy(handle, &h, 64);
    return TERNIX_B200_OK;
}
int ternix_b200_peer_import(const unsigned char handle[64], void** dptr) {
    if (!dptr || !handle) return TERNIX_B200_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    TB_CUDA(cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
    return TERNIX_B200_OK;
}
int ternix_b200_peer_close(void* dptr) {
    TB_CUDA(cudaIpcCloseMemHandle(dptr));
    return TERNIX_B200_OK;
}

int ternix_b200_gemv_batch_noalloc(const ternix_b200_problem* problems, int count, int32_t* d_status, void* stream) {
    if (count < 0 || (count > 0 && !problems)) return TERNIX_B200_ERR_INVALID_ARG;
    if (count > kNoAllocMaxProblems) return TERNIX_B200_ERR_TOO_LARGE;
    for (int i = 0; i < count; ++i) {
        const ternix_b200_problem& q = problems[i];
        if (q.M < 0 || q.K < 0 || q.N < 0 || (q.N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
        if (q.ldc < q.N) return TERNIX_B200_ERR_INVALID_ARG;
        if (q.M == 0 || q.N == 0) continue;
        if (!q.dC || (q.K > 0 && (!q.dA || !q.dW))) return TERNIX_B200_ERR_INVALID_ARG;
        if (q.K > 0 && !group_gemv_ok(q)) return TERNIX_B200_ERR_UNSUPPORTED;     // decode-regime problems only
    }
    // The tables are staged in one fixed host buffer and uploaded with asynchronous copies.  A captured call would
    // record copies that read that buffer when the graph runs, after later calls have rewritten it: refuse.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    TB_CUDA(cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &capturing));
    if (capturing != cudaStreamCaptureStatusNone) return TERNIX_B200_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);     // one caller at a time builds, copies and launches
    unsigned char* d_scratch = nullptr;
    int rc = noalloc_scratch_for_current_device(&d_scratch);
    if (rc) return rc;
    NoAllocHostTables& h = g_noalloc_host;
    const int words = 32, item_cols = words * 16;
    int n_probs = 0, max_m = 0;
    for (int i = 0; i < count; ++i) {
        const ternix_b200_problem& q = problems[i];
        if (q.M == 0 || q.N == 0) continue;
        if (q.K == 0) {        // empty sum: C = 0, as the single-product entry points do (a memset allocates nothing)
            TB_CUDA(cudaMemset2DAsync(q.dC, static_cast<size_t>(q.ldc) * 4, 0, static_cast<size_t>(q.N) * 4, q.M,
                                      static_cast<cudaStream_t>(stream)));
            continue;
        }
        tb200::GroupProblem& gp = h.probs[n_probs];
        gp = tb200::GroupProblem{};
        rc = make_tmap_2d(&gp.tmap_w, q.dW, static_cast<uint64_t>(q.N / 4), static_cast<uint64_t>(q.K),
                          static_cast<uint64_t>(q.N / 4), words * 4, tb200::group_stage_rows(words),
                          CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        gp.A = q.dA; gp.C = q.dC; gp.ldc = q.ldc; gp.M = q.M; gp.K = q.K; gp.N = q.N;
        max_m = std::max(max_m, q.M);
        ++n_probs;
    }
    if (n_probs == 0) return TERNIX_B200_OK;
    const int mr = max_m <= 1 ? 1 : max_m <= 2 ? 2 : 4;
    int n_items = 0;
    for (int pi = 0; pi < n_probs; ++pi) {
        const tb200::GroupProblem& gp = h.probs[pi];
        const int chunks = (gp.N + item_cols - 1) / item_cols;
        for (int row0 = 0; row0 < gp.M; row0 += mr)
            for (int c = 0; c < chunks; ++c) {
                if (n_items == kNoAllocMaxItems) return TERNIX_B200_ERR_TOO_LARGE;
                h.pending[n_items++] = tb200::GroupItem{pi, c, row0, gp.K};     // pad carries the cost (K)
            }
    }
    // heaviest first (ties by problem, chunk, row so the plan is deterministic), each to the least-loaded CTA
    std::sort(h.pending, h.pending + n_items, [](const tb200::GroupItem& x, const tb200::GroupItem& y) {
        if (x.pad != y.pad) return x.pad > y.pad;
        if (x.problem != y.problem) return x.problem < y.problem;
        if (x.chunk != y.chunk) return x.chunk < y.chunk;
        return x.row0 < y.row0;
    });
    const int per_sm = tb200::group_ctas_per_sm(mr);
    int ctas = std::min(n_items, sm_count() * per_sm);
    ctas = std::min(ctas, kNoAllocMaxCtas);
    for (int c = 0; c <= ctas; ++c) h.first[c] = 0;
    for (int c = 0; c < ctas; ++c) h.load[c] = 0;
    for (int i = 0; i < n_items; ++i) {
        int best = 0;
        for (int c = 1; c < ctas; ++c)
            if (h.load[c] < h.load[best]) best = c;
        h.cta_of[i] = static_cast<unsigned short>(best);
        h.load[best] += h.pending[i].pad + 256;
        ++h.first[best + 1];
    }
    for (int c = 0; c < ctas; ++c) h.first[c + 1] += h.first[c];
    for (int c = 0; c < ctas; ++c) h.load[c] = h.first[c];               // reuse as the write cursor
    for (int i = 0; i < n_items; ++i) {
        tb200::GroupItem it = h.pending[i];
        it.pad = 0;
        h.items[h.load[h.cta_of[i]]++] = it;
    }
    // The tables are rewritten in full by every call, so nothing in the scratch has to start at zero.
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned char* d_items = d_scratch + kNoAllocProbBytes;
    unsigned char* d_first = d_items + kNoAllocItemBytes;
    TB_CUDA(cudaMemcpyAsync(d_scratch, h.probs, size_t(n_probs) * sizeof(tb200::GroupProblem), cudaMemcpyHostToDevice, st));
    TB_CUDA(cudaMemcpyAsync(d_items, h.items, size_t(n_items) * sizeof(tb200::GroupItem), cudaMemcpyHostToDevice, st));
    TB_CUDA(cudaMemcpyAsync(d_first, h.first, size_t(ctas + 1) * sizeof(int), cudaMemcpyHostToDevice, st));
    const auto* p_probs = reinterpret_cast<const tb200::GroupProblem*>(d_scratch);
    const auto* p_items = reinterpret_cast<const tb200::GroupItem*>(d_items);
    const auto* p_first = reinterpret_cast<const int*>(d_first);
    // never a programmatic dependent: the table uploads above must be complete, and the shared scratch must not be
    // rewritten under a kernel that is still running
    if (mr == 1) return launch_gemv_group_tables<1, 32>(p_probs, p_items, p_first, ctas, d_status, st, false);
    if (mr == 2) return launch_gemv_group_tables<2, 32>(p_probs, p_items, p_first, ctas, d_status, st, false);
    return launch_gemv_group_tables<4, 32>(p_probs, p_items, p_first, ctas, d_status, st, false);
}

int ternix_b200_gemv_batch_noalloc_limits(int* max_problems, int* max_items, long long* scratch_bytes) {
    if (max_problems) *max_problems = kNoAllocMaxProblems;
    if (max_items) *max_items = kNoAllocMaxItems;
    if (scratch_bytes) *scratch_bytes = static_cast<long long>(kNoAllocBytes);
    return TERNIX_B200_OK;
}

int ternix_b200_weights_create(ternix_b200_weights** out, const uint8_t* dW, int K, int N) {
    if (!out) return TERNIX_B200_ERR_INVALID_ARG;
    *out = nullptr;
    if (K < 0 || N < 0 || (N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (K > 0 && N > 0 && !dW) return TERNIX_B200_ERR_INVALID_ARG;
    ternix_b200_weights* w = new (std::nothrow) ternix_b200_weights();
    if (!w) return TERNIX_B200_ERR_INVALID_ARG;
    w->dW = dW;
    w->K = K;
    w->N = N;
    w->device = current_device();
    w->fast = K >= 16 && N >= 64 && (N % 64) == 0 && (K % 16) == 0 && K <= kMaxScaledK && aligned(dW, 16);
    if (w->fast) {
        int rc = make_tmap_2d(&w->tmap_w_skinny, dW, static_cast<uint64_t>(N / 4), static_cast<uint64_t>(K),
                              static_cast<uint64_t>(N / 4), tb200::kSkWpRowBytes, tb200::kSkBK, CU_TENSOR_MAP_SWIZZLE_64B);
        if (!rc) rc = make_tc3_weight_map(&w->tmap_w_tc3, dW, K, N);
        if (rc) { delete w; return rc; }
    }
    *out = w;
    return TERNIX_B200_OK;
}

int ternix_b200_weights_matmul_host(ternix_b200_weights* w, const int8_t* A, int32_t* C, int M) {
    if (!w) return TERNIX_B200_ERR_INVALID_ARG;
    if (M < 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    const int K = w->K, N = w->N;
    if (M == 0 || N == 0) return TERNIX_B200_OK;
    if (!C || (K > 0 && !A)) return TERNIX_B200_ERR_INVALID_ARG;
    // Row slabs of about 64 MB of C (multiples of 256 rows, at most 16 slabs): the activations of slab j+1 go up while
    // slab j is computed and slab j-1 comes down.  A product with a small C runs as one slab.
    const long long c_bytes = static_cast<long long>(M) * N * 4;
    long long slabs = std::min<long long>(HostPipe::kMaxSlabs, std::max<long long>(1, c_bytes / (static_cast<long long>(64) << 20)));
    long long rows = (M + slabs - 1) / slabs;
    rows = std::min<long long>(M, ((rows + 255) / 256) * 256);
    if ((M + rows - 1) / rows + 1 > HostPipe::kMaxSlabs) rows = M;          // + 1: the short first slab
    return matmul_host_pipelined(A, nullptr, C, M, K, N, TERNIX_B200_KERNEL_AUTO, static_cast<int>(rows), true, w->dW);
}

void ternix_b200_weights_destroy(ternix_b200_weights* w) { delete w; }

int ternix_b200_weights_matmul(ternix_b200_weights* w, const int8_t* dA, int32_t* dC, int M, long long ldc,
                               int32_t* d_status, void* stream) {
    if (!w) return TERNIX_B200_ERR_INVALID_ARG;
    if (M < 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (ldc < w->N) return TERNIX_B200_ERR_INVALID_ARG;
    if (M == 0 || w->N == 0) return TERNIX_B200_OK;
    const int K = w->K, N = w->N;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int kernel = (w->fast && dA && dC) ? select_kernel(dA, w->dW, M, K, N) : TERNIX_B200_KERNEL_AUTO;
    if (kernel == TERNIX_B200_KERNEL_SKINNY_TC) {
        tb200::SkProblem prob{};
        {
            std::lock_guard<std::mutex> lock(w->mu);
            if (w->a_ptr[0] != dA || w->a_rows[0] != M) {
                const int rc = make_tmap_2d(&w->tmap_a[0], dA, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                                            static_cast<uint64_t>(K), 128, skinny_rows_class(M), CU_TENSOR_MAP_SWIZZLE_128B);
                if (rc) return rc;
                w->a_ptr[0] = dA;
                w->a_rows[0] = M;
            }
            prob.tmap_a = w->tmap_a[0];
        }
        prob.tmap_w = w->tmap_w_skinny;
        prob.C = dC; prob.ldc = ldc; prob.M = M; prob.K = K; prob.N = N;
        g_last_launched = TERNIX_B200_LAUNCHED_SKINNY_TC;
        return launch_skinny_problem(prob, d_status, st);
    }
    if (kernel == TERNIX_B200_KERNEL_GEMM_TC && options().tc3 && options().tc_bn == 0 && M > 64 && N >= 256 && (ldc % 4) == 0 &&
        aligned(dC, 16)) {
        CUtensorMap tmap_a;
        tb200::Tc3Stores stores{};
        {
            std::lock_guard<std::mutex> lock(w->mu);
            const int tile_rows = tc3_tile_rows(M);          // part of the key: an option can change it between calls
            if (w->a_ptr[1] != dA || w->a_rows[1] != M || w->a_tile_rows != tile_rows) {
                const int rc = make_tc3_act_map(&w->tmap_a[1], dA, M, K, tile_rows);
                if (rc) return rc;
                w->a_ptr[1] = dA;
                w->a_rows[1] = M;
                w->a_tile_rows = tile_rows;
            }
            if (w->c_ptr != dC || w->c_rows != M || w->c_ld != ldc) {
                const int rc = make_tc3_store_map(&w->tmap_c, dC, M, N, ldc);
                if (rc) return rc;
                w->c_ptr = dC;
                w->c_rows = M;
                w->c_ld = ldc;
            }
            tmap_a = w->tmap_a[1];
            stores.tmap_c[0] = w->tmap_c;
        }
        stores.count = 1;
        g_last_launched = TERNIX_B200_LAUNCHED_GEMM_TC3;
        return launch_gemm_tc3_maps(tmap_a, w->tmap_w_tc3, stores, dC, M, K, N, ldc, d_status, st);
    }
    return ternix_b200_matmul_ex(dA, w->dW, dC, M, K, N, ldc, TERNIX_B200_KERNEL_AUTO, d_status, stream);
}

int ternix_b200_selftest_wait_timeout(unsigned long long limit_ns, int32_t* d_status, unsigned long long* d_waited_ns,
                                      void* stream) {
    if (limit_ns == 0 || limit_ns > 100000000ull) return TERNIX_B200_ERR_INVALID_ARG;      // at most 100 ms
    wait_timeout_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, d_status, d_waited_ns);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

int ternix_b200_peer_barrier(void* const* flag_arrays, int world, int rank, unsigned epoch, unsigned long long limit_ns,
                             int32_t* d_status, void* stream) {
    if (world < 1 || world > kPeerBarrierMaxRanks || rank < 0 || rank >= world || !flag_arrays) return TERNIX_B200_ERR_INVALID_ARG;
    if (limit_ns == 0) limit_ns = tb200::kWaitLimitNs;
    if (limit_ns > tb200::kWaitLimitNs) return TERNIX_B200_ERR_INVALID_ARG;
    if (world == 1) return TERNIX_B200_OK;
    PeerFlags pf{};
    for (int r = 0; r < world; ++r) {
        if (!flag_arrays[r]) return TERNIX_B200_ERR_INVALID_ARG;
        pf.flags[r] = static_cast<unsigned*>(flag_arrays[r]);
    }
    peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, world, rank, epoch, limit_ns, d_status);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

int ternix_b200_pack_ternary_device(uint8_t* d_packed, const int8_t* d_unpacked, size_t size, void* stream) {
    const size_t n_bytes = size / 4;
    if (n_bytes == 0) return TERNIX_B200_OK;
    if (!d_packed || !d_unpacked) return TERNIX_B200_ERR_INVALID_ARG;
    const size_t threads_wanted = (n_bytes + 3) / 4;
    size_t blocks = (threads_wanted + 255) / 256;
    const size_t cap = static_cast<size_t>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    pack_ternary_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(d_unpacked, d_packed,
                                                                                                     n_bytes);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

int ternix_b200_quantize_rows(const void* dX, int x_dtype, long long ldx, int8_t* dA, float* d_row_scale, int M, int K,
                              void* stream) {
    if (M < 0 || K < 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (x_dtype != TERNIX_B200_DTYPE_F32 && x_dtype != TERNIX_B200_DTYPE_BF16) return TERNIX_B200_ERR_INVALID_ARG;
    if (M == 0) return TERNIX_B200_OK;
    if (!dX || !dA || !d_row_scale || ldx < K) return TERNIX_B200_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == TERNIX_B200_DTYPE_F32)
        quantize_rows_kernel<float><<<M, 256, 0, st>>>(static_cast<const float*>(dX), ldx, dA, d_row_scale, M, K);
    else
        quantize_rows_kernel<__nv_bfloat16><<<M, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dX), ldx, dA, d_row_scale, M, K);
    TB_CUDA(cudaGetLastError());
    return TERNIX_B200_OK;
}

int ternix_b200_matmul_dequant(const int8_t* dA, const uint8_t* dW, void* const* dY_list, int n_dest,
                               const float* d_row_scale, float w_scale, int M, int K, int N, long long ldy,
                               int32_t* d_status, void* stream) {
    if (M < 0 || K < 0 || N < 0 || (N % 4) != 0) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (ldy < N || n_dest < 1 || n_dest > tb200::kTc2MaxDest || !dY_list || !d_row_scale) return TERNIX_B200_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return TERNIX_B200_OK;
    for (int d = 0; d < n_dest; ++d)
        if (!dY_list[d]) return TERNIX_B200_ERR_INVALID_ARG;
    if (K > 0 && (!dA || !dW)) return TERNIX_B200_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K > 0 && gemm_tc2_ok(dA, dW, M, K, N))
        return launch_gemm_tc2_bf16(dA, dW, dY_list, n_dest, d_row_scale, w_scale, M, K, N, ldy, d_status, st);
    // Anything else: exact int32 product into a pool buffer, then one conversion pass.
    cudaMemPool_t pool = nullptr;
    int rc = host_call_pool(&pool);
    if (rc) return rc;
    int32_t* tmp = nullptr;
    TB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&tmp), static_cast<size_t>(M) * N * 4, pool, st));
    rc = ternix_b200_matmul_ex(dA, dW, tmp, M, K, N, N, TERNIX_B200_KERNEL_AUTO, d_status, stream);
    if (rc == TERNIX_B200_OK) {
        tb200::Tc2Dest dest{};
        dest.count = n_dest;
        for (int d = 0; d < n_dest; ++d) dest.c[d] = static_cast<int32_t*>(dY_list[d]);
        const long long total = static_cast<long long>(M) * N;
        long long blocks = (total + 255) / 256;
        const long long cap = static_cast<long long>(sm_count()) * 16;
        if (blocks > cap) blocks = cap;
        dequant_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(tmp, N, dest, ldy, d_row_scale, w_scale, M, N);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = cuda_fail(e);
    }
    cudaFreeAsync(tmp, st);
    return rc;
}

}  // extern "C"
