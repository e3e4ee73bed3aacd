/*
 * ternix_b200 -- C ABI of the B200 (sm_100a) ternary matrix product
 *
 *      C[M,N] int32  =  A[M,K] int8  x  W[K,N] ternary
 *
 * W stays in TernixEngine's packed format: row-major K x (N/4) bytes, four weights per byte,
 * weight j of a group in bits 2j..2j+1, code 00 -> 0, 01 -> +1, 11 -> -1 (code 10 is never produced by
 * the packer and is undefined input).  All arithmetic is exact integer arithmetic.
 *
 * This header is what a foreign-function binding (ctypes, cgo, JNI, ...) binds.  Plain pointers and
 * sizes only; every function returns a status code; nothing throws.  The C++ `ternix::` functions of
 * include/ternix/ and the `ternix_engine` Python module are thin callers of these entry points.
 * There is no CPU fallback: a device entry point on a machine without a usable GPU fails with
 * TERNIX_B200_ERR_CUDA.
 *
 * Each entry point names the reference interface it replaces (path inside the reference project).
 */
#ifndef TERNIX_B200_H
#define TERNIX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes --------------------------------------------------------------------------- */
#define TERNIX_B200_OK                 0
#define TERNIX_B200_ERR_INVALID_SHAPE  1  /* M,K,N out of domain (N % 4 != 0, negative, too large)  */
#define TERNIX_B200_ERR_INVALID_ARG    2  /* null pointer, bad enum, bad pitch                       */
#define TERNIX_B200_ERR_CUDA           3  /* a CUDA call failed; see ternix_b200_last_cuda_error()   */
#define TERNIX_B200_ERR_TIMEOUT        4  /* a bounded device-side wait ran out (kernel returned)    */
#define TERNIX_B200_ERR_UNSUPPORTED    5  /* the kernel that was asked for cannot take this problem  */
#define TERNIX_B200_ERR_TOO_LARGE      6  /* beyond the fixed capacity of an allocation-free entry   */

/* ---- kernel selectors ------------------------------------------------------------------------ */
#define TERNIX_B200_KERNEL_AUTO     0  /* pick by shape and alignment                                 */
#define TERNIX_B200_KERNEL_GENERIC  1  /* any M, K; N % 4 == 0; any pitch or alignment                */
#define TERNIX_B200_KERNEL_GEMV     2  /* decode regime, M <= 16: TMA-streamed packed W, dp4a         */
#define TERNIX_B200_KERNEL_GEMM_TC  3  /* prefill regime: TMA + tcgen05 kind::i8, int32 in TMEM       */
#define TERNIX_B200_KERNEL_DECODE_MMA 4 /* batched decode (a few to a few dozen rows): TMA-streamed   */
                                       /* packed W decoded in registers into mma.sync.m16n8k32       */
#define TERNIX_B200_KERNEL_SKINNY_TC 5 /* batched decode, 1..128 rows: TMA-streamed packed W decoded  */
                                       /* into tensor memory as the A operand of tcgen05 kind::i8     */

/* ---- what a single-product call launched (ternix_b200_last_launched_kernel) ------------------- */
#define TERNIX_B200_LAUNCHED_GENERIC     1
#define TERNIX_B200_LAUNCHED_GEMV        2
#define TERNIX_B200_LAUNCHED_GEMM_TC1    3  /* single-CTA tcgen05 tiles, weights expanded in shared memory */
#define TERNIX_B200_LAUNCHED_DECODE_MMA  4
#define TERNIX_B200_LAUNCHED_SKINNY_TC   5
#define TERNIX_B200_LAUNCHED_GEMM_TC2    6  /* paired CTAs, weights expanded in shared memory              */
#define TERNIX_B200_LAUNCHED_GEMM_TC3    7  /* paired CTAs, weights decoded into tensor memory             */

const char *ternix_b200_status_string(int status);
/* cudaError_t (as int) of the last failing CUDA call made by the calling thread, 0 if none. */
int ternix_b200_last_cuda_error(void);
/* Text of a cudaError_t value (cudaGetErrorString), so that bindings need not link the CUDA runtime. */
const char *ternix_b200_cuda_error_string(int cuda_error);
/* Library version, major*10000 + minor*100 + patch. */
int ternix_b200_version(void);
/* The kernel the calling thread's last ternix_b200_matmul / _matmul_ex / _matmul_bcast call launched
 * (TERNIX_B200_LAUNCHED_*, 0 if none) and that kernel's name, so a benchmark can report what actually ran. */
int ternix_b200_last_launched_kernel(void);
const char *ternix_b200_launched_kernel_name(int launched);
/* Tuning options.  The defaults are the measured best; tests and experiments force the other paths.  Each option is
 * read once from the environment variable TERNIX_B200_<NAME> when the library is first used and can be changed
 * afterwards only here (value NULL or "" restores the default); do not change options while another thread
 * launches.  Names: tc3 (0|1), tc_tile_rows (0|128|256: activation rows per pair instruction of the prefill kernel), tc_bn (0|2|128|256), tc_ksplit (0|1), gemv_plan ("words,ksplit"), group_words
 * (16|32), gemv_pdl (-1|0|1), mma_rows ("lo,hi"), mma_slices, mma_cluster (0|2|4|8), skinny_rows ("lo,hi"), skinny_group_rows ("lo,hi", lo 0 = never), skinny_split (0|1|2),
 * host_slab (<columns>|r<rows>|0).  Unknown name: TERNIX_B200_ERR_INVALID_ARG. */
int ternix_b200_set_option(const char *name, const char *value);
/* The host-pointer entry point (and the unfused dequantising path) take device memory from a stream-ordered pool
 * private to this library, which keeps up to 1 GiB of freed blocks per device for the next call, where the
 * reference's wrapper frees everything before it returns (src/cuda_kernels.cu:153).  This call hands all cached
 * blocks of every device back to the driver. */
int ternix_b200_release_cached_memory(void);

/* ---- host side: the packed weight format -------------------------------------------------------
 * replaces: ternix::pack_ternary_weights / unpack_ternary_weights / interleave_weights_offline,
 *           include/ternix/bitpack.hpp:6-8, src/bitpack.cpp:5-33.  Byte-for-byte the same output;
 *           `size` counts weights, size/4 bytes are produced (a tail of size%4 weights is dropped). */
void ternix_b200_pack_ternary(uint8_t *packed, const int8_t *unpacked, size_t size);
void ternix_b200_unpack_ternary(int8_t *unpacked, const uint8_t *packed, size_t size);
void ternix_b200_interleave_offline(uint8_t *interleaved, const uint8_t *packed, size_t size);
/* Index of the first value outside {-1,0,+1}, or -1 if all are in the domain
 * (the check bindings/python/pybind11_wrapper.cpp:26-27 makes before packing). */
long long ternix_b200_find_non_ternary(const int8_t *unpacked, size_t size);
/* Copy the column shard [n0, n0+n_cols) of a packed K x (N/4) matrix into a packed K x (n_cols/4)
 * matrix (n0, n_cols multiples of 4).  Host memory.  Used for N-column sharding across GPUs. */
int ternix_b200_slice_columns(uint8_t *dst, const uint8_t *packed, size_t K, size_t N, size_t n0, size_t n_cols);

/* ---- device side -----------------------------------------------------------------------------
 * replaces: ternix::mul_mat_ternary_cuda_naive / _tiled, include/ternix/cuda_kernels.cuh:11-17,
 *           src/cuda_kernels.cu:126-140.
 * dA [M,K] int8 row-major, dW packed K x (N/4), dC [M,N] int32 row-major: device pointers.
 * Asynchronous on `stream` (a cudaStream_t passed as void*; NULL = default stream).  C is fully
 * overwritten.  Shape errors are reported before any pointer is touched.  Launch errors are returned;
 * errors that occur while the kernel runs surface at the next synchronisation on the stream. */
int ternix_b200_matmul(const int8_t *dA, const uint8_t *dW, int32_t *dC, int M, int K, int N, void *stream);

/* Same, with control: `kernel` is one of TERNIX_B200_KERNEL_*; `ldc` is the row pitch of C in int32
 * elements (>= N), so a column shard can be written straight into its place in a wider matrix;
 * `d_status`, if not NULL, is a device int32 that a kernel sets to TERNIX_B200_ERR_TIMEOUT when one of
 * its bounded waits runs out (the caller zeroes it and reads it after synchronising). */
int ternix_b200_matmul_ex(const int8_t *dA, const uint8_t *dW, int32_t *dC, int M, int K, int N, long long ldc,
                          int kernel, int32_t *d_status, void *stream);

/* The kernel TERNIX_B200_KERNEL_AUTO would choose for this problem (no GPU needed). */
int ternix_b200_select_kernel(const void *dA, const void *dW, const void *dC, int M, int K, int N, long long ldc);

/* replaces: ternix::mul_mat_ternary_cuda_host, include/ternix/cuda_kernels.cuh:20-21,
 *           src/cuda_kernels.cu:142-156.  HOST pointers: allocates, copies in, runs, copies back,
 *           frees, synchronises.  Also the target of the CPU-named ternix::mul_mat_ternary_* shims.
 *           The device buffer comes from a stream-ordered pool private to this library and is returned to
 *           it before the call ends; the pool keeps the pages so later calls skip the driver allocation.
 *           Above 64 MB of C the call runs as a pipeline over slabs of C on three private streams (inputs of
 *           the next slab up, current slab computed, previous slab down); the bytes of C are the same. */
int ternix_b200_matmul_host(const int8_t *A, const uint8_t *W_packed, int32_t *C, int M, int K, int N, int kernel);

/* ---- weight handle -----------------------------------------------------------------------------------
 * No reference counterpart (the reference has no weight object on this path; interleave_weights_offline,
 * src/bitpack.cpp:29-33, is its placeholder for one).  create() encodes the TMA descriptors of a packed weight matrix
 * once, for every kernel family that can take it; matmul() is ternix_b200_matmul_ex with AUTO dispatch that encodes
 * nothing for operands it has seen on the previous call (the handle remembers the last A and C it was given), so a
 * steady decode loop makes no cuTensorMapEncodeTiled call at all.  Allocates no device memory.  dW must stay valid
 * while the handle lives.  A handle may be shared by threads; its calls take a mutex for the descriptor cache. */
typedef struct ternix_b200_weights ternix_b200_weights;
int ternix_b200_weights_create(ternix_b200_weights **out, const uint8_t *dW, int K, int N);
int ternix_b200_weights_matmul(ternix_b200_weights *weights, const int8_t *dA, int32_t *dC, int M, long long ldc,
                               int32_t *d_status, void *stream);
/* The serving form of the host-pointer call: the weights stay on the device (the handle), the activations come from
 * host memory and C goes back to host memory, in row slabs on three streams (upload of slab j+1, product of slab j,
 * download of slab j-1), so that the call takes little more than the download of C.  Pinned host memory makes the
 * copies asynchronous; pageable memory works and is slower.  Synchronous: C is complete when it returns.  Calls on one
 * device run one after the other. */
int ternix_b200_weights_matmul_host(ternix_b200_weights *weights, const int8_t *A_host, int32_t *C_host, int M);
void ternix_b200_weights_destroy(ternix_b200_weights *weights);

/* replaces: ternix::pack_ternary_weights (src/bitpack.cpp:5-15) for weights that are already on the device: the same
 * bytes as ternix_b200_pack_ternary, produced by a kernel.  `size` counts weights; size/4 bytes are written. */
int ternix_b200_pack_ternary_device(uint8_t *d_packed, const int8_t *d_unpacked, size_t size, void *stream);

/* Self-test of the bounded device-side waits, with no counterpart in the reference: launches one small CTA in which
 * one warp waits, for at most limit_ns (<= 100 ms), on a shared-memory barrier nobody arrives on; the wait runs out,
 * the CTA takes the same abort and drain path as the product kernels, writes TERNIX_B200_ERR_TIMEOUT into *d_status
 * (atomicMax) and the nanoseconds it waited into *d_waited_ns (may be NULL), and returns.  Nothing faults and the
 * context stays usable. */
int ternix_b200_selftest_wait_timeout(unsigned long long limit_ns, int32_t *d_status, unsigned long long *d_waited_ns,
                                      void *stream);

/* ---- problem groups: many projections per launch ----------------------------------------------
 * No reference counterpart (the reference launches one product at a time; its README lists
 * graph-captured projection sets as future work, README.md:213).  A group is built once from a list of
 * problems on device pointers and then run any number of times.  Members that a TMA descriptor can describe
 * (K % 16 == 0, N % 64 == 0, 16-byte aligned A and W) share launches by regime: one-row members (K <= 8192) ONE
 * persistent kernel that streams all their weights back to back; members with 2..16 rows one launch of the
 * mma.sync decode kernel per row-group size (8, 16); members with 17..128 rows one launch of the tensor-memory
 * decode kernel per batch class (16, 32, 64, 128); members with more than 128 rows (N >= 256) ONE launch of the
 * paired-CTA tensor-core GEMM that walks all their tiles.  The others are launched one by one behind them.
 * create() allocates small device tables (TMA descriptors and the work lists) and copies them synchronously;
 * run() only launches, on `stream`.  The pointers inside the problems must stay valid while the group lives.
 * A one-row batch with at most four work items per CTA is launched as a programmatic dependent of the kernel
 * before it on the stream: behind another decode batch of this library it starts streaming weights while that
 * batch finishes (activations are read and C is written only after it has completed). */
typedef struct ternix_b200_problem {
    const int8_t *dA;      /* [M,K] int8 row-major          */
    const uint8_t *dW;     /* packed K x (N/4)              */
    int32_t *dC;           /* [M,N] int32, row pitch ldc    */
    int M, K, N;
    long long ldc;
} ternix_b200_problem;
typedef struct ternix_b200_group ternix_b200_group;
int ternix_b200_group_create(ternix_b200_group **out, const ternix_b200_problem *problems, int count);
/* Same, with n_peers (< 8) extra destinations per problem: peer_dC[i * n_peers + j] receives the same C as
 * problems[i].dC (same ldc), typically the same columns of C in a peer GPU's memory.  Prefill-regime members
 * (M > 128, N >= 256, TMA-able) share ONE launch of the paired-CTA GEMM, which stores to all destinations
 * from its epilogue; other members are computed as usual and copied. */
int ternix_b200_group_create_ex(ternix_b200_group **out, const ternix_b200_problem *problems, int count,
                                int32_t *const *peer_dC, int n_peers);
/* Prepacked weights for the decode regime (the reference keeps a placeholder for an offline layout,
 * interleave_weights_offline, src/bitpack.cpp:29-33, README.md:205; this is a real one, kept beside -- not instead
 * of -- the packed interchange format).  ternix_b200_prepack_k4 rewrites a packed K x (N/4) matrix on the device so
 * that the four bytes a decode step needs from four consecutive k-rows sit in one 32-bit word:
 * word [k/4][b] = { W[4r][b], W[4r+1][b], W[4r+2][b], W[4r+3][b] }, zero beyond K; ceil(K/4) * N bytes.  A group
 * created with ternix_b200_group_create_prepacked takes problems whose dW point at such matrices (decode-regime
 * members only, same limits as above) and skips the in-kernel byte transpose.  Results are identical. */
size_t ternix_b200_prepack_k4_bytes(int K, int N);
int ternix_b200_prepack_k4(const uint8_t *dW, uint8_t *dW_prepacked, int K, int N, void *stream);
int ternix_b200_group_create_prepacked(ternix_b200_group **out, const ternix_b200_problem *problems, int count);
int ternix_b200_group_run(const ternix_b200_group *group, int32_t *d_status, void *stream);
/* Kernel launches one run() makes (one per regime in use + 1 per problem no grouped kernel could take). */
int ternix_b200_group_launches(const ternix_b200_group *group);
void ternix_b200_group_destroy(ternix_b200_group *group);

/* ---- a decode batch for callers that must not allocate ---------------------------------------------
 * No counterpart in the reference.  Some callers cannot have the library call cudaMalloc on their behalf:
 * an inference server whose device memory is owned entirely by its own pool allocator, a caller inside a
 * memory-capped or real-time section, a plugin host that forbids allocation after start-up.  For them
 * this entry point runs the same persistent decode kernel as ternix_b200_group_run, but the tables that
 * kernel reads (TMA descriptors, work list) sit in a fixed array inside the library image instead of a
 * cudaMalloc'ed block, and the host side uses fixed buffers too: no cudaMalloc, cudaFree or other
 * allocating call is made.  The caller passes inputs and outputs exactly as for a group.
 *   - Limits: at most 256 problems and 4096 work items (one item per 512-column chunk per group of up to
 *     4 rows) per call; beyond that TERNIX_B200_ERR_TOO_LARGE.  Only decode-regime problems are taken
 *     (M <= 16, K <= 8192, K % 16 == 0, N % 64 == 0, 16-byte aligned A and W), else
 *     TERNIX_B200_ERR_UNSUPPORTED.  The fixed array is 117,504 bytes and every GPU that loads the library
 *     holds it until the process exits (ternix_b200_gemv_batch_noalloc_limits reports the numbers).
 *   - The first call on a device looks up the array's device address (with that device current); make that
 *     first call outside any stream capture.
 *   - A call on a stream that is being captured is refused with TERNIX_B200_ERR_UNSUPPORTED: the tables are
 *     uploaded from one fixed host buffer, and a graph would read that buffer at replay time, after later calls
 *     have rewritten it.  A member with K == 0 gets its C zeroed, as in the single-product calls.
 *   - All calls share the one array and each call rewrites the tables it uses, so nothing needs clearing,
 *     but two calls whose work overlaps on the GPU (different streams, or a second call issued before the
 *     first one's kernel has finished on another stream) race on it.  Calls on one stream are safe. */
int ternix_b200_gemv_batch_noalloc(const ternix_b200_problem *problems, int count, int32_t *d_status, void *stream);
int ternix_b200_gemv_batch_noalloc_limits(int *max_problems, int *max_items, long long *scratch_bytes);

/* ---- one product, several destinations (fused gather) -------------------------------------------
 * No reference counterpart.  Computes C[M,N] once and writes it to every pointer in dC_list (all with row
 * pitch ldc): the caller's own C first and, for N-column-sharded weights, the same columns of C in each
 * peer GPU's memory, through peer-mapped pointers.  For tensor-core-sized problems the stores are issued
 * by the GEMM epilogue itself, tile by tile, so the transfer overlaps the main loop and no separate
 * all-gather is needed; other problems are computed into dC_list[0] and copied.  n_dest <= 8.  The caller
 * synchronises the GPUs (e.g. a barrier on the same stream) before anyone reads the gathered C. */
int ternix_b200_matmul_bcast(const int8_t *dA, const uint8_t *dW, int32_t *const *dC_list, int n_dest, int M, int K,
                             int N, long long ldc, int32_t *d_status, void *stream);

/* Device buffers that other processes on the same node can map (CUDA IPC): allocate, export a 64-byte
 * handle, import a peer's handle (enables peer access), close, free. */
int ternix_b200_peer_alloc(void **dptr, size_t bytes);
int ternix_b200_peer_free(void *dptr);
int ternix_b200_peer_export(void *dptr, unsigned char handle[64]);
int ternix_b200_peer_import(const unsigned char handle[64], void **dptr);
int ternix_b200_peer_close(void *dptr);
/* A barrier between the ranks of a sharded product, enqueued on `stream` (one small kernel; no library collective):
 * flag_arrays[r] is rank r's flag array (`world` 32-bit slots, zeroed once, from ternix_b200_peer_alloc; the own
 * rank's entry is the local allocation, the others are imported mappings).  Every rank calls it with the same epoch,
 * which must grow by one from call to call.  When the kernel has finished on this rank, every rank's work enqueued
 * before its own call has finished and its stores into this rank's memory are visible here.  A peer that does not
 * arrive within limit_ns (0 = the library's 2 s limit) sets TERNIX_B200_ERR_TIMEOUT in *d_status; nothing traps.
 * Replaces the 4-byte ncclAllReduce that served as the barrier before (18 us per step against 5 us). */
int ternix_b200_peer_barrier(void *const *flag_arrays, int world, int rank, unsigned epoch, unsigned long long limit_ns,
                             int32_t *d_status, void *stream);

/* ---- the steps either side of the product in a BitNet-style layer -----------------------------------
 * No counterpart in the reference (its README lists activation/absmean scaling as missing, README.md:203); the
 * arithmetic is the published BitNet b1.58 recipe, stated exactly so that it can be checked bit for bit:
 *   quantize_rows:  absmax = max_k |x[m,k]|;  q = rint(x * (127 / absmax)) clamped to [-127,127] (fp32, nearest
 *                   even);  row_scale[m] = absmax / 127  (all-zero row: q = 0, row_scale = 1).
 *   matmul_dequant: y[m,n] = bf16_rn((float(c[m,n]) * row_scale[m]) * w_scale) with c the exact int32 product;
 *                   bfloat16 out (ldy in elements), up to 8 destinations as for ternix_b200_matmul_bcast.  Large
 *                   problems do this in the GEMM epilogue; others compute int32 into a pool buffer and convert. */
#define TERNIX_B200_DTYPE_F32   0
#define TERNIX_B200_DTYPE_BF16  1
int ternix_b200_quantize_rows(const void *dX, int x_dtype, long long ldx, int8_t *dA, float *d_row_scale, int M, int K,
                              void *stream);
int ternix_b200_matmul_dequant(const int8_t *dA, const uint8_t *dW, void *const *dY_list, int n_dest,
                               const float *d_row_scale, float w_scale, int M, int K, int N, long long ldy,
                               int32_t *d_status, void *stream);

/* ---- N-column sharding plan (host arithmetic only) ---------------------------------------------
 * Splits N columns over `world` ranks in granules of `granule` columns (a multiple of 4; 64 keeps each
 * shard's packed rows 16-byte aligned).  Writes the first column and the column count of `rank`.
 * Shards differ by at most one granule; trailing ranks may get zero columns when N is small. */
int ternix_b200_shard_columns(int N, int world, int rank, int granule, int *n0, int *n_cols);

/* Scatter a rank-major gather buffer [world][M][n_pad] (what an all-gather of equal-sized blocks
 * delivers) into row-major dC[M, ldc] using the plan above.  Device pointers, asynchronous. */
int ternix_b200_unpack_gathered(const int32_t *d_gathered, int32_t *dC, int M, int N, long long ldc, int world,
                                int granule, int n_pad, void *stream);

/* ---- seeded synthetic inputs (host) ----------------------------------------------------------
 * Counter-based generator (splitmix64 of seed and index), so any slice can be regenerated anywhere.
 * mode 0: int8 uniform on [-128,127]; mode 1: uniform on [-127,127]. */
void ternix_b200_synth_activations(int8_t *A, size_t count, uint64_t seed, int mode);
/* iid ternary with P(-1) = P(+1) = 0.3, P(0) = 0.4, already packed: K x (N/4) bytes. */
void ternix_b200_synth_packed_weights(uint8_t *W_packed, size_t K, size_t N, uint64_t seed);
/* The same weights, unpacked, for checking: K x N int8. */
void ternix_b200_synth_weights(int8_t *W, size_t K, size_t N, uint64_t seed);

#ifdef __cplusplus
}
#endif
#endif /* TERNIX_B200_H */
