/*
 * CPU oracle for the ternary matrix product -- TEST INFRASTRUCTURE ONLY (see ternary_oracle.h).
 * Plain C restatement of the reference's CPU algorithm; parity pinned against the reference's own
 * sources compiled unmodified and against golden vectors made from them.
 */
#include "ternary_oracle.h"

#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* reference: src/bitpack.cpp:5-15 */
void oracle_pack_ternary(uint8_t *packed, const int8_t *unpacked, size_t size)
{
    const size_t nbytes = size / 4;
    for (size_t g = 0; g < nbytes; ++g) {
        unsigned byte = 0;
        for (int f = 0; f < 4; ++f) {
            const int v = unpacked[4 * g + f];
            const unsigned code = (v == 1) ? 1u : (v == -1) ? 3u : 0u;
            byte |= code << (2 * f);
        }
        packed[g] = (uint8_t)byte;
    }
}

/* reference: src/bitpack.cpp:17-27 */
void oracle_unpack_ternary(int8_t *unpacked, const uint8_t *packed, size_t size)
{
    const size_t nbytes = size / 4;
    for (size_t g = 0; g < nbytes; ++g) {
        const unsigned byte = packed[g];
        for (int f = 0; f < 4; ++f) {
            const unsigned code = (byte >> (2 * f)) & 3u;
            unpacked[4 * g + f] = (int8_t)(code == 1u ? 1 : code == 3u ? -1 : 0);
        }
    }
}

/* reference: src/bitpack.cpp:29-33 */
void oracle_interleave_offline(uint8_t *out, const uint8_t *packed, size_t size)
{
    memmove(out, packed, size / 4);
}

/* reference: src/mul_mat_ternary.cpp:38-58 */
void oracle_matmul_scalar(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N)
{
    const size_t pitch = N / 4;
    for (size_t i = 0; i < M; ++i) {
        int32_t *crow = C + i * N;
        memset(crow, 0, N * sizeof(int32_t));
        for (size_t k = 0; k < K; ++k) {
            const int32_t a = A[i * K + k];
            const uint8_t *wrow = Wp + k * pitch;
            for (size_t j = 0; j < N; ++j) {
                const int code = (wrow[j / 4] >> (2 * (j % 4))) & 3;
                crow[j] += a * ((code & 1) - (code & 2));
            }
        }
    }
}

/* reference: src/mul_mat_ternary.cpp:8-36 */
void oracle_matmul_naive(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N)
{
    const size_t pitch = N / 4;
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; ++j) {
            int32_t acc = 0;
            for (size_t k = 0; k < K; ++k) {
                const unsigned code = (Wp[k * pitch + j / 4] >> (2 * (j % 4))) & 3u;
                const int w = code == 1u ? 1 : code == 3u ? -1 : 0;
                acc += (int32_t)A[i * K + k] * w;
            }
            C[i * N + j] = acc;
        }
}

/* reference: src/mul_mat_ternary.cpp:60-105 (and :107-152, which performs the same adds in the same
 * k order for four rows at a time).  The vector lanes are written out as an 8-wide inner loop. */
void oracle_matmul_avx2_semantics(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N)
{
    const size_t pitch = N / 4;
    for (size_t i = 0; i < M; ++i)
        for (size_t j = 0; j < N; j += 8) {
            int32_t lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (size_t k = 0; k < K; ++k) {
                const int32_t a = A[i * K + k];
                const unsigned two = (unsigned)Wp[k * pitch + j / 4] | ((unsigned)Wp[k * pitch + j / 4 + 1] << 8);
                for (int l = 0; l < 8; ++l) {
                    const unsigned code = (two >> (2 * l)) & 3u;
                    /* shift-left 30 then arithmetic shift-right 30: 0->0, 1->+1, 2->-2, 3->-1 */
                    const int w = (int)code - ((code & 2u) ? 4 : 0);
                    /* psignd: a if w>0, 0 if w==0, -a if w<0 */
                    lane[l] += (w > 0) ? a : (w < 0) ? -a : 0;
                }
            }
            memcpy(C + i * N + j, lane, sizeof lane);
        }
}

/* reference: tests/test_ternary_matmul.cpp:31-39 */
void oracle_matmul_unpacked(const int8_t *A, const int8_t *W, int32_t *C, size_t M, size_t K, size_t N)
{
    memset(C, 0, M * N * sizeof(int32_t));
    for (size_t i = 0; i < M; ++i)
        for (size_t k = 0; k < K; ++k) {
            const int32_t a = A[i * K + k];
            const int8_t *wrow = W + k * N;
            int32_t *crow = C + i * N;
            for (size_t j = 0; j < N; ++j) crow[j] += a * wrow[j];
        }
}

/* Columns [n0, n0+Nn) of the product; n0 and Nn multiples of 4.  Unpacks the column slice once and
 * runs the unpacked GEMM of tests/test_ternary_matmul.cpp:31-39 with bands of rows on pthreads. */
struct band_job {
    const int8_t *A;
    const int8_t *W;
    int32_t *C;
    size_t r0, r1, K, Nn;
};

static void *band_main(void *arg)
{
    const struct band_job *b = (const struct band_job *)arg;
    for (size_t i = b->r0; i < b->r1; ++i) {
        int32_t *crow = b->C + i * b->Nn;
        memset(crow, 0, b->Nn * sizeof(int32_t));
        for (size_t k = 0; k < b->K; ++k) {
            const int32_t a = b->A[i * b->K + k];
            const int8_t *wrow = b->W + k * b->Nn;
            for (size_t j = 0; j < b->Nn; ++j) crow[j] += a * wrow[j];
        }
    }
    return NULL;
}

int oracle_matmul_columns(const int8_t *A, const uint8_t *Wp, int32_t *Cslice, size_t M, size_t K, size_t N,
                          size_t n0, size_t Nn, int threads)
{
    if (N % 4 || n0 % 4 || Nn % 4 || n0 + Nn > N) return 1;
    const size_t wbytes = K * Nn;
    int8_t *W = (int8_t *)malloc(wbytes ? wbytes : 1);
    if (!W) return 2;
    const size_t pitch = N / 4;
    for (size_t k = 0; k < K; ++k)
        oracle_unpack_ternary(W + k * Nn, Wp + k * pitch + n0 / 4, Nn);

    if (threads <= 0) {
        const long n = sysconf(_SC_NPROCESSORS_ONLN);
        threads = n > 0 ? (int)n : 1;
    }
    if ((size_t)threads > M) threads = M ? (int)M : 1;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    struct band_job job[256];
    const size_t band = (M + (size_t)threads - 1) / (size_t)threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        const size_t r0 = (size_t)t * band, r1 = r0 + band < M ? r0 + band : M;
        if (r0 >= r1) break;
        job[t] = (struct band_job){A, W, Cslice, r0, r1, K, Nn};
        if (t == threads - 1 || r1 == M) {      /* run the last band on the calling thread */
            band_main(&job[t]);
            break;
        }
        if (pthread_create(&tid[t], NULL, band_main, &job[t]) != 0) band_main(&job[t]);
        else started = t + 1;
    }
    for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
    free(W);
    return 0;
}

int oracle_matmul_fast(const int8_t *A, const uint8_t *Wp, int32_t *C, size_t M, size_t K, size_t N, int threads)
{
    return oracle_matmul_columns(A, Wp, C, M, K, N, 0, N, threads);
}
