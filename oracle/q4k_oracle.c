/*
 * q4k_oracle.c -- CPU restatement of the reference's Q4_K decode and of the
 * "expected value" computation its kernel tests use for the Q4_K matmul.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library or in the Python
 * package links, imports or calls this file; only the test-suite, the smoke
 * check and the benchmark's CPU-baseline leg do, and there only as the checker
 * or as the timed CPU baseline.
 *
 * Parity status: PINNED.  The functions below are checked bit-for-bit against
 * the reference's own runtime/gguf_loader.cpp compiled from its sources (the
 * build recipe is the Makefile beside this file, target `ref`), and against
 * the four formula-defined Q4_K fixtures of runtime/tests/kernel_test.cpp
 * whose expected values were generated with that compiled reference and are
 * stored under tests/golden/.
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared (no -march=native, no
 * fast-math: the summation order and single-rounding behaviour are the
 * specification).
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256u
#define Q4K_BLOCK_BYTES 144u

/* Exact binary16 -> binary32, subnormals renormalised, inf/nan kept.
 * Follows runtime/gguf_loader.cpp:428-453 (kq_fp16_to_f32). */
float oracle_fp16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = ((uint32_t)h >> 10) & 0x1Fu;
    uint32_t m = (uint32_t)h & 0x3FFu;
    uint32_t bits;
    if (e == 31u) {
        bits = sign | 0x7F800000u | (m << 13);
    } else if (e != 0u) {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    } else if (m == 0u) {
        bits = sign;
    } else {
        /* subnormal: shift the mantissa up until the hidden bit appears */
        uint32_t ee = 113u;
        do { m <<= 1; ee--; } while ((m & 0x400u) == 0u);
        bits = sign | (ee << 23) | ((m & 0x3FFu) << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* The eight 6-bit (scale, min) pairs of one super-block from its 12 packed
 * bytes.  Follows runtime/gguf_loader.cpp:471-479 and, from the shader side,
 * runtime/kernels/quant_kq/q4k_matmul.wgsl:52-64. */
static void unpack_scales(const uint8_t *p, uint32_t sc[8], uint32_t mn[8])
{
    for (uint32_t j = 0; j < 4; j++) {
        sc[j] = p[j] & 63u;
        mn[j] = p[j + 4] & 63u;
        sc[j + 4] = (p[j + 8] & 15u) | ((p[j] >> 2) & 0x30u);
        mn[j + 4] = (p[j + 8] >> 4) | ((p[j + 4] >> 2) & 0x30u);
    }
}

/* One 144-byte super-block -> 256 floats.
 * w = (d*sc)*q - dmin*mn with every operation a separately rounded binary32
 * operation, exactly as runtime/gguf_loader.cpp:480-492 evaluates it. */
static void dequant_block(const uint8_t *blk, float *out)
{
    uint16_t dh, mh;
    memcpy(&dh, blk, 2);
    memcpy(&mh, blk + 2, 2);
    const float d = oracle_fp16_to_f32(dh);
    const float dmin = oracle_fp16_to_f32(mh);
    uint32_t sc[8], mn[8];
    unpack_scales(blk + 4, sc, mn);
    const uint8_t *codes = blk + 16;
    for (uint32_t sb = 0; sb < 8; sb++) {
        const float s = d * (float)sc[sb];
        const float m = dmin * (float)mn[sb];
        const uint8_t *q = codes + (sb >> 1) * 32u;
        const uint32_t shift = (sb & 1u) * 4u;
        for (uint32_t i = 0; i < 32; i++) {
            const float qv = (float)((q[i] >> shift) & 15u);
            out[sb * 32u + i] = s * qv - m; /* two roundings: built with -ffp-contract=off */
        }
    }
}

/* dequant_kquant(raw, out, N, K, Q4_K) of runtime/gguf_loader.cpp:455-496.
 * nBlocks = K / 256 (floor); elements with index >= nBlocks*256 are not
 * written, as in the reference.  `raw` holds N rows of nBlocks blocks with no
 * padding. */
void oracle_q4k_dequant(const void *raw, float *out, uint32_t N, uint32_t K)
{
    const uint8_t *src = (const uint8_t *)raw;
    const uint32_t nb = K / QK_K;
    for (uint32_t r = 0; r < N; r++)
        for (uint32_t b = 0; b < nb; b++)
            dequant_block(src + ((uint64_t)r * nb + b) * Q4K_BLOCK_BYTES,
                          out + (uint64_t)r * K + (uint64_t)b * QK_K);
}

/* pack_q4k of runtime/gguf_loader.cpp:359-379: the identity re-layout into
 * u32 words; returns rowStrideWords and nBlocks, copies N rows. */
void oracle_pack_q4k(const void *raw, uint32_t N, uint32_t K, uint32_t *words,
                     uint32_t *row_stride_words, uint32_t *n_blocks)
{
    const uint32_t nb = (K + QK_K - 1u) / QK_K;
    const uint32_t rs = nb * (Q4K_BLOCK_BYTES / 4u);
    if (n_blocks) *n_blocks = nb;
    if (row_stride_words) *row_stride_words = rs;
    if (!words) return;
    const uint64_t row_bytes = (uint64_t)nb * Q4K_BLOCK_BYTES;
    for (uint32_t r = 0; r < N; r++)
        memcpy(words + (uint64_t)r * rs, (const uint8_t *)raw + r * row_bytes, row_bytes);
}

/* Rows [n0, n1) of  Y[m][n] = bias[n] + sum_{k ascending} X[m][k] * deq[n][k]
 * in binary32 -- the expected-value code of runtime/tests/kernel_test.cpp:1682
 * (M = 1, accumulator starts at 0 and bias is 0) and :1688, :1728, :1746
 * (accumulator starts at bias[n]).  A zero start and a start at bias 0.0f are
 * the same float sequence, so one loop covers both.  `w_row_off` (rows) and
 * `y_off` (floats) give the indirect expert form of
 * runtime/kernels/quant_kq/iq4xs_matmul_moe.wgsl:55-66,96-99:
 * weight row = n + w_row_off, output index = y_off + m*N + n. */
static void matmul_rows(const float *X, const uint8_t *raw, const float *bias, float *Y,
                        uint32_t M, uint32_t N, uint32_t K, uint32_t n0, uint32_t n1,
                        uint64_t w_row_off, uint64_t y_off)
{
    const uint32_t nb = K / QK_K;
    float *deq = (float *)malloc((size_t)nb * QK_K * sizeof(float) + 4);
    for (uint32_t n = n0; n < n1; n++) {
        const uint8_t *row = raw + (w_row_off + n) * (uint64_t)nb * Q4K_BLOCK_BYTES;
        for (uint32_t b = 0; b < nb; b++)
            dequant_block(row + (uint64_t)b * Q4K_BLOCK_BYTES, deq + (size_t)b * QK_K);
        for (uint32_t m = 0; m < M; m++) {
            const float *x = X + (uint64_t)m * K;
            float a = bias ? bias[n] : 0.0f;
            for (uint32_t k = 0; k < nb * QK_K; k++) {
                a += x[k] * deq[k]; /* product rounded, then sum rounded */
            }
            Y[y_off + (uint64_t)m * N + n] = a;
        }
    }
    free(deq);
}

void oracle_q4k_matmul(const float *X, const void *raw, const float *bias, float *Y,
                       uint32_t M, uint32_t N, uint32_t K)
{
    matmul_rows(X, (const uint8_t *)raw, bias, Y, M, N, K, 0, N, 0, 0);
}

/* Indirect (expert-stacked) form: one call per routed slot, as the reference
 * dispatches it (runtime/model_runner.cpp:3584-3651). */
void oracle_q4k_matmul_moe_slot(const float *X, const void *raw, const float *bias, float *Y,
                                uint32_t M, uint32_t N, uint32_t K, const uint32_t *offsets,
                                uint32_t slot, uint32_t y_offset)
{
    matmul_rows(X, (const uint8_t *)raw, bias, Y, M, N, K, 0, N, offsets[slot], y_offset);
}

/* Row-parallel version of oracle_q4k_matmul for the timed CPU baseline: the
 * same per-row arithmetic, rows split contiguously over `threads` pthreads. */
struct mt_job {
    const float *X; const uint8_t *raw; const float *bias; float *Y;
    uint32_t M, N, K, n0, n1;
};
static void *mt_worker(void *p)
{
    struct mt_job *j = (struct mt_job *)p;
    matmul_rows(j->X, j->raw, j->bias, j->Y, j->M, j->N, j->K, j->n0, j->n1, 0, 0);
    return NULL;
}
void oracle_q4k_matmul_mt(const float *X, const void *raw, const float *bias, float *Y,
                          uint32_t M, uint32_t N, uint32_t K, uint32_t threads)
{
    if (threads <= 1 || N < threads) { oracle_q4k_matmul(X, raw, bias, Y, M, N, K); return; }
    pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * threads);
    struct mt_job *jobs = (struct mt_job *)malloc(sizeof(struct mt_job) * threads);
    for (uint32_t t = 0; t < threads; t++) {
        jobs[t] = (struct mt_job){X, (const uint8_t *)raw, bias, Y, M, N, K,
                                  (uint32_t)((uint64_t)N * t / threads),
                                  (uint32_t)((uint64_t)N * (t + 1) / threads)};
        pthread_create(&tid[t], NULL, mt_worker, &jobs[t]);
    }
    for (uint32_t t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    free(jobs);
    free(tid);
}

/* float64-accumulate variant, used only to attribute error (which of two
 * float32 results is closer to the exact sum). */
void oracle_q4k_matmul_f64(const float *X, const void *raw, const float *bias, double *Y,
                           uint32_t M, uint32_t N, uint32_t K)
{
    const uint8_t *src = (const uint8_t *)raw;
    const uint32_t nb = K / QK_K;
    float *deq = (float *)malloc((size_t)nb * QK_K * sizeof(float) + 4);
    for (uint32_t n = 0; n < N; n++) {
        for (uint32_t b = 0; b < nb; b++)
            dequant_block(src + ((uint64_t)n * nb + b) * Q4K_BLOCK_BYTES, deq + (size_t)b * QK_K);
        for (uint32_t m = 0; m < M; m++) {
            double a = bias ? (double)bias[n] : 0.0;
            for (uint32_t k = 0; k < nb * QK_K; k++)
                a += (double)X[(uint64_t)m * K + k] * (double)deq[k];
            Y[(uint64_t)m * N + n] = a;
        }
    }
    free(deq);
}
