/*
 * kq_oracle.c -- CPU restatement of the reference's Q5_K and Q6_K decode, of
 * their packers, and of the "expected value" computation its kernel tests use
 * for the K-quant matmuls, with a type-dispatching front (Q4_K goes to
 * q4k_oracle.c, which is linked into the same library).
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library or in the Python
 * package links, imports or calls this file; only the test-suite, the smoke
 * check and the benchmark's CPU-baseline leg do.
 *
 * Parity status: PINNED.  Checked bit-for-bit against the reference's own
 * runtime/gguf_loader.cpp compiled from its sources (Makefile target `ref`)
 * and against the formula-defined Q5_K / Q6_K fixtures of
 * runtime/tests/kernel_test.cpp (q5k_matmul_reference :1669-1676,
 * q6k_matmul_reference :1691-1698, q6k_gather_reference, q6k_matmul_wide_reference,
 * q6k_gather_batched_reference, q5k/q6k_matmul_batched4_reference :1732-1742),
 * whose expected values were generated with that compiled reference and are
 * stored under tests/golden/.
 *
 * One function at the end, oracle_prologue (the element-wise step of the reference's
 * fused decode shaders), is UNPINNED: it follows the reference's CPU formulas refSilu
 * (runtime/tests/kernel_test.cpp:165-166) and refRMSNorm (runtime/tests/op_test.cpp:684-693),
 * but those are file-static functions of test programs that cannot be built without the
 * reference's GPU backend, and the fused shaders have neither a test nor a caller.
 *
 * Type numbers are the reference's GGUFType values (runtime/gguf_loader.h:27-30):
 * Q4_K = 12, Q5_K = 13, Q6_K = 14.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256u
#define KQ_Q4_K 12u
#define KQ_Q5_K 13u
#define KQ_Q6_K 14u

float oracle_fp16_to_f32(uint16_t h);                                          /* q4k_oracle.c */
void oracle_q4k_dequant(const void *raw, float *out, uint32_t N, uint32_t K);  /* q4k_oracle.c */

/* Bytes of one 256-weight super-block as stored in a GGUF file; 0 for a type this file does not know. */
uint32_t oracle_kq_block_bytes(uint32_t type)
{
    return type == KQ_Q4_K ? 144u : type == KQ_Q5_K ? 176u : type == KQ_Q6_K ? 210u : 0u;
}

/* Q5_K super-block (176 bytes): fp16 d, fp16 dmin, 12 packed 6-bit scale/min
 * bytes (same packing as Q4_K), 32 bytes of fifth bits (bit sb of byte i
 * belongs to weight sb*32+i), 128 bytes of low nibbles laid out as in Q4_K.
 * w = (d*sc)*q - dmin*mn, q in 0..31, every operation rounded on its own.
 * Follows runtime/gguf_loader.cpp:497-534. */
static void q5k_block(const uint8_t *blk, float *out)
{
    uint16_t dh, mh;
    memcpy(&dh, blk, 2);
    memcpy(&mh, blk + 2, 2);
    const float d = oracle_fp16_to_f32(dh), dmin = oracle_fp16_to_f32(mh);
    const uint8_t *p = blk + 4, *qh = blk + 16, *qs = blk + 48;
    for (uint32_t sb = 0; sb < 8; sb++) {
        uint32_t sc, mn;
        if (sb < 4) {
            sc = p[sb] & 63u;
            mn = p[sb + 4] & 63u;
        } else {
            sc = (p[sb + 4] & 15u) | ((p[sb - 4] >> 2) & 0x30u);
            mn = (p[sb + 4] >> 4) | ((p[sb] >> 2) & 0x30u);
        }
        const float s = d * (float)sc, m = dmin * (float)mn;
        const uint8_t *q = qs + (sb >> 1) * 32u;
        const uint32_t shift = (sb & 1u) * 4u;
        for (uint32_t i = 0; i < 32; i++) {
            const uint32_t v = ((q[i] >> shift) & 15u) | (((qh[i] >> sb) & 1u) << 4);
            out[sb * 32u + i] = s * (float)v - m;
        }
    }
}

/* Q6_K super-block (210 bytes): 128 bytes of low nibbles, 64 bytes of high
 * bit pairs, 16 signed 8-bit scales (one per 16 weights), fp16 d at byte 208.
 * w = (d*sc)*q with q = 6-bit code - 32.  Element order follows
 * runtime/gguf_loader.cpp:535-573: each half of 128 weights takes 64 nibble
 * bytes and 32 bit-pair bytes; nibble byte l holds weights l (low) and l+64
 * (high), byte l+32 holds l+32 and l+96; bit-pair byte l holds the top bits of
 * weights l, l+32, l+64, l+96 from the least significant pair upwards. */
static void q6k_block(const uint8_t *blk, float *out)
{
    uint16_t dh;
    memcpy(&dh, blk + 208, 2);
    const float d = oracle_fp16_to_f32(dh);
    const int8_t *scales = (const int8_t *)(blk + 192);
    for (uint32_t half = 0; half < 2; half++) {
        const uint8_t *ql = blk + half * 64u, *qh = blk + 128u + half * 32u;
        const int8_t *sc = scales + half * 8u;
        float *o = out + half * 128u;
        for (uint32_t l = 0; l < 32; l++) {
            const uint32_t is = l / 16u;
            const int q1 = (int)((ql[l] & 15u) | (((qh[l] >> 0) & 3u) << 4)) - 32;
            const int q2 = (int)((ql[l + 32] & 15u) | (((qh[l] >> 2) & 3u) << 4)) - 32;
            const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3u) << 4)) - 32;
            const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3u) << 4)) - 32;
            o[l] = d * (float)sc[is] * (float)q1; /* (d*sc)*q, two roundings */
            o[l + 32] = d * (float)sc[is + 2] * (float)q2;
            o[l + 64] = d * (float)sc[is + 4] * (float)q3;
            o[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
    }
}

static void kq_block(uint32_t type, const uint8_t *blk, float *out)
{
    if (type == KQ_Q5_K) q5k_block(blk, out);
    else q6k_block(blk, out);
}

/* dequant_kquant(raw, out, N, K, type) of runtime/gguf_loader.cpp:455-573;
 * nBlocks = K/256 (floor), `raw` = N rows of nBlocks blocks without padding.
 * (The reference indexes the Q6_K output with 32-bit arithmetic; this
 * restatement uses 64 bits and is the same below 2^32 weights.) */
void oracle_kq_dequant(uint32_t type, const void *raw, float *out, uint32_t N, uint32_t K)
{
    if (type == KQ_Q4_K) { oracle_q4k_dequant(raw, out, N, K); return; }
    const uint32_t bb = oracle_kq_block_bytes(type);
    if (!bb) return;
    const uint8_t *src = (const uint8_t *)raw;
    const uint32_t nb = K / QK_K;
    for (uint32_t r = 0; r < N; r++)
        for (uint32_t b = 0; b < nb; b++)
            kq_block(type, src + ((uint64_t)r * nb + b) * bb, out + (uint64_t)r * K + (uint64_t)b * QK_K);
}

/* pack_q4k / pack_q5k / pack_q6k of runtime/gguf_loader.cpp:359-424: rows copied
 * into u32 words; the row stride is the row's bytes rounded up to a whole word
 * (only Q6_K rows, 210 bytes per block, ever need the padding, which is zero). */
void oracle_kq_pack(uint32_t type, const void *raw, uint32_t N, uint32_t K, uint32_t *words,
                    uint32_t *row_stride_words, uint32_t *n_blocks)
{
    const uint32_t bb = oracle_kq_block_bytes(type);
    const uint32_t nb = (K + QK_K - 1u) / QK_K;
    const uint32_t row_bytes = nb * bb;
    const uint32_t rs = (row_bytes + 3u) / 4u;
    if (n_blocks) *n_blocks = nb;
    if (row_stride_words) *row_stride_words = rs;
    if (!words || !bb) return;
    memset(words, 0, (size_t)N * rs * 4u);
    for (uint32_t r = 0; r < N; r++)
        memcpy((uint8_t *)(words + (uint64_t)r * rs), (const uint8_t *)raw + (uint64_t)r * row_bytes, row_bytes);
}

/* Rows [n0, n1) of Y[m][n] = bias[n] + sum_{k ascending} X[m][k]*deq[n][k] in
 * binary32: the expected-value loops of runtime/tests/kernel_test.cpp:1669-1676,
 * 1691-1698 (M = 1, zero start) and the *_wide / *_batched4 tests (start at
 * bias[n]). */
static void kq_rows(uint32_t type, const float *X, const uint8_t *raw, const float *bias, float *Y,
                    uint32_t M, uint32_t N, uint32_t K, uint32_t n0, uint32_t n1)
{
    const uint32_t nb = K / QK_K, bb = oracle_kq_block_bytes(type);
    float *deq = (float *)malloc((size_t)nb * QK_K * sizeof(float) + 4);
    for (uint32_t n = n0; n < n1; n++) {
        if (type == KQ_Q4_K) {
            oracle_q4k_dequant(raw + (uint64_t)n * nb * bb, deq, 1, nb * QK_K);
        } else {
            for (uint32_t b = 0; b < nb; b++) kq_block(type, raw + ((uint64_t)n * nb + b) * bb, deq + (size_t)b * QK_K);
        }
        for (uint32_t m = 0; m < M; m++) {
            const float *x = X + (uint64_t)m * K;
            float a = bias ? bias[n] : 0.0f;
            for (uint32_t k = 0; k < nb * QK_K; k++) a += x[k] * deq[k];
            Y[(uint64_t)m * N + n] = a;
        }
    }
    free(deq);
}

struct kq_job {
    uint32_t type;
    const float *X; const uint8_t *raw; const float *bias; float *Y;
    uint32_t M, N, K, n0, n1;
};
static void *kq_worker(void *p)
{
    struct kq_job *j = (struct kq_job *)p;
    kq_rows(j->type, j->X, j->raw, j->bias, j->Y, j->M, j->N, j->K, j->n0, j->n1);
    return NULL;
}

/* Whole matmul; `threads` > 1 splits the rows contiguously over pthreads (same
 * arithmetic per output). */
void oracle_kq_matmul(uint32_t type, const float *X, const void *raw, const float *bias, float *Y,
                      uint32_t M, uint32_t N, uint32_t K, uint32_t threads)
{
    if (!oracle_kq_block_bytes(type)) return;
    if (threads <= 1 || N < threads) {
        kq_rows(type, X, (const uint8_t *)raw, bias, Y, M, N, K, 0, N);
        return;
    }
    pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * threads);
    struct kq_job *jobs = (struct kq_job *)malloc(sizeof(struct kq_job) * threads);
    for (uint32_t t = 0; t < threads; t++) {
        jobs[t] = (struct kq_job){type, X, (const uint8_t *)raw, bias, Y, M, N, K,
                                  (uint32_t)((uint64_t)N * t / threads), (uint32_t)((uint64_t)N * (t + 1) / threads)};
        pthread_create(&tid[t], NULL, kq_worker, &jobs[t]);
    }
    for (uint32_t t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    free(jobs);
    free(tid);
}

/* The element-wise step the reference's fused decode shaders apply to the activation row before
 * the matmul, in binary32.  Where the reference holds a CPU formula for the step, that formula's
 * order of operations is followed:
 *   kind 1  rms = sqrtf(sum(x^2)/K + eps), out = x / rms * aux
 *           -- refRMSNorm of runtime/tests/op_test.cpp:684-693 (division by rms, then the weight:
 *           one more rounding than x * rstd * aux); the shader form is
 *           runtime/kernels/quant_kq/q4k_matmul_norm.wgsl:47-92, which adds the squares in 256
 *           strided partial sums and a tree where refRMSNorm (and this code) add in index order.
 *   kind 2  out = 0.5*g*(1 + tanh(0.7978845608*(g + 0.044715*g*g*g))) * aux
 *           -- the tanh form of runtime/kernels/quant_kq/q4k_down_gelu.wgsl:54-59.  The
 *           reference's CPU formula is the erf form (refGelu, runtime/tests/kernel_test.cpp:167),
 *           and its own test widens the tolerance to 5e-4 because the shaders use tanh
 *           (kernel_test.cpp:382-384); the shader's form is the one restated here.
 *   kind 3  out = g * (1/(1 + expf(-g))) * aux
 *           -- refSilu = x * refSigmoid(x) of runtime/tests/kernel_test.cpp:165-166, then the
 *           multiply of silu_mul_fused ahead of the down projection (runtime/model_runner.cpp:3755-3766).
 * Parity of this function is UNPINNED: refSilu and refRMSNorm are file-static functions of test
 * programs that need the Dawn GPU backend to build, so they cannot be compiled and run here, and
 * the reference has no test or caller for the fused shaders themselves. */
void oracle_prologue(uint32_t kind, const float *x, const float *aux, float eps, uint32_t K, float *out)
{
    if (kind == 1u) {
        float ss = 0.0f;
        for (uint32_t k = 0; k < K; k++) ss += x[k] * x[k];
        const float rms = sqrtf(ss / (float)K + eps);
        for (uint32_t k = 0; k < K; k++) out[k] = x[k] / rms * aux[k];
    } else if (kind == 2u) {
        for (uint32_t k = 0; k < K; k++) {
            const float g = x[k];
            const float inner = 0.7978845608f * (g + 0.044715f * g * g * g);
            out[k] = 0.5f * g * (1.0f + tanhf(inner)) * aux[k];
        }
    } else if (kind == 3u) {
        for (uint32_t k = 0; k < K; k++) {
            const float sig = 1.0f / (1.0f + expf(-x[k]));
            out[k] = x[k] * sig * aux[k];
        }
    } else {
        memcpy(out, x, (size_t)K * sizeof(float));
    }
}
