/*
 * Plain-C restatement of the reference's CPU path for TQ1_G128 packed ternary
 * weights. TEST INFRASTRUCTURE ONLY: it is the checker and the timed CPU
 * baseline, never part of the shipped library.
 *
 * Parity status: pinned. tests/test_oracle_golden.py compares every function
 * here with fixtures produced by the unmodified reference.
 *
 * Follows, in the reference project:
 *   src/bonsai_tq1/format.py:66-91    encode  (tq1o_encode)
 *   src/bonsai_tq1/format.py:94-122   decode + fail-closed byte scan (tq1o_decode)
 *   src/bonsai_tq1/reference.py:14-39 decode-then-dot GEMV, FP32 (tq1o_matmul_f32)
 *   src/ternel_mlx/reference.py:196-230 row gather (tq1o_get_rows_f32)
 *
 * Build: see oracle/Makefile (gcc -O3 -pthread -shared -fPIC).
 */
#include <stdint.h>
#include <string.h>
#include <math.h>
#include <pthread.h>
#include <unistd.h>

#define GROUP 128
#define BLOCK_BYTES 28

/* IEEE binary16 -> binary32 without relying on compiler half support. */
static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {            /* subnormal: normalise */
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* 0 on success, -1 when a trit is outside {0,1,2} (n_bad = how many). */
int tq1o_encode(const uint8_t *scales, const uint8_t *trits, uint8_t *blocks,
                int64_t groups, int64_t *n_bad) {
    int64_t bad = 0;
    for (int64_t i = 0; i < groups * GROUP; ++i) bad += trits[i] > 2;
    if (n_bad) *n_bad = bad;
    if (bad) return -1;
    for (int64_t g = 0; g < groups; ++g) {
        const uint8_t *c = trits + g * GROUP;
        uint8_t *b = blocks + g * BLOCK_BYTES;
        b[0] = scales[2 * g];
        b[1] = scales[2 * g + 1];
        for (int j = 0; j < 25; ++j) {
            const uint8_t *p = c + 5 * j;
            b[2 + j] = (uint8_t)(p[0] + 3 * p[1] + 9 * p[2] + 27 * p[3] + 81 * p[4]);
        }
        b[27] = (uint8_t)(c[125] + 3 * c[126] + 9 * c[127]);
    }
    return 0;
}

/* 0 on success, -1 when validate is set and an illegal byte exists (counts returned). */
int tq1o_decode(const uint8_t *blocks, uint8_t *scales, uint8_t *trits, int64_t groups,
                int validate, int64_t *n_bad_full, int64_t *n_bad_tail) {
    int64_t bf = 0, bt = 0;
    if (validate) {
        for (int64_t g = 0; g < groups; ++g) {
            const uint8_t *b = blocks + g * BLOCK_BYTES;
            for (int j = 2; j < 27; ++j) bf += b[j] > 242;
            bt += b[27] > 26;
        }
    }
    if (n_bad_full) *n_bad_full = bf;
    if (n_bad_tail) *n_bad_tail = bt;
    if (bf || bt) return -1;
    for (int64_t g = 0; g < groups; ++g) {
        const uint8_t *b = blocks + g * BLOCK_BYTES;
        uint8_t *c = trits + g * GROUP;
        scales[2 * g] = b[0];
        scales[2 * g + 1] = b[1];
        for (int j = 0; j < 25; ++j) {
            unsigned v = b[2 + j];
            for (int i = 0; i < 5; ++i) { c[5 * j + i] = (uint8_t)(v % 3); v /= 3; }
        }
        unsigned t = b[27];
        for (int i = 0; i < 3; ++i) { c[125 + i] = (uint8_t)(t % 3); t /= 3; }
    }
    return 0;
}

/*
 * y[m][n] = sum_g f32(scale[n][g]) * (sum_{k in g} (c-1) * x[m][k]), FP32 throughout,
 * groups added in ascending order. Rows are independent, so contiguous row ranges
 * are handed to `threads` POSIX threads (<=0: one per online core).
 */
typedef struct {
    const uint8_t *blocks;
    const float *x;
    float *y;
    int M, N, K, n_begin, n_end;
    const float (*tab)[5];
} matmul_job;

static void *matmul_rows(void *arg) {
    const matmul_job *j = (const matmul_job *)arg;
    const int gpr = j->K / GROUP;
    for (int n = j->n_begin; n < j->n_end; ++n) {
        const uint8_t *row = j->blocks + (int64_t)n * gpr * BLOCK_BYTES;
        for (int m = 0; m < j->M; ++m) {
            const float *xm = j->x + (int64_t)m * j->K;
            float acc = 0.0f;
            for (int g = 0; g < gpr; ++g) {
                const uint8_t *b = row + g * BLOCK_BYTES;
                const float *xg = xm + g * GROUP;
                float dot = 0.0f;
                for (int s = 0; s < 25; ++s) {
                    /* callers validate first; the clamp only keeps the table read in bounds */
                    const float *t = j->tab[b[2 + s] > 242 ? 121 : b[2 + s]];
                    const float *xs = xg + 5 * s;
                    dot += t[0] * xs[0];
                    dot += t[1] * xs[1];
                    dot += t[2] * xs[2];
                    dot += t[3] * xs[3];
                    dot += t[4] * xs[4];
                }
                const float *t = j->tab[b[27] > 26 ? 13 : b[27]];
                dot += t[0] * xg[125];
                dot += t[1] * xg[126];
                dot += t[2] * xg[127];
                acc += dot * half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
            }
            j->y[(int64_t)m * j->N + n] = acc;
        }
    }
    return 0;
}

int tq1o_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

int tq1o_matmul_f32(const uint8_t *blocks, const float *x, float *y,
                    int M, int N, int K, int threads) {
    if (K % GROUP || M <= 0 || N <= 0) return -1;
    float tab[243][5];
    for (int v = 0; v < 243; ++v) {
        int r = v;
        for (int i = 0; i < 5; ++i) { tab[v][i] = (float)(r % 3 - 1); r /= 3; }
    }
    if (threads <= 0) threads = tq1o_threads();
    if (threads > N) threads = N;
    if (threads > 256) threads = 256;
    pthread_t tid[256];
    matmul_job jobs[256];
    for (int t = 0; t < threads; ++t) {
        matmul_job job = {blocks, x, y, M, N, K,
                          (int)((int64_t)N * t / threads), (int)((int64_t)N * (t + 1) / threads),
                          (const float (*)[5])tab};
        jobs[t] = job;
        if (t + 1 == threads) matmul_rows(&jobs[t]);
        else if (pthread_create(&tid[t], 0, matmul_rows, &jobs[t])) return -2;
    }
    for (int t = 0; t + 1 < threads; ++t) pthread_join(tid[t], 0);
    return 0;
}

/* out[t][k] = (c-1)*scale for row ids[t]; an id outside [0,V) gives a zero row. */
int tq1o_get_rows_f32(const uint8_t *blocks, const int64_t *ids, float *out,
                      int64_t T, int64_t V, int K) {
    if (K % GROUP) return -1;
    const int gpr = K / GROUP;
    for (int64_t t = 0; t < T; ++t) {
        float *o = out + t * K;
        if (ids[t] < 0 || ids[t] >= V) { memset(o, 0, sizeof(float) * (size_t)K); continue; }
        const uint8_t *row = blocks + ids[t] * gpr * BLOCK_BYTES;
        for (int g = 0; g < gpr; ++g) {
            const uint8_t *b = row + g * BLOCK_BYTES;
            float s = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
            for (int k = 0; k < GROUP; ++k) {
                unsigned v = k < 125 ? b[2 + k / 5] : b[27];
                int d = k < 125 ? k % 5 : k - 125;
                for (int i = 0; i < d; ++i) v /= 3;
                o[g * GROUP + k] = (float)((int)(v % 3) - 1) * s;
            }
        }
    }
    return 0;
}
