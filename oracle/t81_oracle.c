/*
 * TEST INFRASTRUCTURE — NOT THE PRODUCT.  See t81_oracle.h for the contract,
 * the parity pin and the reference file:line each function follows.
 * Build: make -C oracle oracle   (gcc -O2 -ffp-contract=off, no fast-math).
 */
#include "t81_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>

/* Row-parallel helper (pthreads; the image has no OpenMP runtime).  The row
 * ranges are disjoint, so results do not depend on the thread count. */
static int g_threads = 1;
int t81o_num_threads(void) { return g_threads; }
void t81o_set_num_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }

typedef void (*range_fn)(int64_t lo, int64_t hi, void *ctx);
typedef struct { range_fn fn; int64_t lo, hi; void *ctx; } range_job;
static void *range_thunk(void *p) {
    range_job *j = (range_job *)p;
    j->fn(j->lo, j->hi, j->ctx);
    return NULL;
}
static void parallel_rows(int64_t n, range_fn fn, void *ctx) {
    int nt = g_threads;
    if (nt > n) nt = (int)(n > 0 ? n : 1);
    if (nt <= 1) { fn(0, n, ctx); return; }
    pthread_t tid[256];
    range_job job[256];
    for (int t = 0; t < nt; ++t) {
        job[t].fn = fn; job[t].ctx = ctx;
        job[t].lo = n * t / nt; job[t].hi = n * (t + 1) / nt;
        if (pthread_create(&tid[t], NULL, range_thunk, &job[t]) != 0) {
            fn(job[t].lo, job[t].hi, ctx); tid[t] = 0; job[t].fn = NULL;
        }
    }
    for (int t = 0; t < nt; ++t) if (job[t].fn) pthread_join(tid[t], NULL);
}

/* ---- codec: core/detail/lut.hpp:13-49 ---------------------------------- */

static inline uint8_t tryte_of(int t0, int t1, int t2) {
    return (uint8_t)(t0 + 3 * t1 + 9 * t2 + 13);
}

/* Inverse of tryte_of for b in 0..26: balanced digits of (b - 13). */
static inline void trits_of(uint8_t b, int8_t out[3]) {
    int v = (int)b - 13;
    for (int i = 0; i < 3; ++i) {
        int r = ((v % 3) + 3) % 3; /* 0,1,2 */
        int d = r == 2 ? -1 : r;
        out[i] = (int8_t)d;
        v = (v - d) / 3;
    }
}

int8_t t81o_quantize_trit(float value, float threshold) {
    /* std::clamp(value, -1, 1): NaN passes through and fails both compares. */
    float c = value;
    if (c < -1.0f) c = -1.0f;
    if (c > 1.0f) c = 1.0f;
    if (c >= threshold) return 1;
    if (c <= -threshold) return -1;
    return 0;
}

void t81o_quantize_to_trits(const float *src, size_t n, float threshold, int8_t *dst) {
    for (size_t i = 0; i < n; ++i) dst[i] = t81o_quantize_trit(src[i], threshold);
}

static void pack_limb(const int8_t trits[T81O_TRITS_PER_LIMB], uint8_t *dst) {
    for (int b = 0; b < T81O_BYTES_PER_LIMB; ++b)
        dst[b] = tryte_of(trits[3 * b], trits[3 * b + 1], trits[3 * b + 2]);
}

void t81o_pack_trits_rowwise(const int8_t *trits, int64_t rows, int64_t cols, uint8_t *packed) {
    const int64_t kl = (cols + 47) / 48;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t l = 0; l < kl; ++l) {
            int8_t t[T81O_TRITS_PER_LIMB];
            for (int i = 0; i < 48; ++i) {
                int64_t c = l * 48 + i;
                t[i] = c < cols ? trits[r * cols + c] : 0;
            }
            pack_limb(t, packed + (r * kl + l) * 16);
        }
}

void t81o_pack_trits_columnwise(const int8_t *trits, int64_t k, int64_t cols, uint8_t *packed) {
    const int64_t kl = (k + 47) / 48;
    for (int64_t l = 0; l < kl; ++l)
        for (int64_t c = 0; c < cols; ++c) {
            int8_t t[T81O_TRITS_PER_LIMB];
            for (int i = 0; i < 48; ++i) {
                int64_t kk = l * 48 + i;
                t[i] = kk < k ? trits[kk * cols + c] : 0;
            }
            pack_limb(t, packed + (l * cols + c) * 16);
        }
}

typedef struct {
    const float *w; int64_t cols, ld; float thr; uint8_t *packed; float *row_scale;
} pack_ctx;

static void pack_fixed_rows(int64_t lo, int64_t hi, void *p) {
    const pack_ctx *c = (const pack_ctx *)p;
    const int64_t kl = (c->cols + 47) / 48;
    for (int64_t r = lo; r < hi; ++r)
        for (int64_t l = 0; l < kl; ++l) {
            int8_t t[T81O_TRITS_PER_LIMB];
            for (int i = 0; i < 48; ++i) {
                int64_t col = l * 48 + i;
                t[i] = col < c->cols ? t81o_quantize_trit(c->w[r * c->ld + col], c->thr) : 0;
            }
            pack_limb(t, c->packed + (r * kl + l) * 16);
        }
}

void t81o_pack_dense_matrix(const float *w, int64_t rows, int64_t cols, int64_t ld,
                            float threshold, uint8_t *packed) {
    pack_ctx c = {w, cols, ld, threshold, packed, NULL};
    parallel_rows(rows, pack_fixed_rows, &c);
}

static float absmean_group_sum(const float *row, int64_t g, int64_t cols) {
    float v[4];
    for (int c = 0; c < 4; ++c) v[c] = 4 * g + c < cols ? fabsf(row[4 * g + c]) : 0.0f;
    volatile float lo = v[0] + v[1], hi = v[2] + v[3]; /* fp32, each sum rounded */
    volatile float s = lo + hi;
    return s;
}

static float absmean_row_scale(const float *row, int64_t cols) {
    const int64_t groups = (cols + 3) / 4;
    double part[T81O_ABSMEAN_LANES];
    for (int i = 0; i < T81O_ABSMEAN_LANES; ++i) part[i] = 0.0;
    /* chunks of 96 groups go round the four blocks of 32 partials; inside a chunk group j adds to partial j % 32 */
    for (int64_t g = 0; g < groups; ++g) {
        const int64_t chunk = g / 96;
        const int idx = (int)(chunk % (T81O_ABSMEAN_LANES / 32)) * 32 + (int)((g % 96) % 32);
        part[idx] += (double)absmean_group_sum(row, g, cols);
    }
    double grp[T81O_ABSMEAN_LANES / 32];
    for (int g = 0; g < T81O_ABSMEAN_LANES / 32; ++g) {
        double *v = part + 32 * g;
        for (int off = 16; off >= 1; off >>= 1)
            for (int j = 0; j < off; ++j) v[j] += v[j + off];
        grp[g] = v[0];
    }
    for (int off = T81O_ABSMEAN_LANES / 64; off >= 1; off >>= 1)
        for (int j = 0; j < off; ++j) grp[j] += grp[j + off];
    volatile float total = (float)grp[0], n = (float)cols;
    volatile float mean = total / n; /* fp32 division of the two rounded values */
    return mean;
}

static void pack_absmean_rows(int64_t lo, int64_t hi, void *p) {
    const pack_ctx *cx = (const pack_ctx *)p;
    const int64_t cols = cx->cols, kl = (cols + 47) / 48;
    const float threshold = cx->thr;
    uint8_t *packed = cx->packed;
    for (int64_t r = lo; r < hi; ++r) {
        const float *row = cx->w + r * cx->ld;
        const float s = cols > 0 ? absmean_row_scale(row, cols) : 0.0f;
        volatile float product = threshold * s; /* one fp32 multiply, rounded */
        const float cut = s > 0.0f ? product : INFINITY; /* a mean that is 0 or NaN: zero trits */
        if (cx->row_scale) cx->row_scale[r] = s;
        for (int64_t l = 0; l < kl; ++l) {
            int8_t t[T81O_TRITS_PER_LIMB];
            for (int i = 0; i < 48; ++i) {
                int64_t c = l * 48 + i;
                t[i] = 0;
                if (c < cols) t[i] = row[c] <= -cut ? -1 : (row[c] >= cut ? 1 : 0);
            }
            pack_limb(t, packed + (r * kl + l) * 16);
        }
    }
}

void t81o_pack_dense_matrix_absmean(const float *w, int64_t rows, int64_t cols, int64_t ld,
                                    float threshold, uint8_t *packed, float *row_scale) {
    pack_ctx c = {w, cols, ld, threshold, packed, row_scale};
    parallel_rows(rows, pack_absmean_rows, &c);
}

int t81o_unpack_packed_limbs(const uint8_t *packed, int64_t rows, int64_t k_limbs,
                             int64_t cols, int8_t *trits) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t l = 0; l < k_limbs; ++l) {
            const uint8_t *src = packed + (r * k_limbs + l) * 16;
            for (int b = 0; b < 16; ++b) {
                if (src[b] > 26) return -1;
                int8_t t[3];
                trits_of(src[b], t);
                for (int i = 0; i < 3; ++i) {
                    int64_t c = l * 48 + 3 * b + i;
                    if (c < cols) trits[r * cols + c] = t[i];
                }
            }
        }
    return 0;
}

/* ---- LIMB mode ---------------------------------------------------------- */

static void limb_trits(const uint8_t *limb, int8_t out[48]) {
    for (int b = 0; b < 16; ++b) trits_of(limb[b] > 26 ? 13 : limb[b], out + 3 * b);
}

/* include/t81/linalg/gemm.hpp:28-57: table[pos][tryte] with weight *= 27.0,
 * summed over the 16 positions in ascending order. */
static double g_contrib[16][27];
static int g_contrib_ready = 0;
static void build_contrib(void) {
    double weight = 1.0;
    for (int pos = 0; pos < 16; ++pos) {
        for (int b = 0; b < 27; ++b) {
            int8_t t[3];
            trits_of((uint8_t)b, t);
            g_contrib[pos][b] = t[0] * weight + t[1] * weight * 3.0 + t[2] * weight * 9.0;
        }
        weight *= 27.0;
    }
    g_contrib_ready = 1;
}

static double digits_to_double(const int *digits48) {
    double r = 0.0;
    for (int pos = 0; pos < 16; ++pos) {
        int b = digits48[3 * pos] + 3 * digits48[3 * pos + 1] + 9 * digits48[3 * pos + 2] + 13;
        r += g_contrib[pos][b];
    }
    return r;
}

/* core/detail/simd_impl.hpp:185-235 (mul_wide_scalar): 48x48 digit convolution,
 * carried to canonical balanced digits; gemm.hpp:58-64: low + high * 3^48. */
static double limb_product(const int8_t a[48], const int8_t b[48]) {
    int acc[97];
    memset(acc, 0, sizeof acc);
    for (int i = 0; i < 48; ++i) {
        if (!a[i]) continue;
        for (int j = 0; j < 48; ++j) acc[i + j] += a[i] * b[j];
    }
    for (int k = 0; k < 96; ++k) {
        int x = acc[k];
        int r = ((x % 3) + 3) % 3;
        int d = r == 2 ? -1 : r;
        acc[k] = d;
        acc[k + 1] += (x - d) / 3;
    }
    const double radix = 79766443076872509863361.0; /* 3^48 */
    return digits_to_double(acc) + digits_to_double(acc + 48) * radix;
}

typedef struct {
    const uint8_t *A; const int8_t *bt; float *C; int64_t N, k_limbs; float alpha, beta;
} limb_ctx;

static void gemm_limb_rows(int64_t lo, int64_t hi, void *p) {
    const limb_ctx *c = (const limb_ctx *)p;
    const int64_t N = c->N, k_limbs = c->k_limbs;
    for (int64_t i = lo; i < hi; ++i) {
        int8_t at[48];
        for (int64_t j = 0; j < N; ++j) {
            double acc = (double)c->C[i * N + j] * c->beta;
            for (int64_t k = 0; k < k_limbs; ++k) {
                limb_trits(c->A + (i * k_limbs + k) * 16, at);
                acc += limb_product(at, c->bt + (k * N + j) * 48) * (double)c->alpha;
            }
            c->C[i * N + j] = (float)acc;
        }
    }
}

void t81o_gemm_limb(const uint8_t *A, const uint8_t *B, float *C, int64_t M, int64_t N,
                    int64_t k_limbs, float alpha, float beta) {
    if (M == 0 || N == 0) return;
    if (!g_contrib_ready) build_contrib();
    int8_t *bt = (int8_t *)malloc((size_t)(k_limbs * N > 0 ? k_limbs * N : 1) * 48);
    for (int64_t i = 0; i < k_limbs * N; ++i) limb_trits(B + i * 16, bt + i * 48);
    limb_ctx c = {A, bt, C, N, k_limbs, alpha, beta};
    parallel_rows(M, gemm_limb_rows, &c);
    free(bt);
}

/* ---- TRIT mode ---------------------------------------------------------- */

typedef struct {
    const uint8_t *A; const float *B; float *C; int64_t N, K, ldb_k, ldb_n, ldc_m, ldc_n;
    float alpha, beta;
} trit_ctx;

static void gemm_trit_rows(int64_t lo, int64_t hi, void *p) {
    const trit_ctx *c = (const trit_ctx *)p;
    const int64_t N = c->N, K = c->K, kl = (K + 47) / 48;
    int8_t *t = (int8_t *)malloc((size_t)(kl > 0 ? kl : 1) * 48);
    double *acc = (double *)malloc((size_t)N * sizeof(double));
    for (int64_t i = lo; i < hi; ++i) {
        for (int64_t l = 0; l < kl; ++l) limb_trits(c->A + (i * kl + l) * 16, t + l * 48);
        for (int64_t j = 0; j < N; ++j)
            acc[j] = c->beta != 0.0f ? (double)c->C[i * c->ldc_m + j * c->ldc_n] * c->beta : 0.0;
        for (int64_t k = 0; k < K; ++k) {
            if (!t[k]) continue; /* adding an exact zero changes nothing */
            const double tv = (double)t[k];
            const float *brow = c->B + k * c->ldb_k;
            for (int64_t j = 0; j < N; ++j)
                acc[j] += tv * (double)brow[j * c->ldb_n] * (double)c->alpha;
        }
        for (int64_t j = 0; j < N; ++j) c->C[i * c->ldc_m + j * c->ldc_n] = (float)acc[j];
    }
    free(t);
    free(acc);
}

void t81o_gemm_trit(const uint8_t *A, const float *B, float *C, int64_t M, int64_t N, int64_t K,
                    int64_t ldb_k, int64_t ldb_n, int64_t ldc_m, int64_t ldc_n,
                    float alpha, float beta) {
    if (M == 0 || N == 0) return;
    trit_ctx c = {A, B, C, N, K, ldb_k, ldb_n, ldc_m, ldc_n, alpha, beta};
    parallel_rows(M, gemm_trit_rows, &c);
}

typedef struct {
    const uint8_t *W; const float *row_scale, *bias, *x; float *y;
    int64_t tokens, out_features, in_features;
} lin_ctx;

static void linear_rows(int64_t lo, int64_t hi, void *p) {
    const lin_ctx *c = (const lin_ctx *)p;
    const int64_t in_features = c->in_features, kl = (in_features + 47) / 48;
    int8_t *t = (int8_t *)malloc((size_t)(kl > 0 ? kl : 1) * 48);
    for (int64_t o = lo; o < hi; ++o) {
        for (int64_t l = 0; l < kl; ++l) limb_trits(c->W + (o * kl + l) * 16, t + l * 48);
        for (int64_t m = 0; m < c->tokens; ++m) {
            const float *xr = c->x + m * in_features;
            double acc = 0.0;
            for (int64_t k = 0; k < in_features; ++k)
                if (t[k]) acc += (double)t[k] * (double)xr[k];
            if (c->row_scale) acc *= (double)c->row_scale[o];
            if (c->bias) acc += (double)c->bias[o];
            c->y[m * c->out_features + o] = (float)acc;
        }
    }
    free(t);
}

void t81o_linear_forward(const uint8_t *W, const float *row_scale, const float *bias,
                         const float *x, float *y, int64_t tokens, int64_t out_features,
                         int64_t in_features) {
    lin_ctx c = {W, row_scale, bias, x, y, tokens, out_features, in_features};
    parallel_rows(out_features, linear_rows, &c);
}
