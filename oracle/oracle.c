/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement, in plain C, of the definition of the reference's integer-exact FP32 GEMM.
 * It exists so the tests, the smoke check and the CPU-baseline leg of the benchmark have an
 * independent checker for the CUDA path.  Nothing in the shipped library calls into this file.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks this file against
 *   - the known-answer vectors of the three scalar functions (tests/golden/scalar_vectors.json,
 *     produced by calling the reference's own repro_gemm_math.cuh functions),
 *   - the FNV-1a-64 output hashes the reference commits for its 21 GPT-2-shaped GEMM operations
 *     (gpt2_ops_suite/results/<machine>/cpu.txt, lines 2-22; identical in every committed result file),
 *   - the reference's cpu_gemm compiled from its own sources (oracle/_ref) wherever that
 *     library has been built.
 *
 * What each function follows in the reference (paths inside the reference project):
 *   orc_scale_exponent   repro_gemm_cuda/repro_gemm_math.cuh:59-69
 *   orc_fixed_point      repro_gemm_cuda/repro_gemm_math.cuh:47-55, 74-83
 *   orc_round_to_float   repro_gemm_cuda/repro_gemm_math.cuh:96-119
 *   orc_gemm             repro_gemm_cuda/repro_gemm_cpu.h:25-51
 *   orc_gemm_partial     same dot products, cut to a k-range and left unrounded (what a K-shard holds)
 *   orc_round_partials   repro_gemm_cuda/repro_gemm.cu:156-165
 *   orc_conv2d*          repro_conv_cuda/repro_conv_math.cuh:10-17, repro_conv_cpu.h:25-90 (pinned against
 *                        the reference's cpu_conv2d* through tests/golden/conv_hashes.json and oracle/_ref)
 *   orc_fnv1a64          repro_gemm_cuda/repro_test_util.h:20-24
 *   orc_rng_* / fills    repro_gemm_cuda/repro_test_util.h:30-48, gpt2_ops_suite/gpt2_ops_suite.cu:59-76
 *
 * Build: see oracle/Makefile (no fast-math, no FMA contraction; both are part of the definition).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static uint32_t f2u(float x) { uint32_t b; memcpy(&b, &x, 4); return b; }
static float u2f(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }
static float pow2f(int n) { return u2f((uint32_t)(n + 127) << 23); } /* n in [-126, 127] */

/* ------------------------------------------------------------------------------------------
 * Scalar definition
 * ---------------------------------------------------------------------------------------- */

/* Smallest integer e with 2^e >= RN32(m / 127); 0 when m <= 0 or when the quotient is zero. */
int orc_scale_exponent(float m) {
    if (!(m > 0.0f)) return 0;
    volatile float q = m / 127.0f; /* one IEEE division, kept out of the optimiser's hands */
    uint32_t b = f2u(q);
    uint32_t expo = (b >> 23) & 0xFFu, frac = b & 0x7FFFFFu;
    if (expo != 0) return (int)expo - 127 + (frac != 0);
    if (frac == 0) return 0;               /* the quotient underflowed to zero */
    int top = 31 - __builtin_clz(frac);    /* subnormal: q = frac * 2^-149 */
    return top - 149 + ((frac & (frac - 1)) != 0);
}

/* RNE(x * 2^(7(S-1) - se)) clamped to +-127 * 2^(7(S-1)).  The scaling is exact wherever the
 * result can be non-zero, so there is exactly one rounding, the conversion to integer. */
int orc_fixed_point(float x, int se, int S) {
    int n = 7 * (S - 1) - se;
    /* 2^n can exceed the float range only upwards (n <= 163); split off the excess. */
    int n_first = n > 127 ? 127 : n, n_rest = n - n_first;
    volatile float v = x * pow2f(n_first);
    v = v * pow2f(n_rest);
    int lim = 127 << (7 * (S - 1));
    float r = nearbyintf(v);               /* default rounding mode: to nearest, ties to even */
    if (r > (float)lim) return lim;
    if (r < (float)-lim) return -lim;
    return (int)r;
}

/* Shift right by s (1..63) with round-to-nearest, ties-to-even. */
static uint64_t shr_rne(uint64_t m, int s) {
    uint64_t q = m >> s, rest = m & ((1ull << s) - 1), half = 1ull << (s - 1);
    return q + (rest > half || (rest == half && (q & 1)));
}

/* Correctly rounded (nearest-even) binary32 of the exact value T * 2^E, built directly as a bit
 * pattern: subnormals, overflow to infinity, +0 for T == 0 and -0 for a negative value that
 * rounds to zero. */
uint32_t orc_round_to_float_bits(int64_t T, int E) {
    if (T == 0) return 0;
    uint32_t sign = T < 0 ? 0x80000000u : 0;
    uint64_t m = T < 0 ? 0 - (uint64_t)T : (uint64_t)T;
    int p = 63 - __builtin_clzll(m);       /* leading bit of m */
    int e = p + E;                          /* ... and of the value */
    if (e > 127) return sign | 0x7F800000u;
    if (e >= -126) {                        /* normal range: keep 24 significant bits */
        int s = p - 23;
        uint64_t q = s <= 0 ? m << -s : shr_rne(m, s);
        if (q == (1ull << 24)) { q >>= 1; ++e; }
        if (e > 127) return sign | 0x7F800000u;
        return sign | ((uint32_t)(e + 127) << 23) | ((uint32_t)q & 0x7FFFFFu);
    }
    /* below the normal range: count units of 2^-149 */
    int s = -(E + 149);
    uint64_t q = s <= 0 ? m << -s : (s >= 64 ? 0 : shr_rne(m, s));
    return sign | (uint32_t)q;              /* q == 2^23 encodes the smallest normal, as it should */
}

float orc_round_to_float(int64_t T, int E) { return u2f(orc_round_to_float_bits(T, E)); }

/* Balanced base-128 digits of X, most significant first: X = sum d[p] * 128^(S-1-p),
 * |d[0]| <= 127, d[p>0] in [-64, 63]  (repro_gemm_cuda/repro_gemm.cu:20-21, 41-46). */
void orc_digits(int X, int S, int8_t* d) {
    for (int p = S - 1; p >= 1; --p) {
        int low = ((X + 64) & 127) - 64;
        d[p] = (int8_t)low;
        X = (X - low) >> 7;
    }
    d[0] = (int8_t)X;
}

/* ------------------------------------------------------------------------------------------
 * Thread pool helper
 * ---------------------------------------------------------------------------------------- */
typedef void (*row_fn)(int i, void* ctx);
typedef struct { int n; volatile int next; row_fn fn; void* ctx; } job_t;

static void* worker(void* arg) {
    job_t* j = (job_t*)arg;
    for (;;) {
        int i = __sync_fetch_and_add(&j->next, 1);
        if (i >= j->n) break;
        j->fn(i, j->ctx);
    }
    return NULL;
}

static void parallel_for(int n, int threads, row_fn fn, void* ctx) {
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    job_t j = {n, 0, fn, ctx};
    pthread_t tid[256];
    for (int t = 1; t < threads; ++t) pthread_create(&tid[t], NULL, worker, &j);
    worker(&j);
    for (int t = 1; t < threads; ++t) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------------------------------
 * GEMM
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    const float *A, *B;
    float* C;
    int64_t* T;
    int M, N, K, ta, tb, S, k0, k1;
    int *eA, *eB;
    int32_t *X, *Y;
    const float *maxA, *maxB; /* optional externally supplied max |.| per row / column */
} gemm_t;

static float a_at(const gemm_t* g, int r, int k) {
    return g->ta ? g->A[(size_t)k * g->M + r] : g->A[(size_t)r * g->K + k];
}
static float b_at(const gemm_t* g, int k, int c) {
    return g->tb ? g->B[(size_t)c * g->K + k] : g->B[(size_t)k * g->N + c];
}

static void quant_a(int r, void* ctx) {
    gemm_t* g = (gemm_t*)ctx;
    float m = 0.0f;
    if (g->maxA) m = g->maxA[r];
    else for (int k = 0; k < g->K; ++k) m = fmaxf(m, fabsf(a_at(g, r, k)));
    g->eA[r] = orc_scale_exponent(m);
    for (int k = 0; k < g->K; ++k) g->X[(size_t)r * g->K + k] = orc_fixed_point(a_at(g, r, k), g->eA[r], g->S);
}
static void quant_b(int c, void* ctx) {
    gemm_t* g = (gemm_t*)ctx;
    float m = 0.0f;
    if (g->maxB) m = g->maxB[c];
    else for (int k = 0; k < g->K; ++k) m = fmaxf(m, fabsf(b_at(g, k, c)));
    g->eB[c] = orc_scale_exponent(m);
    for (int k = 0; k < g->K; ++k) g->Y[(size_t)c * g->K + k] = orc_fixed_point(b_at(g, k, c), g->eB[c], g->S);
}
static void dot_rows(int r, void* ctx) {
    gemm_t* g = (gemm_t*)ctx;
    const int32_t* x = g->X + (size_t)r * g->K;
    for (int c = 0; c < g->N; ++c) {
        const int32_t* y = g->Y + (size_t)c * g->K;
        int64_t t = 0;
        for (int k = g->k0; k < g->k1; ++k) t += (int64_t)x[k] * y[k];
        if (g->T) g->T[(size_t)r * g->N + c] = t;
        else g->C[(size_t)r * g->N + c] = orc_round_to_float(t, g->eA[r] + g->eB[c] - 14 * (g->S - 1));
    }
}

static int run_gemm(gemm_t* g, int threads) {
    g->eA = (int*)malloc(sizeof(int) * (size_t)g->M);
    g->eB = (int*)malloc(sizeof(int) * (size_t)g->N);
    g->X = (int32_t*)malloc(sizeof(int32_t) * (size_t)g->M * g->K);
    g->Y = (int32_t*)malloc(sizeof(int32_t) * (size_t)g->N * g->K);
    int ok = g->eA && g->eB && g->X && g->Y;
    if (ok) {
        parallel_for(g->M, threads, quant_a, g);
        parallel_for(g->N, threads, quant_b, g);
        parallel_for(g->M, threads, dot_rows, g);
    }
    free(g->eA); free(g->eB); free(g->X); free(g->Y);
    return ok ? 0 : -1;
}

/* C[M,N] = op(A)[M,K] * op(B)[K,N].  ta: A stored K x M.  tb: B stored N x K.  Row-major. */
int orc_gemm(const float* A, const float* B, float* C, int M, int N, int K, int ta, int tb, int S, int threads) {
    gemm_t g;
    memset(&g, 0, sizeof g);
    g.A = A; g.B = B; g.C = C; g.M = M; g.N = N; g.K = K; g.ta = ta; g.tb = tb; g.S = S; g.k0 = 0; g.k1 = K;
    return run_gemm(&g, threads);
}

/* Unrounded exact sums over k in [k0, k1) with the scales fixed by the given row/column maxima
 * (taken over the whole K): what one rank of a K-split holds before the integer reduction. */
int orc_gemm_partial(const float* A, const float* B, int64_t* T, const float* maxA, const float* maxB,
                     int M, int N, int K, int ta, int tb, int S, int k0, int k1, int threads) {
    gemm_t g;
    memset(&g, 0, sizeof g);
    g.A = A; g.B = B; g.T = T; g.M = M; g.N = N; g.K = K; g.ta = ta; g.tb = tb; g.S = S; g.k0 = k0; g.k1 = k1;
    g.maxA = maxA; g.maxB = maxB;
    return run_gemm(&g, threads);
}

/* max |x| over k for every row of op(A) (rows = M, ta) or every column of op(B) (rows = N, !tb). */
void orc_absmax(const float* src, float* out, int R, int K, int k_strided) {
    for (int r = 0; r < R; ++r) {
        float m = 0.0f;
        for (int k = 0; k < K; ++k) m = fmaxf(m, fabsf(k_strided ? src[(size_t)k * R + r] : src[(size_t)r * K + k]));
        out[r] = m;
    }
}

/* C = round(sum over `parts` integer partials, scaled by the row/column exponents). */
void orc_round_partials(const int64_t* T, int parts, const float* maxA, const float* maxB, float* C,
                        int M, int N, int S) {
    for (int r = 0; r < M; ++r)
        for (int c = 0; c < N; ++c) {
            int64_t t = 0;
            for (int p = 0; p < parts; ++p) t += T[((size_t)p * M + r) * N + c];
            int E = orc_scale_exponent(maxA[r]) + orc_scale_exponent(maxB[c]) - 14 * (S - 1);
            C[(size_t)r * N + c] = orc_round_to_float(t, E);
        }
}

/* ------------------------------------------------------------------------------------------
 * Convolution (repro_conv_cuda/repro_conv_math.cuh:10-17, repro_conv_cpu.h:25-90).
 * shape = {N, C, H, W, F, KH, KW, SY, SX, PY, PX}.  Forward and weight gradient are restated the
 * way the reference's own test states them (test_repro_conv.cu:84-112): the GEMM definition on the
 * im2col matrix.  The input gradient is restated directly: dY scaled per image, all weights with
 * one scale, exact integer sum over the taps that touch a pixel, one rounding.
 * ---------------------------------------------------------------------------------------- */
typedef struct { int N, C, H, W, F, KH, KW, SY, SX, PY, PX, OH, OW, K; } conv_t;

static conv_t conv_shape(const int* s) {
    conv_t g = {s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[7], s[8], s[9], s[10], 0, 0, 0};
    g.OH = (g.H + 2 * g.PY - g.KH) / g.SY + 1;
    g.OW = (g.W + 2 * g.PX - g.KW) / g.SX + 1;
    g.K = g.C * g.KH * g.KW;
    return g;
}

/* X[w][k]: value at position k = (c, ky, kx) of window w = (n, oy, ox); zero in the padding. */
static float* conv_im2col(const float* x, const conv_t* g) {
    size_t windows = (size_t)g->N * g->OH * g->OW;
    float* X = (float*)malloc(sizeof(float) * windows * g->K);
    if (!X) return NULL;
    size_t at = 0;
    for (int n = 0; n < g->N; ++n)
        for (int oy = 0; oy < g->OH; ++oy)
            for (int ox = 0; ox < g->OW; ++ox)
                for (int c = 0; c < g->C; ++c)
                    for (int ky = 0; ky < g->KH; ++ky)
                        for (int kx = 0; kx < g->KW; ++kx) {
                            int y = oy * g->SY - g->PY + ky, xx = ox * g->SX - g->PX + kx;
                            X[at++] = (y < 0 || y >= g->H || xx < 0 || xx >= g->W)
                                          ? 0.0f : x[(((size_t)n * g->C + c) * g->H + y) * g->W + xx];
                        }
    return X;
}

int orc_conv2d(const float* x, const float* w, float* out, const int* shape, int S, int threads) {
    conv_t g = conv_shape(shape);
    int per = g.OH * g.OW, windows = g.N * per;
    float* X = conv_im2col(x, &g);
    float* Y = (float*)malloc(sizeof(float) * (size_t)windows * g.F);
    int rc = (X && Y) ? orc_gemm(X, w, Y, windows, g.F, g.K, 0, 1, S, threads) : -1;   /* Y = X W^T */
    if (rc == 0)
        for (int i = 0; i < windows; ++i)
            for (int f = 0; f < g.F; ++f)
                out[((size_t)(i / per) * g.F + f) * per + i % per] = Y[(size_t)i * g.F + f];
    free(X); free(Y);
    return rc;
}

int orc_conv2d_grad_weight(const float* dy, const float* x, float* dw, const int* shape, int S, int threads) {
    conv_t g = conv_shape(shape);
    int per = g.OH * g.OW, windows = g.N * per;
    float* X = conv_im2col(x, &g);
    float* D = (float*)malloc(sizeof(float) * (size_t)windows * g.F);
    int rc = -1;
    if (X && D) {
        for (int i = 0; i < windows; ++i)
            for (int f = 0; f < g.F; ++f)
                D[(size_t)i * g.F + f] = dy[((size_t)(i / per) * g.F + f) * per + i % per];
        rc = orc_gemm(D, X, dw, g.F, g.K, windows, 1, 0, S, threads);                  /* dW = D^T X */
    }
    free(X); free(D);
    return rc;
}

typedef struct { conv_t g; const int32_t *D, *Wq; const int* eI; int eW, S; float* dx; } conv_dx_t;

static void conv_dx_plane(int i, void* ctx) {     /* one (n, c) plane of dX */
    conv_dx_t* t = (conv_dx_t*)ctx;
    const conv_t* g = &t->g;
    int n = i / g->C, c = i % g->C;
    for (int y = 0; y < g->H; ++y)
        for (int xx = 0; xx < g->W; ++xx) {
            int64_t sum = 0;
            for (int ky = 0; ky < g->KH; ++ky) {
                int ry = y + g->PY - ky;
                if (ry < 0 || ry % g->SY != 0 || ry / g->SY >= g->OH) continue;
                for (int kx = 0; kx < g->KW; ++kx) {
                    int rx = xx + g->PX - kx;
                    if (rx < 0 || rx % g->SX != 0 || rx / g->SX >= g->OW) continue;
                    for (int f = 0; f < g->F; ++f)
                        sum += (int64_t)t->D[(((size_t)n * g->F + f) * g->OH + ry / g->SY) * g->OW + rx / g->SX] *
                               t->Wq[(((size_t)f * g->C + c) * g->KH + ky) * g->KW + kx];
                }
            }
            t->dx[(((size_t)n * g->C + c) * g->H + y) * g->W + xx] =
                orc_round_to_float(sum, t->eI[n] + t->eW - 14 * (t->S - 1));
        }
}

int orc_conv2d_grad_input(const float* dy, const float* w, float* dx, const int* shape, int S, int threads) {
    conv_dx_t t;
    t.g = conv_shape(shape);
    size_t per = (size_t)t.g.F * t.g.OH * t.g.OW, nw = (size_t)t.g.F * t.g.K;
    int32_t* D = (int32_t*)malloc(sizeof(int32_t) * per * t.g.N);
    int32_t* Wq = (int32_t*)malloc(sizeof(int32_t) * nw);
    int* eI = (int*)malloc(sizeof(int) * (size_t)t.g.N);
    int ok = D && Wq && eI;
    if (ok) {
        for (int n = 0; n < t.g.N; ++n) {          /* dY: one scale per image */
            float m = 0.0f;
            for (size_t i = 0; i < per; ++i) m = fmaxf(m, fabsf(dy[n * per + i]));
            eI[n] = orc_scale_exponent(m);
            for (size_t i = 0; i < per; ++i) D[n * per + i] = orc_fixed_point(dy[n * per + i], eI[n], S);
        }
        float mw = 0.0f;                           /* weights: one scale for all */
        for (size_t i = 0; i < nw; ++i) mw = fmaxf(mw, fabsf(w[i]));
        t.eW = orc_scale_exponent(mw);
        for (size_t i = 0; i < nw; ++i) Wq[i] = orc_fixed_point(w[i], t.eW, S);
        t.D = D; t.Wq = Wq; t.eI = eI; t.S = S; t.dx = dx;
        parallel_for(t.g.N * t.g.C, threads, conv_dx_plane, &t);
    }
    free(D); free(Wq); free(eI);
    return ok ? 0 : -1;
}

/* ------------------------------------------------------------------------------------------
 * Fixtures: FNV-1a-64 and the SplitMix64 input generators
 * ---------------------------------------------------------------------------------------- */
uint64_t orc_fnv1a64(const void* data, size_t n, uint64_t h) {
    const unsigned char* p = (const unsigned char*)data;
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 0x100000001b3ull; }
    return h;
}

static uint64_t rng_next(uint64_t* s) {
    uint64_t z = (*s += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
static double rng_u01(uint64_t* s) { return (double)(rng_next(s) >> 40) * (1.0 / 16777216.0); }
static double rng_normal(uint64_t* s) { double t = 0; for (int i = 0; i < 12; ++i) t += rng_u01(s); return t - 6.0; }
static int rng_range(uint64_t* s, int lo, int hi) { return lo + (int)(rng_next(s) % (uint64_t)(hi - lo + 1)); }
static float rng_wide(uint64_t* s, int elo, int ehi) {
    double mant = 1.0 + rng_u01(s);
    double v = ldexp(mant, rng_range(s, elo, ehi));
    return (float)((rng_next(s) & 1) ? -v : v);
}

/* Every fill continues from *state and leaves the advanced state behind, so one generator can be
 * drawn from for A and then for B exactly as the reference's tools do. */
void orc_fill_uniform_pm1(float* out, size_t n, uint64_t* state) {
    for (size_t i = 0; i < n; ++i) out[i] = (float)(2.0 * rng_u01(state) - 1.0);
}
void orc_fill_normal(float* out, size_t n, double scale, uint64_t* state) {
    for (size_t i = 0; i < n; ++i) out[i] = (float)(scale * rng_normal(state));
}
void orc_fill_u01(float* out, size_t n, double scale, uint64_t* state) {
    for (size_t i = 0; i < n; ++i) out[i] = (float)(scale * rng_u01(state));
}
void orc_fill_wide(float* out, size_t n, int elo, int ehi, uint64_t* state) {
    for (size_t i = 0; i < n; ++i) out[i] = rng_wide(state, elo, ehi);
}
/* Wide dynamic range with exact zeros (1 %) and subnormals (0.1 %).  Four draws per element, always:
 * r = next() % 1000, mantissa m = 1 + u01(), exponent word w = next(), sign bit = next() & 1.
 * r < 10 -> +0; r == 10 -> a subnormal, +-m * 2^(-149 + w % 23); else +-m * 2^(elo + w % (ehi-elo+1)). */
void orc_fill_wide_mixed(float* out, size_t n, int elo, int ehi, uint64_t* state) {
    for (size_t i = 0; i < n; ++i) {
        uint64_t r = rng_next(state) % 1000;
        double mant = 1.0 + rng_u01(state);
        uint64_t w = rng_next(state);
        int neg = (int)(rng_next(state) & 1);
        int e = r == 10 ? -149 + (int)(w % 23) : elo + (int)(w % (uint64_t)(ehi - elo + 1));
        double v = ldexp(mant, e);
        out[i] = r < 10 ? 0.0f : (float)(neg ? -v : v);
    }
}
/* Row-softmax-like matrix: u = u01 + 2^-25 per entry, row sum in double in index order, p = u / sum. */
void orc_fill_prob_rows(float* out, size_t rows, size_t cols, uint64_t* state) {
    double* u = (double*)malloc(sizeof(double) * cols);
    for (size_t r = 0; r < rows; ++r) {
        double sum = 0.0;
        for (size_t c = 0; c < cols; ++c) { u[c] = rng_u01(state) + 1.0 / 33554432.0; sum += u[c]; }
        for (size_t c = 0; c < cols; ++c) out[r * cols + c] = (float)(u[c] / sum);
    }
    free(u);
}
