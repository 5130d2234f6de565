/*
 * CPU oracle for the FP8 GEMM family, the tiled sum-reduce and the FP8-encoded
 * allreduce.  TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA path and
 * the timed CPU baseline; no product code may call it.
 *
 * Parity status: the reference holds no golden vectors for these paths and its
 * host code is HIP (it needs <hip/hip_fp8.h>, which cannot be compiled without
 * the ROCm toolchain), so this restatement is "parity unpinned" against
 * reference outputs.  It is pinned instead against self-generated known-answer
 * vectors cross-checked with torch.float8_e4m3fn and ml_dtypes
 * (tests/golden/).
 *
 * What it follows in the reference (paths within the reference project):
 *   - GEMM arithmetic: projects/skinny_gemm/test.cu:23-38 - decode both fp8
 *     operands, multiply, accumulate sequentially in fp32 in k order, multiply
 *     by the scale once, cast once.  projects/async_gemm_16x16x64/test.cu:22-37
 *     is the same loop without the scale and with an fp32 result.
 *   - fp8 conversion: projects/common.cuh:103 - saturate-to-finite,
 *     round-to-nearest-even.  The reference byte format is AMD e4m3 FNUZ; the
 *     B200 tensor cores implement OCP e4m3fn, so the byte format here is
 *     e4m3fn (bias 7, max 448, NaN 0x7F/0xFF) with the same conversion rule.
 *   - sum reduce: projects/tiled_sum_reduce/test.cu:13-25.
 *   - comparison metric: projects/skinny_gemm/test.cu:94-107 (max / total
 *     absolute delta).
 *   - The FP8-encoded allreduce and the 2:4 pruning have no reference code;
 *     they restate the configuration text: per-128-element blocks, fp32 scale
 *     amax/448, e4m3fn saturating RN of x/scale, fp32 accumulation in rank
 *     order, one bf16 rounding; keep the 2 largest magnitudes of each group of
 *     4 along K (ties: lowest index).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ------------------------------------------------- minimal parallel-for */
/* Rows of independent work are spread over POSIX threads (the image has no
 * OpenMP runtime).  ORC_ORACLE_THREADS overrides the online-core count. */
typedef void (*orc_range_fn)(size_t lo, size_t hi, void *ctx);
typedef struct { orc_range_fn fn; void *ctx; size_t lo, hi; } orc_job;

int orc_num_threads(void)
{
    const char *e = getenv("ORC_ORACLE_THREADS");
    long n = e ? atol(e) : sysconf(_SC_NPROCESSORS_ONLN);
    if (n < 1) n = 1;
    if (n > 256) n = 256;
    return (int)n;
}

static void *orc_job_main(void *p) { orc_job *j = (orc_job *)p; j->fn(j->lo, j->hi, j->ctx); return NULL; }

static void orc_parallel_for(size_t n, orc_range_fn fn, void *ctx)
{
    int nt = orc_num_threads();
    if ((size_t)nt > n) nt = n ? (int)n : 1;
    if (nt <= 1) { fn(0, n, ctx); return; }
    pthread_t th[256];
    orc_job jobs[256];
    for (int t = 0; t < nt; t++) {
        jobs[t].fn = fn; jobs[t].ctx = ctx;
        jobs[t].lo = n * (size_t)t / nt; jobs[t].hi = n * (size_t)(t + 1) / nt;
        if (pthread_create(&th[t], NULL, orc_job_main, &jobs[t]) != 0) { fn(jobs[t].lo, jobs[t].hi, ctx); th[t] = 0; }
    }
    for (int t = 0; t < nt; t++) if (th[t]) pthread_join(th[t], NULL);
}

#define ORC_E4M3_MAX 448.0f

/* ------------------------------------------------------------------ codecs */

static float f32_from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinities;
 * S.1111.111 is NaN; largest finite S.1111.110 = 448; subnormal step 2^-9. */
float orc_e4m3fn_decode(uint8_t b)
{
    const int sign = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0xF && m == 7) return f32_from_bits(0x7FC00000u);
    if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf((float)(8 + m), e - 10);
    return sign ? -v : v;
}

/* Saturating round-to-nearest-even conversion (the __HIP_SATFINITE rule of
 * projects/common.cuh:103 applied to the e4m3fn grid).  NaN -> 0x7F. */
uint8_t orc_e4m3fn_encode(float x)
{
    const uint32_t u = f32_bits(x);
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    const float a = fabsf(x);
    if (x != x) return 0x7F;
    if (a >= ORC_E4M3_MAX) return sign | 0x7E;          /* saturate (also +-inf) */
    if (a < ldexpf(1.0f, -6)) {
        /* subnormal range: grid step 2^-9; rintf honours round-half-even */
        const float q = rintf(a * 512.0f);               /* exact scaling */
        return sign | (uint8_t)q;                        /* q == 8 lands on 0x08 = 2^-6 */
    }
    {
        int e;                                           /* a = f * 2^e, f in [0.5,1) */
        const float f = frexpf(a, &e);
        /* mantissa with 4 significant bits: f*16 in [8,16) */
        float q = rintf(f * 16.0f);
        int E = e - 1 + 7;                               /* biased exponent of 1.xxx form */
        if (q == 16.0f) { q = 8.0f; E += 1; }
        if (E > 15 || (E == 15 && q > 14.0f)) return sign | 0x7E;
        return sign | (uint8_t)((E << 3) | ((int)q - 8));
    }
}

/* bf16 = upper 16 bits of fp32, round-to-nearest-even; NaN stays NaN. */
uint16_t orc_bf16_encode(float x)
{
    uint32_t u = f32_bits(x);
    if (x != x) return (uint16_t)((u >> 16) | 0x0040);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float orc_bf16_decode(uint16_t h) { return f32_from_bits((uint32_t)h << 16); }

void orc_e4m3fn_decode_n(const uint8_t *q, float *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = orc_e4m3fn_decode(q[i]);
}

void orc_e4m3fn_encode_n(const float *x, uint8_t *q, size_t n)
{
    for (size_t i = 0; i < n; i++) q[i] = orc_e4m3fn_encode(x[i]);
}

void orc_bf16_encode_n(const float *x, uint16_t *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = orc_bf16_encode(x[i]);
}

/* --------------------------------------------------------------- quantisers */

/* Per-tensor: scale = amax/448 (1 when the tensor is all zero),
 * q = e4m3fn_sat_rn(x / scale) with an fp32 division. */
void orc_quantize_per_tensor(const float *x, size_t n, uint8_t *q, float *scale)
{
    float amax = 0.0f;
    for (size_t i = 0; i < n; i++) { const float a = fabsf(x[i]); if (a > amax) amax = a; }
    const float s = amax > 0.0f ? amax / ORC_E4M3_MAX : 1.0f;
    for (size_t i = 0; i < n; i++) q[i] = orc_e4m3fn_encode(x[i] / s);
    *scale = s;
}

/* Per-128-element blocks over a bf16 vector; n must be a multiple of 128.
 * scales[b] = amax_b/448 (1 for an all-zero block). */
void orc_quantize_blocks128(const uint16_t *x_bf16, size_t n, uint8_t *q, float *scales)
{
    for (size_t b = 0; b < n / 128; b++) {
        const uint16_t *xb = x_bf16 + b * 128;
        float amax = 0.0f;
        for (int i = 0; i < 128; i++) { const float a = fabsf(orc_bf16_decode(xb[i])); if (a > amax) amax = a; }
        const float s = amax > 0.0f ? amax / ORC_E4M3_MAX : 1.0f;
        for (int i = 0; i < 128; i++) q[b * 128 + i] = orc_e4m3fn_encode(orc_bf16_decode(xb[i]) / s);
        scales[b] = s;
    }
}

/* -------------------------------------------------------------------- GEMMs */

static void decode_table(float *t) { for (int i = 0; i < 256; i++) t[i] = orc_e4m3fn_decode((uint8_t)i); }

/* D[i,j] = bf16( (sum_k a[i,k]*b[j,k], sequential fp32) * (scale_a*scale_b) ).
 * A is [M,K] row-major, B is [N,K] with row pitch ldb (K-contiguous).
 * Products of two e4m3fn values are exact in fp32 (the reference multiplies
 * in fp16, exact for its FNUZ range; 448^2 needs fp32).  Rows are spread over
 * threads; each dot product stays sequential. */
typedef struct {
    const uint8_t *B; const float *Af; const float *lut; void *D; double *mag;
    const uint8_t *A; float scale; int M, N, K, ldb, out_bf16;
} gemm_ctx;

static void gemm_rows(size_t lo, size_t hi, void *p)
{
    const gemm_ctx *c = (const gemm_ctx *)p;
    const int K = c->K;
    float *bf = (float *)malloc((size_t)K * sizeof(float));
    for (size_t j = lo; j < hi; j++) {
        const uint8_t *b = c->B + j * (size_t)c->ldb;
        for (int l = 0; l < K; l++) bf[l] = c->lut[b[l]];
        for (int i = 0; i < c->M; i++) {
            const float *a = c->Af + (size_t)i * K;
            float acc = 0.0f;
            for (int l = 0; l < K; l++) acc += a[l] * bf[l];       /* sequential, k order */
            if (c->out_bf16) ((uint16_t *)c->D)[(size_t)i * c->N + j] = orc_bf16_encode(acc * c->scale);
            else ((float *)c->D)[(size_t)i * c->N + j] = acc;
        }
    }
    free(bf);
}

void orc_gemm_fp8_bf16(const uint8_t *A, const uint8_t *B, float scale_a, float scale_b,
                       uint16_t *D, int M, int N, int K, int ldb)
{
    float lut[256];
    decode_table(lut);
    float *Af = (float *)malloc((size_t)M * K * sizeof(float));
    for (size_t i = 0; i < (size_t)M * K; i++) Af[i] = lut[A[i]];
    gemm_ctx c = { B, Af, lut, D, NULL, A, scale_a * scale_b, M, N, K, ldb, 1 };
    orc_parallel_for((size_t)N, gemm_rows, &c);
    free(Af);
}

static void gemm64_rows(size_t lo, size_t hi, void *p)
{
    const gemm_ctx *c = (const gemm_ctx *)p;
    const double scale = (double)c->scale;
    for (size_t j = lo; j < hi; j++) {
        const uint8_t *b = c->B + j * (size_t)c->ldb;
        for (int i = 0; i < c->M; i++) {
            const uint8_t *a = c->A + (size_t)i * c->K;
            double acc = 0.0, am = 0.0;
            for (int l = 0; l < c->K; l++) {
                const double pr = (double)c->lut[a[l]] * (double)c->lut[b[l]];
                acc += pr;
                am += fabs(pr);
            }
            ((double *)c->D)[(size_t)i * c->N + j] = acc * scale;
            if (c->mag) c->mag[(size_t)i * c->N + j] = am * fabs(scale);
        }
    }
}

/* Same contraction accumulated in fp64, returned unrounded (already scaled):
 * the adjudicator for per-element ulp checks.  Also returns sum_k |a*b|*scale
 * in `mag` (may be NULL), the magnitude the fp32 summation-order error of any
 * implementation is proportional to. */
void orc_gemm_fp8_f64(const uint8_t *A, const uint8_t *B, float scale_a, float scale_b,
                      double *D, double *mag, int M, int N, int K, int ldb)
{
    float lut[256];
    decode_table(lut);
    gemm_ctx c = { B, NULL, lut, D, mag, A, scale_a * scale_b, M, N, K, ldb, 0 };
    orc_parallel_for((size_t)N, gemm64_rows, &c);
}

/* The async_gemm projects' oracle: fp32 result, no scale
 * (projects/async_gemm_16x16x64/test.cu:22-37). */
void orc_gemm_fp8_f32(const uint8_t *A, const uint8_t *B, float *D, int M, int N, int K)
{
    float lut[256];
    decode_table(lut);
    float *Af = (float *)malloc((size_t)M * K * sizeof(float));
    for (size_t i = 0; i < (size_t)M * K; i++) Af[i] = lut[A[i]];
    gemm_ctx c = { B, Af, lut, D, NULL, A, 1.0f, M, N, K, K, 0 };
    orc_parallel_for((size_t)N, gemm_rows, &c);
    free(Af);
}

/* --------------------------------------------------------------- sum reduce */

/* D[k] = sum_b (A[b,k] + B[b,k]) in batch order, fp32
 * (projects/tiled_sum_reduce/test.cu:13-25). */
void orc_tiled_sum_reduce(const float *A, const float *B, float *D, int b, int m, int n)
{
    const size_t mn = (size_t)m * n;
    for (size_t k = 0; k < mn; k++) D[k] = 0.0f;
    for (int ib = 0; ib < b; ib++) {
        for (size_t k = 0; k < mn; k++) D[k] += A[k] + B[k];
        A += mn;
        B += mn;
    }
}

/* ---------------------------------------------------------------- allreduce */

typedef struct {
    const uint16_t *xs; uint8_t *q; float *s; const float *lut; uint16_t *out;
    int nranks; size_t n, nb;
} ar_ctx;

static void ar_encode_blocks(size_t lo, size_t hi, void *p)
{
    const ar_ctx *c = (const ar_ctx *)p;     /* block index runs over [rank][block] */
    orc_quantize_blocks128(c->xs + lo * 128, (hi - lo) * 128, c->q + lo * 128, c->s + lo);
}

static void ar_reduce_blocks(size_t lo, size_t hi, void *p)
{
    const ar_ctx *c = (const ar_ctx *)p;
    for (size_t i = lo * 128; i < hi * 128; i++) {
        float acc = 0.0f;
        for (int r = 0; r < c->nranks; r++)
            acc += c->lut[c->q[(size_t)r * c->n + i]] * c->s[(size_t)r * c->nb + i / 128];
        c->out[i] = orc_bf16_encode(acc);
    }
}

/* out[i] = bf16( sum_{r=0..nranks-1} fp32(q_r[i]) * s_r[block(i)] ), summed in
 * rank order, where (q_r, s_r) is rank r's per-128-block encoding of x_r.
 * Every rank's contribution is encoded, the receiving rank's own included, so
 * all ranks produce identical bits.  xs is nranks consecutive bf16 vectors of
 * n elements.  q_out / s_out (may be NULL) receive the encodings
 * [nranks][n] and [nranks][n/128] for bit-exact comparison. */
void orc_allreduce_fp8(const uint16_t *xs, int nranks, size_t n, uint16_t *out,
                       uint8_t *q_out, float *s_out)
{
    const size_t nb = n / 128;
    uint8_t *q = q_out ? q_out : (uint8_t *)malloc((size_t)nranks * n);
    float *s = s_out ? s_out : (float *)malloc((size_t)nranks * nb * sizeof(float));
    float lut[256];
    decode_table(lut);
    ar_ctx c = { xs, q, s, lut, out, nranks, n, nb };
    orc_parallel_for((size_t)nranks * nb, ar_encode_blocks, &c);
    orc_parallel_for(nb, ar_reduce_blocks, &c);
    if (!q_out) free(q);
    if (!s_out) free(s);
}

/* --------------------------------------------------------------- 2:4 sparse */

/* Prune W [N,K] (fp32) in place: in each aligned group of 4 along K keep the 2
 * entries of largest magnitude (ties: lowest index) and zero the rest. */
void orc_prune_2of4(float *W, int N, int K)
{
    for (size_t g = 0; g < (size_t)N * K / 4; g++) {
        float *w = W + g * 4;
        int i0 = 0, i1 = -1;
        for (int i = 1; i < 4; i++) if (fabsf(w[i]) > fabsf(w[i0])) i0 = i;
        for (int i = 0; i < 4; i++) {
            if (i == i0) continue;
            if (i1 < 0 || fabsf(w[i]) > fabsf(w[i1])) i1 = i;
        }
        for (int i = 0; i < 4; i++) if (i != i0 && i != i1) w[i] = 0.0f;
    }
}

/* Compress a quantised 2:4 matrix Wq [N,K] into values [N,K/2] and 2-bit
 * positions: meta[N,K/4] holds (idx_hi << 2) | idx_lo per group, idx_lo <
 * idx_hi being the positions of the two kept values in ascending order.  A
 * group with fewer than two non-zero bytes keeps the lowest unused positions
 * so that the pair is always strictly ascending.  Returns the number of groups
 * that had more than two non-zero bytes (0 for a valid 2:4 matrix). */
int orc_compress_2of4(const uint8_t *Wq, int N, int K, uint8_t *vals, uint8_t *meta)
{
    int bad = 0;
    for (size_t g = 0; g < (size_t)N * K / 4; g++) {
        const uint8_t *w = Wq + g * 4;
        int idx[4], cnt = 0;
        for (int i = 0; i < 4; i++) if ((w[i] & 0x7F) != 0) idx[cnt++] = i;
        if (cnt > 2) { bad++; cnt = 2; }
        for (int i = 0; i < 4 && cnt < 2; i++) {
            int used = 0;
            for (int j = 0; j < cnt; j++) if (idx[j] == i) used = 1;
            if (!used) idx[cnt++] = i;
        }
        if (idx[0] > idx[1]) { const int t = idx[0]; idx[0] = idx[1]; idx[1] = t; }
        vals[g * 2 + 0] = w[idx[0]];
        vals[g * 2 + 1] = w[idx[1]];
        meta[g] = (uint8_t)((idx[1] << 2) | idx[0]);
    }
    return bad;
}

/* Inverse of orc_compress_2of4. */
void orc_expand_2of4(const uint8_t *vals, const uint8_t *meta, int N, int K, uint8_t *Wq)
{
    for (size_t g = 0; g < (size_t)N * K / 4; g++) {
        uint8_t *w = Wq + g * 4;
        w[0] = w[1] = w[2] = w[3] = 0;
        w[meta[g] & 3] = vals[g * 2 + 0];
        w[(meta[g] >> 2) & 3] = vals[g * 2 + 1];
    }
}

/* ------------------------------------------------------------------ metrics */

/* max and total absolute delta, as projects/skinny_gemm/test.cu:94-107. */
void orc_deltas(const float *x, const float *ref, size_t n, float *max_delta, float *total_delta)
{
    float mx = 0.0f, sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        const float d = fabsf(x[i] - ref[i]);
        sum += d;
        if (d > mx) mx = d;
    }
    *max_delta = mx;
    *total_delta = sum;
}
