/*
 * blaze_oracle.c -- CPU restatement of the Blaze GEMM hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA library: tests, the smoke entry and the bench's
 * cpu_baseline leg call it; the product library never links or loads it.
 *
 * What it restates (paths are inside the Blaze project):
 *   - the host reference GEMM: tests/test_gemm_naive.cu:38-48 (gemm_cpu_fp16): fp32 accumulator,
 *     loop nest i, j, kk with kk innermost and ascending, sum += a*b with no fused multiply-add;
 *   - block-scaled semantics: D = sum_k (a*sfa)(b*sfb), then times tensor_scale_A*tensor_scale_B
 *     (include/gemm/tmem_utils.cuh:551-554, src/kernels/gemm_fp4_blkscaled_sm100.cu:280,291);
 *   - E2M1 magnitudes {0,.5,1,1.5,2,3,4,6} (include/gemm/fp4_gemm_sm100.cuh:26-28), one E4M3
 *     scale per 16 values along K (include/gemm/fp4_blkscaled_gemm_sm100.cuh:43);
 *   - epilogue order scale -> bias -> SiLU / residual -> narrow
 *     (src/kernels/gemm_mixed_sm100.cu:202-229, SiLU = x/(1+exp(-x)) as gemm_fp8_sm100.cu:171);
 *   - the seeded fill (tests/test_gemm_naive.cu:50-56): srand(seed); (rand()/RAND_MAX-0.5)*2.
 *
 * Quantisers are not part of Blaze (its quantiser phase is absent); they are defined here:
 *   FP8   : s = 448/amax(X); q = e4m3_rn(x*s); C = (sum qa*qb) * (1/(s_a*s_b))
 *   NVFP4 : g = amax(X)/(6*448); per 16 values along K: sf = e4m3_rn((amax_blk/6)/g);
 *           q = e2m1_rn(x/(g*float(sf))), zero when sf is zero; dequantised x^ = q*sf*g.
 * Packed nibbles: even K index in the low nibble, odd K index in the high nibble.
 *
 * Pins: the number formats are checked against CUDA's host conversions (pin_formats.cu), the
 * GEMM loop against Blaze's own gemm_cpu_fp16 compiled from its source (oracle/_ref) and the
 * committed golden vectors it produced, plus the byte patterns Blaze's tests use
 * (0x38 = 1.0, 0x3C = 1.5 in E4M3; 0x2 = 1.0, 0x5 = 3.0 in E2M1; tests/test_gemm.cu:193-194,338-342).
 * Seeded-random results of Blaze's tcgen05 kernels are not pinned by Blaze's own tests.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ formats */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float blzo_f16_to_f32(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023;
    if (e == 0) {
        if (m == 0) return u2f(s);
        float v = (float)m * (1.0f / 16777216.0f); /* m * 2^-24 */
        return s ? -v : v;
    }
    if (e == 31) return u2f(s | 0x7f800000u | (m << 13));
    return u2f(s | ((e + 112) << 23) | (m << 13));
}

/* round-to-nearest-even fp32 -> fp16; satfinite != 0 clamps finite overflow to +-65504 */
uint16_t blzo_f32_to_f16_ex(float f, int satfinite) {
    uint32_t u = f2u(f), s = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(s | 0x7fffu);            /* NaN */
    if (a == 0x7f800000u) return (uint16_t)(s | (satfinite ? 0x7bffu : 0x7c00u));
    if (a >= 0x477ff000u) return (uint16_t)(s | (satfinite ? 0x7bffu : 0x7c00u)); /* >= 65520 rounds to inf */
    if (a < 0x33000001u) return (uint16_t)s;                        /* <= 2^-25 rounds to zero */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;                   /* bits dropped from the 24-bit significand */
    uint32_t kept = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1))) kept++;
    uint32_t out = (e < -14) ? kept : (((uint32_t)(e + 15) << 10) + (kept - 1024u));
    return (uint16_t)(s | out);
}
uint16_t blzo_f32_to_f16(float f) { return blzo_f32_to_f16_ex(f, 0); }

float blzo_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }
uint16_t blzo_f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

/* E4M3 (finite-only "fn" flavour): bias 7, max 448, 0x7f/0xff = NaN, no infinities. */
float blzo_e4m3_to_f32(uint8_t b) {
    uint32_t e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) return u2f(0x7fc00000u | ((uint32_t)(b & 0x80) << 24));
    if (e == 0) v = (float)m * 0.001953125f;                        /* m * 2^-9 */
    else v = u2f(((e + 120) << 23) | (m << 20));
    return (b & 0x80) ? -v : v;
}
/* round-to-nearest-even, saturating to +-448; NaN -> 0x7f */
uint8_t blzo_f32_to_e4m3(float f) {
    uint32_t u = f2u(f), a = u & 0x7fffffffu;
    uint8_t s = (uint8_t)((u >> 24) & 0x80);
    if (a > 0x7f800000u) return (uint8_t)(s | 0x7f);
    float x = u2f(a);
    if (x >= 464.0f) return (uint8_t)(s | 0x7e);                    /* above the 448/480 midpoint region saturates */
    if (x > 448.0f) return (uint8_t)(s | 0x7e);
    /* scale so that one unit is the spacing at the value's binade */
    int e;
    if (x < 0.015625f) {                                            /* below 2^-6: subnormal spacing 2^-9 */
        float q = x * 512.0f;
        float r = nearbyintf(q);                                    /* ties-to-even under the default rounding mode */
        uint32_t m = (uint32_t)r;                                   /* 0..8 */
        if (m >= 8) return (uint8_t)(s | 0x08);
        return (uint8_t)(s | m);
    }
    (void)frexpf(x, &e);                                            /* x = f*2^e, f in [0.5,1) -> exponent e-1 */
    int ex = e - 1;                                                 /* -6..8 */
    float q = ldexpf(x, 3 - ex);                                    /* in [8,16) */
    float r = nearbyintf(q);
    uint32_t m = (uint32_t)r;                                       /* 8..16 */
    if (m == 16) { m = 8; ex++; }
    if (ex > 8 || (ex == 8 && m > 14)) return (uint8_t)(s | 0x7e);
    return (uint8_t)(s | ((uint32_t)(ex + 7) << 3) | (m - 8));
}

/* E2M1: 1 sign, 2 exponent, 1 mantissa; magnitudes 0,.5,1,1.5,2,3,4,6. */
static const float E2M1_MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
float blzo_e2m1_to_f32(uint8_t n) {
    float v = E2M1_MAG[n & 7];
    return (n & 8) ? -v : v;
}
/* round-to-nearest, ties to the code with an even mantissa bit, saturating at 6; NaN -> +6 (0x7) */
uint8_t blzo_f32_to_e2m1(float f) {
    uint32_t u = f2u(f), a = u & 0x7fffffffu;
    uint8_t s = (uint8_t)((u >> 28) & 8);
    if (a > 0x7f800000u) return 0x7;
    float x = u2f(a);
    uint8_t c;
    if (x <= 0.25f) c = 0;              /* tie 0.25 -> 0 (even) */
    else if (x < 0.75f) c = 1;
    else if (x <= 1.25f) c = 2;         /* ties 0.75 -> 1.0, 1.25 -> 1.0 */
    else if (x < 1.75f) c = 3;
    else if (x <= 2.5f) c = 4;          /* ties 1.75 -> 2, 2.5 -> 2 */
    else if (x < 3.5f) c = 5;
    else if (x <= 5.0f) c = 6;          /* ties 3.5 -> 4, 5 -> 4 */
    else c = 7;
    return (uint8_t)(s | c);
}

/* vector forms for numpy callers */
void blzo_f16_to_f32_n(const uint16_t* in, float* out, long n) { for (long i = 0; i < n; i++) out[i] = blzo_f16_to_f32(in[i]); }
void blzo_f32_to_f16_n(const float* in, uint16_t* out, long n, int sat) { for (long i = 0; i < n; i++) out[i] = blzo_f32_to_f16_ex(in[i], sat); }
void blzo_bf16_to_f32_n(const uint16_t* in, float* out, long n) { for (long i = 0; i < n; i++) out[i] = blzo_bf16_to_f32(in[i]); }
void blzo_f32_to_bf16_n(const float* in, uint16_t* out, long n) { for (long i = 0; i < n; i++) out[i] = blzo_f32_to_bf16(in[i]); }
void blzo_e4m3_to_f32_n(const uint8_t* in, float* out, long n) { for (long i = 0; i < n; i++) out[i] = blzo_e4m3_to_f32(in[i]); }
void blzo_f32_to_e4m3_n(const float* in, uint8_t* out, long n) { for (long i = 0; i < n; i++) out[i] = blzo_f32_to_e4m3(in[i]); }
void blzo_e2m1_to_f32_n(const uint8_t* in, float* out, long n) { for (long i = 0; i < n; i++) out[i] = blzo_e2m1_to_f32(in[i]); }
void blzo_f32_to_e2m1_n(const float* in, uint8_t* out, long n) { for (long i = 0; i < n; i++) out[i] = blzo_f32_to_e2m1(in[i]); }

/* ------------------------------------------------------------- seeded fill */

/* tests/test_gemm_naive.cu:50-56 -- glibc rand() stream, value in [-1, 1] */
void blzo_fill_uniform_rand(float* out, long n, unsigned seed) {
    srand(seed);
    for (long i = 0; i < n; i++) out[i] = ((float)rand() / (float)RAND_MAX - 0.5f) * 2.0f;
}

/* ------------------------------------------------------------- quantisers */

float blzo_amax(const float* x, long n) {
    float m = 0.0f;
    for (long i = 0; i < n; i++) { float a = fabsf(x[i]); if (a > m) m = a; }
    return m;
}

/* FP8 per-tensor: returns the scale s = 448/amax (1 when amax is 0); q = e4m3_rn(x*s) */
float blzo_quantize_fp8(const float* x, uint8_t* q, long n) {
    float amax = blzo_amax(x, n);
    float s = amax > 0.0f ? 448.0f / amax : 1.0f;
    for (long i = 0; i < n; i++) q[i] = blzo_f32_to_e4m3(x[i] * s);
    return s;
}

/* NVFP4 two-level quantiser of a [rows, K] row-major matrix, K a multiple of 16.
 * data: [rows, K/2] packed; sf: [rows, K/16] E4M3, row-major.  Returns the global scale g.
 * If g_in > 0 it is used instead of amax/(6*448). */
float blzo_quantize_nvfp4(const float* x, long rows, long K, uint8_t* data, uint8_t* sf, float g_in) {
    float g = g_in;
    if (!(g > 0.0f)) {
        float amax = blzo_amax(x, rows * K);
        g = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
    }
    long kb = K / 16;
    for (long r = 0; r < rows; r++) {
        for (long b = 0; b < kb; b++) {
            const float* p = x + r * K + b * 16;
            float am = 0.0f;
            for (int i = 0; i < 16; i++) { float a = fabsf(p[i]); if (a > am) am = a; }
            uint8_t s8 = blzo_f32_to_e4m3((am / 6.0f) / g);
            float sfv = blzo_e4m3_to_f32(s8);
            sf[r * kb + b] = s8;
            float d = g * sfv;
            for (int i = 0; i < 16; i += 2) {
                uint8_t lo = 0, hi = 0;
                if (sfv != 0.0f) { lo = blzo_f32_to_e2m1(p[i] / d); hi = blzo_f32_to_e2m1(p[i + 1] / d); }
                data[r * (K / 2) + b * 8 + i / 2] = (uint8_t)(lo | (hi << 4));
            }
        }
    }
    return g;
}

/* x^ without the global scale: out[r,k] = e2m1(q)*e4m3(sf)  (exact in fp32) */
void blzo_dequant_nvfp4_noglobal(const uint8_t* data, const uint8_t* sf, long rows, long K, float* out) {
    long kb = K / 16;
    for (long r = 0; r < rows; r++)
        for (long k = 0; k < K; k++) {
            uint8_t byte = data[r * (K / 2) + k / 2];
            uint8_t nib = (k & 1) ? (byte >> 4) : (byte & 15);
            out[r * K + k] = blzo_e2m1_to_f32(nib) * blzo_e4m3_to_f32(sf[r * kb + k / 16]);
        }
}

/* SF tiling used by the tensor-core path: [ceil(rows/128)][katoms][512] with
 * byte offset (r%32)*16 + ((r%128)/32)*4 + (kb%4) inside a 512-byte atom; katoms = padded K/64.
 * Unused entries are zero. */
void blzo_tile_sf(const uint8_t* sf, long rows, long kb, uint8_t* out, long row_blocks, long katoms) {
    memset(out, 0, (size_t)(row_blocks * katoms * 512));
    for (long r = 0; r < rows; r++)
        for (long b = 0; b < kb; b++) {
            long off = ((r / 128) * katoms + b / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4);
            out[off] = sf[r * kb + b];
        }
}

/* ------------------------------------------------------------------- GEMM */

typedef struct {
    const float* A;   /* [M, K] row-major */
    const float* Bt;  /* [N, K] row-major (B stored K-major) */
    float* C;         /* [M, N] */
    long M, N, K, r0, r1;
} gemm_job;

/* tests/test_gemm_naive.cu:38-48: for i, for j, sum=0, for kk ascending sum += a*b */
static void* gemm_rows(void* arg) {
    gemm_job* j = (gemm_job*)arg;
    for (long i = j->r0; i < j->r1; i++) {
        const float* a = j->A + i * j->K;
        for (long n = 0; n < j->N; n++) {
            const float* b = j->Bt + n * j->K;
            float sum = 0.0f;
            for (long kk = 0; kk < j->K; kk++) sum += a[kk] * b[kk];
            j->C[i * j->N + n] = sum;
        }
    }
    return 0;
}

/* C = A * Bt^T in fp32, rows split over nthreads host threads (each row's sum order unchanged) */
void blzo_gemm_f32(const float* A, const float* Bt, float* C, long M, long N, long K, int nthreads) {
    if (nthreads < 1) nthreads = 1;
    if (nthreads > M) nthreads = (int)(M > 0 ? M : 1);
    if (nthreads > 256) nthreads = 256;
    pthread_t th[256];
    gemm_job jobs[256];
    long per = (M + nthreads - 1) / nthreads;
    int started = 0;
    for (int t = 0; t < nthreads; t++) {
        long r0 = t * per, r1 = r0 + per > M ? M : r0 + per;
        if (r0 >= r1) break;
        jobs[t] = (gemm_job){A, Bt, C, M, N, K, r0, r1};
        if (t == nthreads - 1 || r1 == M) { gemm_rows(&jobs[t]); break; }
        pthread_create(&th[t], 0, gemm_rows, &jobs[t]);
        started++;
    }
    for (int t = 0; t < started; t++) pthread_join(th[t], 0);
}

/* Same loop with B given [K, N] row-major exactly as Blaze's gemm_cpu_fp16 takes it. */
void blzo_gemm_f32_bkn(const float* A, const float* B, float* C, long M, long N, long K) {
    for (long i = 0; i < M; i++)
        for (long j = 0; j < N; j++) {
            float sum = 0.0f;
            for (long kk = 0; kk < K; kk++) sum += A[i * K + kk] * B[kk * N + j];
            C[i * N + j] = sum;
        }
}

/* Epilogue: v = acc*alpha; + bias[n]; SiLU; + residual[m,n].  mode: 0 none, 1 bias, 2 silu,
 * 3 bias+silu, 4 residual add.  In place on C (fp32); narrowing is done by the caller. */
void blzo_epilogue(float* C, long M, long N, float alpha, const float* bias, const float* residual, int mode) {
    for (long i = 0; i < M; i++)
        for (long n = 0; n < N; n++) {
            float v = C[i * N + n] * alpha;
            if ((mode == 1 || mode == 3) && bias) v += bias[n];
            if (mode == 2 || mode == 3) v = v / (1.0f + expf(-v));
            if (mode == 4 && residual) v += residual[i * N + n];
            C[i * N + n] = v;
        }
}

int blzo_version(void) { return 1; }
