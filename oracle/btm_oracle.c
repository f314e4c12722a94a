/*
 * btm_oracle.c — CPU restatement of the matmul path. TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker that the CUDA kernels are compared with. It is not part of
 * the shipped library and nothing in the product path links or calls it; only the test
 * suite, the smoke check and the CPU-baseline leg of the benchmark may load it.
 *
 * PARITY UNPINNED: the reference project ships no matmul, batched matmul or int4 code
 * (Ops/Algebra/MatMul/MatMul.h:1-8 is an empty include guard; cpu_MatMul.h,
 * gpu_MatMul.h and npu_MatMul.h are zero bytes) and no test, golden vector or fixture
 * for such a path (tests/tensor_tests.cpp:18-30 checks a zero fill only). What the
 * reference does define, and what this file follows, is:
 *   - dtype ordinals and element sizes        Tensor/Dtypes.h:57-92
 *   - row-major contiguous strides            Tensor/Tensor.cpp:157-162
 *   - round-to-nearest-even output narrowing  Tensor/TensorOps.cu:72 (__floats2bfloat162_rn)
 *   - the seeded input generator              Tensor/Tensor.cpp:89-152 (restated in
 *     btmo_ref_random_f32/f64 below and checked against the compiled reference, see
 *     oracle/Makefile target _ref)
 * The matmul arithmetic itself is the textbook definition with fp64 accumulation.
 *
 * Plain C11, no dependencies beyond libm and pthreads.
 */
#define _POSIX_C_SOURCE 200809L
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* dtype ordinals: Tensor/Dtypes.h:57-70 (BFloat16=0, Float16=1, Float32=2, Float64=3). */
enum { BTMO_BF16 = 0, BTMO_F16 = 1, BTMO_F32 = 2, BTMO_F64 = 3 };

/* ------------------------------------------------------------------------------------
 * Narrowing and widening. IEEE 754 round-to-nearest-even from binary64, one rounding
 * step (no intermediate binary32), overflow to infinity, gradual underflow.
 * ---------------------------------------------------------------------------------- */

float btmo_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: value = man * 2^-24 */
            float f = (float)man * 5.9604644775390625e-8f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

float btmo_bf16_to_f32(uint16_t b)
{
    uint32_t bits = (uint32_t)b << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* Round a finite double to `mant_bits` explicit mantissa bits with minimum normal
 * exponent `emin` (unbiased), RNE; returns the rounded value as a double which is then
 * exactly representable in the target format (or +-inf on overflow past `max_finite`). */
static double round_to_format(double x, int mant_bits, int emin, double max_finite)
{
    if (x == 0.0 || isnan(x) || isinf(x)) return x;
    int e;
    double m = frexp(fabs(x), &e); /* |x| = m * 2^e, m in [0.5,1) */
    int ue = e - 1;                /* unbiased exponent of the leading bit */
    if (ue < emin) ue = emin;      /* subnormal range: fixed quantum */
    double quantum = ldexp(1.0, ue - mant_bits);
    double q = fabs(x) / quantum;  /* exact: power-of-two scaling */
    double r = nearbyint(q);       /* default rounding mode is RNE */
    double y = r * quantum;
    (void)m;
    if (y > max_finite) y = INFINITY;
    return copysign(y, x);
}

uint16_t btmo_f64_to_f16_rne(double x)
{
    if (isnan(x)) return 0x7E00u;
    double y = round_to_format(x, 10, -14, 65504.0);
    uint16_t sign = signbit(y) ? 0x8000u : 0;
    double a = fabs(y);
    if (a == 0.0) return sign;
    if (isinf(a)) return (uint16_t)(sign | 0x7C00u);
    int e;
    double m = frexp(a, &e);
    int ue = e - 1;
    if (ue < -14) { /* subnormal: a = man * 2^-24 */
        return (uint16_t)(sign | (uint16_t)(a * 16777216.0));
    }
    uint32_t man = (uint32_t)((m * 2.0 - 1.0) * 1024.0);
    return (uint16_t)(sign | (uint16_t)((ue + 15) << 10) | (uint16_t)man);
}

uint16_t btmo_f64_to_bf16_rne(double x)
{
    if (isnan(x)) return 0x7FC0u;
    double y = round_to_format(x, 7, -126, 3.3895313892515355e38);
    float f = (float)y; /* exact: y has 8 significant bits and is in binary32 range */
    uint32_t bits;
    memcpy(&bits, &f, 4);
    return (uint16_t)(bits >> 16);
}

float btmo_f64_to_f32_rne(double x) { return (float)x; }

static double load_elem(const void *p, int dtype, size_t i)
{
    switch (dtype) {
    case BTMO_BF16: return (double)btmo_bf16_to_f32(((const uint16_t *)p)[i]);
    case BTMO_F16: return (double)btmo_f16_to_f32(((const uint16_t *)p)[i]);
    case BTMO_F32: return (double)((const float *)p)[i];
    default: return ((const double *)p)[i];
    }
}

/* Widen n elements of `dtype` storage to binary64. */
void btmo_widen(const void *src, int dtype, size_t n, double *dst)
{
    for (size_t i = 0; i < n; ++i) dst[i] = load_elem(src, dtype, i);
}

/* Narrow n binary64 values to `dtype` storage with RNE. */
void btmo_narrow(const double *src, int dtype, size_t n, void *dst)
{
    for (size_t i = 0; i < n; ++i) {
        switch (dtype) {
        case BTMO_BF16: ((uint16_t *)dst)[i] = btmo_f64_to_bf16_rne(src[i]); break;
        case BTMO_F16: ((uint16_t *)dst)[i] = btmo_f64_to_f16_rne(src[i]); break;
        case BTMO_F32: ((float *)dst)[i] = (float)src[i]; break;
        default: ((double *)dst)[i] = src[i]; break;
        }
    }
}

/* ------------------------------------------------------------------------------------
 * Dense matmul C[M,N] = A[M,K] . B[K,N], row-major with leading dimensions in elements
 * (Tensor/Tensor.cpp:157-162), accumulated in binary64, result left in binary64.
 * Rows are split over threads the way the reference splits its CPU loops
 * (Tensor/Tensor.cpp:141-151: ceil(n/threads) contiguous chunks).
 * ---------------------------------------------------------------------------------- */

typedef struct {
    int dtype;
    int64_t M, N, K, lda, ldb, ldc;
    const void *A, *B;
    double *C;
    int64_t row0, row1;
} gemm_job;

static void *gemm_worker(void *arg)
{
    gemm_job *j = (gemm_job *)arg;
    double *brow = (double *)malloc(sizeof(double) * (size_t)j->N);
    for (int64_t i = j->row0; i < j->row1; ++i) {
        double *c = j->C + i * j->ldc;
        for (int64_t n = 0; n < j->N; ++n) c[n] = 0.0;
    }
    /* k outermost inside a row block so that each B row is widened once per block. */
    for (int64_t k = 0; k < j->K; ++k) {
        for (int64_t n = 0; n < j->N; ++n) brow[n] = load_elem(j->B, j->dtype, (size_t)(k * j->ldb + n));
        for (int64_t i = j->row0; i < j->row1; ++i) {
            double a = load_elem(j->A, j->dtype, (size_t)(i * j->lda + k));
            double *c = j->C + i * j->ldc;
            for (int64_t n = 0; n < j->N; ++n) c[n] += a * brow[n];
        }
    }
    free(brow);
    return NULL;
}

static int clamp_threads(int threads, int64_t rows)
{
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    if ((int64_t)threads > rows) threads = rows > 0 ? (int)rows : 1;
    return threads;
}

int btmo_gemm(int dtype, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda, const void *B,
              int64_t ldb, double *C, int64_t ldc, int threads)
{
    if (M < 0 || N < 0 || K < 0) return 1;
    if (M == 0 || N == 0) return 0;
    threads = clamp_threads(threads, M);
    gemm_job jobs[256];
    pthread_t tids[256];
    int64_t chunk = (M + threads - 1) / threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        int64_t r0 = t * chunk, r1 = r0 + chunk < M ? r0 + chunk : M;
        if (r0 >= M) break;
        jobs[t] = (gemm_job){dtype, M, N, K, lda, ldb, ldc, A, B, C, r0, r1};
        pthread_create(&tids[t], NULL, gemm_worker, &jobs[t]);
        ++started;
    }
    for (int t = 0; t < started; ++t) pthread_join(tids[t], NULL);
    return 0;
}

/* Batched matmul: `batch` independent products with element strides between them. */
int btmo_bmm(int dtype, int64_t batch, int64_t M, int64_t N, int64_t K, const void *A, int64_t strideA,
             const void *B, int64_t strideB, double *C, int64_t strideC, int threads)
{
    size_t es = (dtype == BTMO_F32) ? 4 : (dtype == BTMO_F64 ? 8 : 2);
    for (int64_t b = 0; b < batch; ++b) {
        int rc = btmo_gemm(dtype, M, N, K, (const char *)A + (size_t)(b * strideA) * es, K,
                           (const char *)B + (size_t)(b * strideB) * es, N, C + b * strideC, N, threads);
        if (rc) return rc;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------
 * int4 weight-only format (the reference has no sub-byte dtype, Tensor/Dtypes.h:57-70;
 * the convention is this build's own and is appended as ordinal 12):
 *   W[n,k] is a signed two's-complement nibble in [-8,7];
 *   byte n*(K/2) + k/2 holds k even in bits 0-3 and k odd in bits 4-7;
 *   scales S[n, k/group] are binary16, row-major [N, K/group];
 *   dequant(n,k) = f16_rne(float(W[n,k]) * float(S[n,k/group])).
 * ---------------------------------------------------------------------------------- */

static inline int nib_lo(uint8_t b) { return (int)((b & 0xF) ^ 8) - 8; }
static inline int nib_hi(uint8_t b) { return (int)((b >> 4) ^ 8) - 8; }

void btmo_int4_pack(const int8_t *w, int64_t N, int64_t K, uint8_t *packed)
{
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; k += 2) {
            uint8_t lo = (uint8_t)(w[n * K + k] & 0xF);
            uint8_t hi = (uint8_t)(w[n * K + k + 1] & 0xF);
            packed[n * (K / 2) + k / 2] = (uint8_t)(lo | (hi << 4));
        }
}

void btmo_int4_unpack(const uint8_t *packed, int64_t N, int64_t K, int8_t *w)
{
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; k += 2) {
            uint8_t b = packed[n * (K / 2) + k / 2];
            w[n * K + k] = (int8_t)nib_lo(b);
            w[n * K + k + 1] = (int8_t)nib_hi(b);
        }
}

void btmo_int4_dequant(const uint8_t *packed, const uint16_t *scales, int64_t N, int64_t K, int64_t group,
                       uint16_t *out_f16)
{
    int64_t G = K / group;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) {
            uint8_t b = packed[n * (K / 2) + k / 2];
            int w = (k & 1) ? nib_hi(b) : nib_lo(b);
            double s = (double)btmo_f16_to_f32(scales[n * G + k / group]);
            /* |w| <= 8 and s has 11 significant bits: the product is exact in binary32
             * and binary64, so one RNE step to binary16 defines the result. */
            out_f16[n * K + k] = btmo_f64_to_f16_rne((double)w * s);
        }
}

typedef struct {
    int64_t M, N, K, group;
    const uint16_t *act, *scales;
    const uint8_t *packed;
    double *out;
    int64_t n0, n1;
} int4_job;

static void *int4_worker(void *arg)
{
    int4_job *j = (int4_job *)arg;
    int64_t G = j->K / j->group;
    double *a = (double *)malloc(sizeof(double) * (size_t)j->K);
    for (int64_t m = 0; m < j->M; ++m) {
        for (int64_t k = 0; k < j->K; ++k) a[k] = (double)btmo_f16_to_f32(j->act[m * j->K + k]);
        for (int64_t n = j->n0; n < j->n1; ++n) {
            double acc = 0.0;
            for (int64_t g = 0; g < G; ++g) {
                double part = 0.0;
                for (int64_t k = g * j->group; k < (g + 1) * j->group; ++k) {
                    uint8_t b = j->packed[n * (j->K / 2) + k / 2];
                    int w = (k & 1) ? nib_hi(b) : nib_lo(b);
                    part += a[k] * (double)w;
                }
                acc += (double)btmo_f16_to_f32(j->scales[n * G + g]) * part;
            }
            j->out[m * j->N + n] = acc;
        }
    }
    free(a);
    return NULL;
}

/* out[m,n] = sum_g float(S[n,g]) * sum_{k in g} float(act[m,k]) * W[n,k], in binary64. */
int btmo_int4_matmul(int64_t M, int64_t N, int64_t K, int64_t group, const uint16_t *act_f16,
                     const uint8_t *packed, const uint16_t *scales_f16, double *out, int threads)
{
    if (group <= 0 || K % group || K % 2) return 1;
    threads = clamp_threads(threads, N);
    int4_job jobs[256];
    pthread_t tids[256];
    int64_t chunk = (N + threads - 1) / threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        int64_t n0 = t * chunk, n1 = n0 + chunk < N ? n0 + chunk : N;
        if (n0 >= N) break;
        jobs[t] = (int4_job){M, N, K, group, act_f16, scales_f16, packed, out, n0, n1};
        pthread_create(&tids[t], NULL, int4_worker, &jobs[t]);
        ++started;
    }
    for (int t = 0; t < started; ++t) pthread_join(tids[t], NULL);
    return 0;
}

/* Relative Frobenius error ||X - R||_F / ||R||_F where X is in `dtype` storage. */
double btmo_rel_frobenius(const void *X, int dtype, const double *R, size_t n)
{
    double num = 0.0, den = 0.0;
    for (size_t i = 0; i < n; ++i) {
        double d = load_elem(X, dtype, i) - R[i];
        num += d * d;
        den += R[i] * R[i];
    }
    if (den == 0.0) return num == 0.0 ? 0.0 : INFINITY;
    return sqrt(num / den);
}

/* ------------------------------------------------------------------------------------
 * The reference's seeded input generator, restated: Tensor/Tensor.cpp:89-152.
 * numel <= threads*1024 -> one mt19937(seed) stream; otherwise `threads` contiguous
 * chunks of ceil(numel/threads) elements, chunk t drawn from mt19937(seed + t). Each
 * element is std::uniform_real_distribution<double>(min,max) cast to the element type.
 * `threads` is the reference's uint8_t hardware thread count (Helper/Hardware.h:14,41-44).
 * The distribution follows libstdc++'s generate_canonical<double,53> over a 32-bit
 * engine: two draws, (x0 + x1*2^32) / 2^64, clamped below 1.
 * ---------------------------------------------------------------------------------- */

typedef struct {
    uint32_t mt[624];
    int idx;
} mt19937_t;

static void mt_seed(mt19937_t *s, uint32_t seed)
{
    s->mt[0] = seed;
    for (int i = 1; i < 624; ++i) s->mt[i] = 1812433253u * (s->mt[i - 1] ^ (s->mt[i - 1] >> 30)) + (uint32_t)i;
    s->idx = 624;
}

static uint32_t mt_next(mt19937_t *s)
{
    if (s->idx >= 624) {
        for (int i = 0; i < 624; ++i) {
            uint32_t y = (s->mt[i] & 0x80000000u) | (s->mt[(i + 1) % 624] & 0x7FFFFFFFu);
            uint32_t v = s->mt[(i + 397) % 624] ^ (y >> 1);
            if (y & 1u) v ^= 0x9908B0DFu;
            s->mt[i] = v;
        }
        s->idx = 0;
    }
    uint32_t y = s->mt[s->idx++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9D2C5680u;
    y ^= (y << 15) & 0xEFC60000u;
    y ^= y >> 18;
    return y;
}

static double mt_uniform(mt19937_t *s, double lo, double hi)
{
    double sum = (double)mt_next(s);
    sum += (double)mt_next(s) * 4294967296.0;
    double r = sum / 18446744073709551616.0;
    if (r >= 1.0) r = nextafter(1.0, 0.0);
    return r * (hi - lo) + lo;
}

static void ref_random(void *out, int is_f64, size_t numel, uint64_t seed, double lo, double hi, int threads)
{
    if (threads < 1) threads = 1;
    mt19937_t st;
    size_t chunk = numel, nchunks = 1;
    if (numel > (size_t)threads * 1024) {
        chunk = (numel + (size_t)threads - 1) / (size_t)threads;
        nchunks = (size_t)threads;
    }
    for (size_t t = 0; t < nchunks; ++t) {
        size_t a = t * chunk, b = a + chunk < numel ? a + chunk : numel;
        if (a >= numel) break;
        mt_seed(&st, (uint32_t)(seed + t));
        for (size_t i = a; i < b; ++i) {
            double v = mt_uniform(&st, lo, hi);
            if (is_f64) ((double *)out)[i] = v;
            else ((float *)out)[i] = (float)v;
        }
    }
}

void btmo_ref_random_f32(float *out, size_t numel, uint64_t seed, double lo, double hi, int threads)
{
    ref_random(out, 0, numel, seed, lo, hi, threads);
}

void btmo_ref_random_f64(double *out, size_t numel, uint64_t seed, double lo, double hi, int threads)
{
    ref_random(out, 1, numel, seed, lo, hi, threads);
}

/* ------------------------------------------------------------------------------------
 * Timed CPU baseline ("port"): binary32 matmul over host threads. The reference has no
 * CPU matmul to time (its AVX-512 code converts dtypes only,
 * Intrinsics/AVX512/DTypeConversions.cpp:10-174), so this stands in for it, written the
 * way a tuned CPU GEMM is: B is packed per k-block into panels of 32 columns, a
 * register-blocked 12 x 32 micro-kernel (24 accumulator vectors, AVX-512 FMA) runs over
 * it, and rows are split over threads as the reference splits CPU work
 * (Tensor/Tensor.cpp:141-151). Hosts without AVX-512, and the ragged edges, take the plain
 * loop. Inputs are widened to binary32 by the caller outside the timed region.
 * ---------------------------------------------------------------------------------- */

#define FAST_MR 12
#define FAST_NR 32
#define FAST_KC 384

typedef struct {
    int64_t M, N, K;
    const float *A, *B;
    float *C;
    float *Bp;            /* packed k-block of B: [N / 32 panels][kc][32] */
    int tid, threads;
    int64_t row0, row1;
    int use_avx512;
    pthread_barrier_t *bar;
} fast_job;

#if defined(__x86_64__) && defined(__GNUC__)
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
#endif
static void fast_block(const float *A, const float *B, float *C, int64_t N, int64_t K, int64_t i0, int64_t i1,
                       int64_t k0, int64_t k1, int64_t n0, int64_t n1)
{
    for (int64_t i = i0; i < i1; ++i) {
        float *c = C + i * N;
        for (int64_t k = k0; k < k1; ++k) {
            float a = A[i * K + k];
            const float *b = B + k * N;
            for (int64_t n = n0; n < n1; ++n) c[n] += a * b[n];
        }
    }
}

#if defined(__x86_64__) && defined(__GNUC__)
#include <immintrin.h>
/* C[12 x 32] += Ap[kc x 12] . Bp[kc x 32]; both operands packed (Ap: 12 row values per k, Bp: 32 columns per k). */
__attribute__((target("avx512f")))
static void fast_micro_12x32(const float *Ap, const float *Bp, float *C, int64_t ldc, int64_t kc)
{
    __m512 c0[FAST_MR], c1[FAST_MR];
#pragma GCC unroll 12
    for (int i = 0; i < FAST_MR; ++i) {
        c0[i] = _mm512_loadu_ps(C + i * ldc);
        c1[i] = _mm512_loadu_ps(C + i * ldc + 16);
    }
    for (int64_t k = 0; k < kc; ++k) {
        const __m512 b0 = _mm512_loadu_ps(Bp + k * FAST_NR), b1 = _mm512_loadu_ps(Bp + k * FAST_NR + 16);
#pragma GCC unroll 12
        for (int i = 0; i < FAST_MR; ++i) {
            const __m512 a = _mm512_set1_ps(Ap[k * FAST_MR + i]);
            c0[i] = _mm512_fmadd_ps(a, b0, c0[i]);
            c1[i] = _mm512_fmadd_ps(a, b1, c1[i]);
        }
    }
#pragma GCC unroll 12
    for (int i = 0; i < FAST_MR; ++i) {
        _mm512_storeu_ps(C + i * ldc, c0[i]);
        _mm512_storeu_ps(C + i * ldc + 16, c1[i]);
    }
}
static int host_has_avx512(void) { return __builtin_cpu_supports("avx512f"); }
#else
static void fast_micro_12x32(const float *Ap, const float *Bp, float *C, int64_t ldc, int64_t kc)
{
    (void)Ap; (void)Bp; (void)C; (void)ldc; (void)kc;
}
static int host_has_avx512(void) { return 0; }
#endif

static void *fast_worker(void *arg)
{
    fast_job *j = (fast_job *)arg;
    const int64_t N = j->N, K = j->K;
    const int64_t panels = N / FAST_NR;            /* full 32-column panels; the rest takes the plain loop */
    for (int64_t i = j->row0; i < j->row1; ++i) memset(j->C + i * N, 0, sizeof(float) * (size_t)N);
    if (!j->use_avx512) {
        const int64_t BK = 256, BN = 1024;
        for (int64_t n0 = 0; n0 < N; n0 += BN)
            for (int64_t k0 = 0; k0 < K; k0 += BK)
                fast_block(j->A, j->B, j->C, N, K, j->row0, j->row1, k0, k0 + BK < K ? k0 + BK : K, n0, n0 + BN < N ? n0 + BN : N);
        return NULL;
    }
    const int64_t rows_main = j->row0 + (j->row1 - j->row0) / FAST_MR * FAST_MR;
    /* this thread's rows of A, packed per k-block: [row block of 12][k][12] */
    float *Ap = NULL;
    if (rows_main > j->row0 && posix_memalign((void **)&Ap, 64, sizeof(float) * (size_t)(rows_main - j->row0) * FAST_KC)) Ap = NULL;
    for (int64_t k0 = 0; k0 < K; k0 += FAST_KC) {
        const int64_t kc = k0 + FAST_KC < K ? FAST_KC : K - k0;
        if (Ap)
            for (int64_t i = j->row0; i < rows_main; i += FAST_MR) {
                float *dst = Ap + (i - j->row0) * FAST_KC;
                for (int r = 0; r < FAST_MR; ++r) {
                    const float *src = j->A + (i + r) * K + k0;
                    for (int64_t k = 0; k < kc; ++k) dst[k * FAST_MR + r] = src[k];
                }
            }
        /* every thread packs its share of the panels of this k-block */
        for (int64_t p = j->tid; p < panels; p += j->threads) {
            float *dst = j->Bp + p * FAST_KC * FAST_NR;
            const float *src = j->B + k0 * N + p * FAST_NR;
            for (int64_t k = 0; k < kc; ++k) memcpy(dst + k * FAST_NR, src + k * N, sizeof(float) * FAST_NR);
        }
        pthread_barrier_wait(j->bar);
        for (int64_t p = 0; p < panels; ++p) {
            const float *bp = j->Bp + p * FAST_KC * FAST_NR;
            if (Ap)
                for (int64_t i = j->row0; i < rows_main; i += FAST_MR)
                    fast_micro_12x32(Ap + (i - j->row0) * FAST_KC, bp, j->C + i * N + p * FAST_NR, N, kc);
        }
        if (!Ap && rows_main > j->row0) fast_block(j->A, j->B, j->C, N, K, j->row0, rows_main, k0, k0 + kc, 0, panels * FAST_NR);
        if (rows_main < j->row1) fast_block(j->A, j->B, j->C, N, K, rows_main, j->row1, k0, k0 + kc, 0, panels * FAST_NR);
        if (panels * FAST_NR < N) fast_block(j->A, j->B, j->C, N, K, j->row0, j->row1, k0, k0 + kc, panels * FAST_NR, N);
        pthread_barrier_wait(j->bar); /* the packed block is rewritten next round */
    }
    free(Ap);
    return NULL;
}

int btmo_gemm_f32_threads(int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C, int threads)
{
    if (M <= 0 || N <= 0) return 0;
    threads = clamp_threads(threads, (M + FAST_MR - 1) / FAST_MR);
    /* rows per thread: a multiple of the micro-kernel's 12 where possible */
    int64_t chunk = (M + threads - 1) / threads;
    chunk = (chunk + FAST_MR - 1) / FAST_MR * FAST_MR;
    int used = (int)((M + chunk - 1) / chunk);
    fast_job jobs[256];
    pthread_t tids[256];
    pthread_barrier_t bar;
    const int avx = host_has_avx512();
    float *Bp = NULL;
    if (avx) {
        if (posix_memalign((void **)&Bp, 64, sizeof(float) * (size_t)FAST_KC * (size_t)(N / FAST_NR + 1) * FAST_NR)) return 1;
    }
    pthread_barrier_init(&bar, NULL, (unsigned)used);
    for (int t = 0; t < used; ++t) {
        int64_t r0 = t * chunk, r1 = r0 + chunk < M ? r0 + chunk : M;
        jobs[t] = (fast_job){M, N, K, A, B, C, Bp, t, used, r0, r1, avx, &bar};
        pthread_create(&tids[t], NULL, fast_worker, &jobs[t]);
    }
    for (int t = 0; t < used; ++t) pthread_join(tids[t], NULL);
    pthread_barrier_destroy(&bar);
    free(Bp);
    return 0;
}

/* ------------------------------------------------------------------------------------
 * int4 group quantiser (the producer of the packed format; this build's own convention,
 * the reference has no quantised type): per row n and group g,
 *   S[n,g] = f16_rne(max|w| / 7) in binary32 arithmetic, 1 when the group is all zero;
 *   W[n,k] = clamp(rint(float(w) / float(S)), -8, 7), rint = round half to even.
 * ---------------------------------------------------------------------------------- */
void btmo_int4_quantize(const uint16_t *w_f16, int64_t N, int64_t K, int64_t group, uint8_t *packed, uint16_t *scales_f16)
{
    int64_t G = K / group;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t g = 0; g < G; ++g) {
            const uint16_t *src = w_f16 + n * K + g * group;
            float amax = 0.0f;
            for (int64_t k = 0; k < group; ++k) {
                float v = fabsf(btmo_f16_to_f32(src[k]));
                if (v > amax) amax = v;
            }
            uint16_t sh = btmo_f64_to_f16_rne((double)(amax / 7.0f));
            if (btmo_f16_to_f32(sh) == 0.0f) sh = 0x3C00u;
            float s = btmo_f16_to_f32(sh);
            scales_f16[n * G + g] = sh;
            for (int64_t k = 0; k < group; k += 2) {
                float q0 = rintf(btmo_f16_to_f32(src[k]) / s), q1 = rintf(btmo_f16_to_f32(src[k + 1]) / s);
                if (q0 < -8.0f) q0 = -8.0f;
                if (q0 > 7.0f) q0 = 7.0f;
                if (q1 < -8.0f) q1 = -8.0f;
                if (q1 > 7.0f) q1 = 7.0f;
                packed[n * (K / 2) + (g * group + k) / 2] = (uint8_t)(((int)q0 & 0xF) | (((int)q1 & 0xF) << 4));
            }
        }
}
