/*
 * CPU oracle for the MXFP / minifloat fake-quantisation path of mase-triton.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a scalar C restatement of the
 * reference's pure-PyTorch "fake" path.  It is the checker the CUDA kernels are
 * compared against and the CPU baseline that the benchmark times; the product
 * never calls it.  Only tests, the smoke check and the benchmark's CPU legs may
 * load the shared object built from it.
 *
 * Parity pin: validated bit-for-bit against the reference's own fake path
 * (src/mase_triton/minifloat/fake.py, src/mase_triton/mxfp/fake.py) by
 * oracle/validate_against_reference.py, and against the golden vectors under
 * tests/golden/ that were generated from the reference.
 *
 * All arithmetic is IEEE binary32 with subnormals (build WITHOUT -ffast-math
 * and without flush-to-zero).  NaN sign/payload results follow x86 SSE, which
 * is what the reference produces on the hosts it runs on.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { RM_RN = 0, RM_RU = 1, RM_RD = 2, RM_RZ = 3 };

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ------------------------------------------------------------------------- */
/* minifloat extract: one fp32 value -> uint16 code                           */
/* follows src/mase_triton/minifloat/fake.py:7-78                             */
/* ------------------------------------------------------------------------- */
static inline uint16_t encode_one(float x, int eb, int fb, int is_finite, int rm)
{
    const uint32_t u = f2u(x);
    const uint32_t a = u & 0x7FFFFFFFu;
    const int E = (int)(a >> 23);
    uint32_t M = a & 0x7FFFFFu;
    const int is_nan = (a > 0x7F800000u);
    const int is_inf = (a == 0x7F800000u);

    const int bias = (1 << (eb - 1)) - 1;                        /* fake.py:13 */
    const int emax = is_finite ? (1 << eb) - 1 : (1 << eb) - 2;  /* fake.py:15 */
    const int fmax = (1 << fb) - 1;                              /* fake.py:19 */

    /* fake.py:22  y_sign = x < 0  (false for -0.0 and for every NaN) */
    const int neg = (x < 0.0f);
    /* fake.py:24  flush when the fp32 exponent field is zero */
    const int flush = (E == 0);

    /* fake.py:27-29  frexp of |x|, rescaled to mantissa in [1,2).  glibc frexp
     * reports exponent 0 for Inf/NaN, and nan*2 quiets a signalling payload. */
    int xe;
    if (E == 255) { xe = -1; if (is_nan) M |= 0x400000u; }
    else          { xe = E - 127; }

    const int under = xe < -bias;          /* fake.py:35 */
    const int over  = xe > emax - bias;    /* fake.py:36 */
    int ye = xe + bias;                    /* fake.py:37 */

    /* fake.py:39-56  mantissa rounding.  Every mode except rz first drops the
     * low 8 mantissa bits and rounds the remaining 15-bit integer. */
    int f;
    if (rm == RM_RZ) {
        f = (int)(M >> (23 - fb));
    } else {
        const int t = (int)(M >> 8);
        const int d = 15 - fb;
        const int q = t >> d;
        const int r = t & ((1 << d) - 1);
        if (rm == RM_RD)      f = q;
        else if (rm == RM_RU) f = q + (r != 0);
        else {                                  /* half to even, torch.round */
            const int half = 1 << (d - 1);
            f = q + ((r > half) || (r == half && (q & 1)));
        }
    }

    /* fake.py:58-60  only the binade with biased exponent 0 is made subnormal */
    if (ye == 0 && f != 0) f = (f | (1 << fb)) >> 1;
    if (under) { f = 0; ye = 0; }               /* fake.py:62-63 */
    if (over)  { f = fmax; ye = emax; }         /* fake.py:65-66 */
    if (flush) { f = 0; ye = 0; }               /* fake.py:68-69 */
    if (!is_finite) {                           /* fake.py:70-74 */
        if (is_inf) { f = 0; ye = emax; }
        if (is_nan) { f = fmax; ye = emax; }
    }
    /* fake.py:75-77  bitwise OR: a mantissa carry is lost when ye is odd;
     * arithmetic is int32 and the result is truncated to 16 bits */
    uint32_t code = ((uint32_t)ye << fb) | (uint32_t)f;
    if (neg) code += (1u << (eb + fb));
    return (uint16_t)code;
}

/* ------------------------------------------------------------------------- */
/* minifloat compose: uint16 code -> fp32                                     */
/* follows src/mase_triton/minifloat/fake.py:81-125                           */
/* ------------------------------------------------------------------------- */
static inline float exp2_int(int k)
{
    /* torch.exp2 on an int32 tensor promotes to fp32; exact for integer k */
    if (k > 127) return INFINITY;
    if (k >= -126) return u2f((uint32_t)(k + 127) << 23);
    if (k >= -149) return u2f(1u << (k + 149));
    return 0.0f;
}

static inline float decode_one(uint16_t code, int eb, int fb, int is_finite)
{
    const int c_full = (int)code;
    const int sign = (c_full >> (eb + fb)) & 1;          /* fake.py:98 */
    const int c = c_full & 0x7FFF;                       /* fake.py:100 */
    const int e = (c >> fb) & ((1 << eb) - 1);           /* fake.py:101 */
    const int f = c & ((1 << fb) - 1);                   /* fake.py:102 */
    const int bias = (1 << (eb - 1)) - 1;
    const int is_sub = (e == 0) && (f != 0);
    const int is_zero = (e == 0) && (f == 0);

    int k = e - bias;                                    /* fake.py:111-112 */
    if (is_sub) k += 1;
    const float p = exp2_int(k);                         /* fake.py:113 */
    float m = (float)f / (float)(1 << fb);               /* fake.py:114-116 */
    if (!is_sub) m += 1.0f;
    float y = p * m;                                     /* fake.py:117 */
    if (!is_finite && e == (1 << eb) - 1)                /* fake.py:119-121 */
        y = (f == 0) ? INFINITY : u2f(0x7FC00000u);
    if (is_zero) y = 0.0f;                               /* fake.py:122 */
    if (sign) y = u2f(f2u(y) ^ 0x80000000u);             /* fake.py:123 */
    return y;
}

/* ------------------------------------------------------------------------- */
/* floor(log2f(v)) as the reference's host evaluates it (mxfp/fake.py:44-45). */
/* A correctly rounded log2f returns e+1 for the last few fp32 values below   */
/* 2^(e+1); the count of such values depends on the binade the result lies in.*/
/* ------------------------------------------------------------------------- */
int mxq_oracle_log2_roundup_count(int e)
{
    /* number of mantissas, counted down from 0x7FFFFF, for which
     * floor(log2f(2^e * 1.m)) == e + 1 */
    int mag;   /* magnitude of the result just below e+1 lies in [2^m, 2^(m+1)) */
    if (e >= 1) mag = e;          /* result in [e, e+1), e >= 1               */
    else if (e <= -3) mag = -e - 1; /* result in (e, e+1), |result| > |e+1|   */
    else return 0;                /* results of magnitude < 2: ulp too fine    */
    int m = 0;
    while ((2 << m) <= mag) m++;  /* m = floor(log2(mag))                      */
    /* half an ulp of the result is 2^(m-24); the distance of log2 below e+1 is
     * k * 2^-24 / ln 2 for the k-th value below the power of two */
    return (int)floor(ldexp(0.6931471805599453, m));
}

static inline int32_t floor_log2_quirk(float amax)
{
    const uint32_t a = f2u(amax) & 0x7FFFFFFFu;
    const int E = (int)(a >> 23);
    const uint32_t M = a & 0x7FFFFFu;
    /* log2 of 0, Inf or NaN is -Inf/Inf/NaN; the fp32->int32 cast of those
     * yields INT32_MIN on x86 (mxfp/fake.py:45) */
    if (a == 0 || E == 255) return INT32_MIN;
    if (E == 0) return -127;  /* subnormal: any value <= -127 clamps the same */
    const int e = E - 127;
    const int up = (int)(0x7FFFFFu - M) < mxq_oracle_log2_roundup_count(e);
    return e + up;
}

/* ------------------------------------------------------------------------- */
/* exported entry points (C ABI, fp32 in / fp32 out; the Python wrapper does  */
/* the exact widening of bf16/fp16 inputs and the final .to(output_dtype))    */
/* ------------------------------------------------------------------------- */
void mxq_oracle_minifloat_extract(const float* x, uint16_t* codes, int64_t n,
                                  int eb, int fb, int is_finite, int rm)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) codes[i] = encode_one(x[i], eb, fb, is_finite, rm);
}

void mxq_oracle_minifloat_compose(const uint16_t* codes, float* out, int64_t n,
                                  int eb, int fb, int is_finite)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = decode_one(codes[i], eb, fb, is_finite);
}

void mxq_oracle_minifloat_qdq(const float* x, float* out, int64_t n,
                              int eb, int fb, int is_finite, int rm)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i)
        out[i] = decode_one(encode_one(x[i], eb, fb, is_finite, rm), eb, fb, is_finite);
}

/* follows src/mase_triton/mxfp/fake.py:11-59 */
void mxq_oracle_mxfp_extract(const float* x, uint8_t* scales, uint8_t* elements,
                             int64_t n, int B, int eb, int fb, int is_finite, int rm)
{
    const int bias = (1 << (eb - 1)) - 1;
    const int emax = is_finite ? (1 << eb) - 1 : (1 << eb) - 2;
    const int32_t emax_b = emax - bias;               /* fake.py:27-33 */
    const int64_t nb = n / B;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const float* xb = x + b * B;
        /* fake.py:43  abs().max() propagates NaN */
        float amax = 0.0f; int any_nan = 0; int all_flush = 1;
        for (int j = 0; j < B; ++j) {
            const uint32_t a = f2u(xb[j]) & 0x7FFFFFFFu;
            if (a > 0x7F800000u) any_nan = 1;
            else if (u2f(a) > amax) amax = u2f(a);
            if ((a & 0x7F800000u) != 0) all_flush = 0;   /* fake.py:39-41 */
        }
        if (any_nan) amax = NAN;
        int32_t l = floor_log2_quirk(amax);            /* fake.py:44-45 */
        int32_t se = (int32_t)((uint32_t)l - (uint32_t)emax_b);  /* wraps, fake.py:46 */
        if (se < -127) se = -127;                      /* fake.py:47 */
        if (se > 128) se = 128;
        scales[b] = all_flush ? 0 : (uint8_t)(se + 127);   /* fake.py:48-50 */
        const float sf = exp2_int(se);                 /* fake.py:52 */
        for (int j = 0; j < B; ++j) {
            const float v = xb[j];
            const int flush = (f2u(v) & 0x7F800000u) == 0;
            volatile float q = flush ? 0.0f : v / sf;  /* fake.py:54 */
            elements[b * B + j] = (uint8_t)encode_one(q, eb, fb, is_finite, rm); /* :55-57 */
        }
    }
}

/* follows src/mase_triton/mxfp/fake.py:62-79 */
void mxq_oracle_mxfp_compose(const uint8_t* scales, const uint8_t* elements, float* out,
                             int64_t n, int B, int eb, int fb, int is_finite)
{
    const int64_t nb = n / B;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const float sf = exp2_int((int)scales[b] - 127);         /* fake.py:71-72 */
        for (int j = 0; j < B; ++j) {
            volatile float v = decode_one((uint16_t)elements[b * B + j], eb, fb, is_finite);
            out[b * B + j] = v * sf;                              /* fake.py:77 */
        }
    }
}

void mxq_oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int mxq_oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
