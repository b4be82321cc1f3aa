// Element codec shared by every kernel of the library: fp32 bits <-> minifloat
// code, and the MXFP shared-exponent rule.  Everything here is integer (or one
// exact fp32 multiply) arithmetic that reproduces, bit for bit, the behaviour of
// mase-triton's pure-PyTorch path (src/mase_triton/minifloat/fake.py,
// src/mase_triton/mxfp/fake.py), including its documented oddities:
//   * the mantissa is cut to 15 bits before it is rounded (fake.py:45);
//   * exponent and mantissa are merged with a bitwise OR, so a rounding carry is
//     lost when the biased exponent is odd (fake.py:75);
//   * only the binade with biased exponent 0 is encoded as subnormal, by
//     (f | 2^fb) >> 1 after rounding (fake.py:58-60);
//   * floor(log2f(max)) rounds UP for the last few floats below a power of two
//     (mxfp/fake.py:44-45).
// The header compiles for host and device so the same arithmetic can be checked
// on a CPU against the oracle.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define MXQ_HD __host__ __device__ __forceinline__
#else
#define MXQ_HD inline
#endif

namespace mxq {

enum RoundMode : int { RM_RN = 0, RM_RU = 1, RM_RD = 2, RM_RZ = 3 };
enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };

// Format descriptor with compile-time fields (fast kernels) ...
template <int EB, int FB, bool FIN, int RM>
struct FmtCT {
    static constexpr bool kStatic = true;
    MXQ_HD constexpr int eb() const { return EB; }
    MXQ_HD constexpr int fb() const { return FB; }
    MXQ_HD constexpr bool fin() const { return FIN; }
    MXQ_HD constexpr int rm() const { return RM; }
};
// ... or run-time fields (any exp_bits + frac_bits < 16, any rounding mode).
struct FmtRT {
    static constexpr bool kStatic = false;
    int eb_, fb_, fin_, rm_;
    MXQ_HD int eb() const { return eb_; }
    MXQ_HD int fb() const { return fb_; }
    MXQ_HD bool fin() const { return fin_ != 0; }
    MXQ_HD int rm() const { return rm_; }
};

// Integer adds, subtractions and left shifts written as a * k + b with k read from constant
// memory: the compiler cannot fold k, so it emits an integer multiply-add, which issues on the
// fp32/FMA pipe instead of the (saturated) integer ALU pipe.
#if defined(__CUDACC__)
static __constant__ int mxq_rt_k[12] = {1, 4, 256, 65536, 1 << 24, 1 << 20, 1 << 21, 1 << 22, 0, 64, 16, 32};
#endif
MXQ_HD int rt_k(int i) {
#if defined(__CUDA_ARCH__)
    return mxq_rt_k[i];
#else
    return i == 0 ? 1 : i == 1 ? 4 : i == 2 ? 256 : i == 3 ? 65536 : i == 4 ? (1 << 24) : i <= 7 ? (1 << (15 + i)) : i == 9 ? 64 : i == 10 ? 16 : i == 11 ? 32 : 0;
#endif
}
// 2^(23 - fb) for fb = 1..3 as a run-time factor (entries 7, 6, 5)
MXQ_HD int rt_pow2_shift(int fb) { return rt_k(8 - fb); }
MXQ_HD int mad_add(int a, int b) { return a * rt_k(0) + b; }           // a + b

template <class F> MXQ_HD int fmt_bias(const F& f) { return (1 << (f.eb() - 1)) - 1; }
template <class F> MXQ_HD int fmt_emax(const F& f) { return f.fin() ? (1 << f.eb()) - 1 : (1 << f.eb()) - 2; }

MXQ_HD uint32_t f32_bits(float v) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(v);
#else
    uint32_t u; memcpy(&u, &v, 4); return u;
#endif
}
MXQ_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float v; memcpy(&v, &u, 4); return v;
#endif
}
// fp32 product without contraction, with subnormal operands and results kept
MXQ_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    volatile float r = a * b; return r;
#endif
}

// ---------------------------------------------------------------------------------------------
// Rounded mantissa field f in [0, 2^fb] from the 23-bit fp32 mantissa M (minifloat/fake.py:39-56)
// ---------------------------------------------------------------------------------------------
template <class F>
MXQ_HD int round_mantissa(uint32_t M, const F& f) {
    const int fb = f.fb();
    if (f.rm() == RM_RZ) return (int)(M >> (23 - fb));
    const int t = (int)(M >> 8);          // 15 bits: the low 8 are dropped first
    const int d = 15 - fb;
    const int q = t >> d;
    const int r = t & ((1 << d) - 1);
    if (f.rm() == RM_RD) return q;
    if (f.rm() == RM_RU) return q + (r != 0);
    const int half = 1 << (d - 1);        // round half to even
    return (t + (half - 1) + (q & 1)) >> d;
}

// ---------------------------------------------------------------------------------------------
// Full minifloat encode of one fp32 bit pattern (minifloat/fake.py:7-78). Any format, any mode.
// ---------------------------------------------------------------------------------------------
template <class F>
MXQ_HD uint32_t encode_f32(uint32_t u, const F& f) {
    const int eb = f.eb(), fb = f.fb();
    const uint32_t a = u & 0x7FFFFFFFu;
    const int E = (int)(a >> 23);
    uint32_t M = a & 0x7FFFFFu;
    const bool is_nan = a > 0x7F800000u;
    const bool is_inf = a == 0x7F800000u;
    const int bias = fmt_bias(f), emax = fmt_emax(f), fmax = (1 << fb) - 1;
    // x < 0: false for -0.0 and for NaN
    const bool neg = (u >> 31) && a != 0 && !is_nan;
    int xe = E - 127;
    if (E == 255) { xe = -1; if (is_nan) M |= 0x400000u; }   // frexp of Inf/NaN reports exponent 0
    int ye = xe + bias;
    int fr = round_mantissa(M, f);
    if (ye == 0 && fr != 0) fr = (fr | (1 << fb)) >> 1;
    if (xe < -bias) { fr = 0; ye = 0; }
    if (xe > emax - bias) { fr = fmax; ye = emax; }
    if (E == 0) { fr = 0; ye = 0; }
    if (!f.fin()) {
        if (is_inf) { fr = 0; ye = emax; }
        if (is_nan) { fr = fmax; ye = emax; }
    }
    uint32_t code = ((uint32_t)ye << fb) | (uint32_t)fr;
    if (neg) code += 1u << (eb + fb);
    return code & 0xFFFFu;
}

// ---------------------------------------------------------------------------------------------
// Fast encode core for the round-to-nearest presets (exp_bits <= 5, frac_bits <= 3).
// Most of the work is moved to the fp32 pipe:
//   * the mantissa, re-tagged with exponent 0 so it is a float in [1,2), is rounded half-to-even
//     to frac_bits by adding 2^(23-fb): the low bits of the sum are 2^fb + f with f in [0, 2^fb];
//   * exponent field and f are merged with OR, which reproduces the reference's lost carry;
//   * the single subnormal binade is a 9-entry table held in an immediate.
// qb : bits of the (possibly signed) fp32 value q to encode, its mantissa already cut to 15 bits.
// Returns the magnitude code; no overflow clamp, sign, Inf or NaN handling.
// ---------------------------------------------------------------------------------------------
template <int FB>
MXQ_HD constexpr uint64_t subnormal_table() {
    // entry k (4 bits): code of the biased-exponent-0 binade whose rounded mantissa field is k
    uint64_t t = 0;
    for (int k = 1; k <= (1 << FB); ++k) {
        const uint64_t c = (k == (1 << FB)) ? (1u << (FB - 1)) : (uint64_t)((k | (1 << FB)) >> 1);
        t |= c << (4 * k);
    }
    return t;
}

MXQ_HD float add_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    volatile float r = a + b; return r;
#endif
}

// The three pieces of the fast magnitude encode; encode_mag_fp below strings them together and the
// block quantiser calls them separately so that a whole warp can skip the sub-range piece.
//   encode_mag_normal : code as if the biased exponent were >= 1 (negative for smaller inputs)
//   is_subrange       : |q| < 2^(1-bias), i.e. biased exponent <= 0 (q is never NaN here)
//   subrange_code     : the code of such an input from what encode_mag_normal returned
template <class F>
MXQ_HD int encode_mag_normal(uint32_t qb, const F& f) {
    constexpr int fb = F{}.fb(), eb = F{}.eb();
    static_assert(fb >= 1 && fb <= 3 && eb <= 5, "table-driven subnormal path covers the built-in presets");
    constexpr int sh = 23 - fb;
    constexpr int bias = (1 << (eb - 1)) - 1;
    constexpr uint32_t cbits = (uint32_t)(127 + 23 - fb) << 23;           // 2^(23-fb)
    const float m = bits_f32((qb & 0x007FFFFFu) | 0x3F800000u);
    const int fr = mad_add((int)f32_bits(add_rn(m, bits_f32(cbits))), -(int)(cbits + (1u << fb)));   // 0 .. 2^fb
    (void)f;
    return mad_add((int)(((qb >> sh) & (0xFFu << fb)) | (uint32_t)fr), -((127 - bias) << fb));
}
template <class F>
MXQ_HD bool is_subrange(uint32_t qb, const F& f) {
    constexpr int bias = (1 << (F{}.eb() - 1)) - 1;
    (void)f;
    return __builtin_fabsf(bits_f32(qb)) < bits_f32((uint32_t)(128 - bias) << 23);
}
template <class F>
MXQ_HD int subrange_code(int code, const F& f) {
    constexpr int fb = F{}.fb();
    code = code < 0 ? 0 : code;                                            // biased exponent < 0
    (void)f;
    return (int)((subnormal_table<fb>() >> (code * rt_k(1))) & 0xFu);
}

template <class F>
MXQ_HD int encode_mag_fp(uint32_t qb, const F& f) {
    int code = encode_mag_normal(qb, f);
    if (is_subrange(qb, f)) code = subrange_code(code, f);
    return code;
}

// Minifloat encode, fast path (RN presets, is_finite): full semantics incl. overflow, Inf/NaN, flush.
template <class F>
MXQ_HD uint32_t encode_f32_fast(uint32_t u, const F& f) {
    const int eb = f.eb(), fb = f.fb();
    const int emax = fmt_emax(f);
    const uint32_t sign = 1u << (eb + fb);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) {                       // Inf / NaN: rare
        const bool is_nan = a > 0x7F800000u;
        if (!f.fin()) {
            uint32_t c = ((uint32_t)emax << fb) | (is_nan ? (uint32_t)((1 << fb) - 1) : 0u);
            if (!is_nan && (u >> 31)) c |= sign;
            return c;
        }
        // frexp reports exponent 0: treat as 0.5 * 1.m (m = quieted payload, 0 for Inf)
        const uint32_t m = is_nan ? ((a & 0x7FFFFFu) | 0x400000u) : 0u;
        a = (126u << 23) | m;
        u = is_nan ? a : ((u & 0x80000000u) | a);
    }
    // an fp32 subnormal has exponent field 0 and encodes as magnitude 0 by itself
    int code = encode_mag_fp(a & 0xFFFFFF00u, f);
    const int cmax = (emax << fb) | ((1 << fb) - 1);
    code = code > cmax ? cmax : code;             // emax is odd: a carry at emax was already dropped
    // x < 0 (false for -0.0; NaN was given a clear sign above)
    return (uint32_t)code | (u > 0x80000000u ? sign : 0u);
}

// Minifloat quantize-dequantize of one value, fast path: same result as
// decode_f32_fast(encode_f32_fast(u)) with the sign taken straight from x + 0.0
// (which is +0.0 for x = -0.0 and keeps the sign of everything else).
template <class F>
MXQ_HD uint32_t qdq_f32_fast(uint32_t u, const F& f);

// ---------------------------------------------------------------------------------------------
// Minifloat decode to fp32 bits (minifloat/fake.py:81-125). NaN results are 0x7FC00000 with the
// code's sign, as the reference's host produces them.
// ---------------------------------------------------------------------------------------------
MXQ_HD float exp2_int(int k) {
    if (k > 127) return bits_f32(0x7F800000u);
    if (k >= -126) return bits_f32((uint32_t)(k + 127) << 23);
    if (k >= -149) return bits_f32(1u << (k + 149));
    return 0.0f;
}

template <class F>
MXQ_HD uint32_t decode_f32(uint32_t code, const F& f) {
    const int eb = f.eb(), fb = f.fb();
    const uint32_t sign = (code >> (eb + fb)) & 1u;
    const uint32_t c = code & 0x7FFFu;
    const int e = (int)((c >> fb) & ((1u << eb) - 1u));
    const int fr = (int)(c & ((1u << fb) - 1u));
    const int bias = fmt_bias(f);
    uint32_t y;
    if (e == 0 && fr == 0) y = 0u;
    else if (!f.fin() && e == (1 << eb) - 1) y = fr == 0 ? 0x7F800000u : 0x7FC00000u;
    else {
        const bool sub = (e == 0);
        const float p = exp2_int(e - bias + (sub ? 1 : 0));
        const float m = (float)fr / (float)(1 << fb) + (sub ? 0.0f : 1.0f);   // exact
        y = f32_bits(mul_rn(p, m));
    }
    return y | (sign << 31);
}

// Fast decode for formats with exp_bits <= 7 whose code fits 8 bits... or any code width:
// the magnitude field, placed at the top of an fp32 mantissa/exponent, is a tiny fp32 number
// (subnormal when e == 0) that one exact multiply by 2^(127-bias) turns into the value.
template <class F>
MXQ_HD uint32_t decode_f32_fast(uint32_t code, const F& f) {
    const int eb = f.eb(), fb = f.fb();
    const uint32_t mag = code & ((1u << (eb + fb)) - 1u);
    const uint32_t sign = (code << (31 - eb - fb)) & 0x80000000u;
    uint32_t y = f32_bits(mul_rn(bits_f32(mag << (23 - fb)), bits_f32((uint32_t)(254 - fmt_bias(f)) << 23)));
    if (!f.fin() && (mag >> fb) == (1u << eb) - 1u) y = (mag & ((1u << fb) - 1u)) ? 0x7FC00000u : 0x7F800000u;
    return y | sign;
}

// Quantised magnitude of a finite value, built directly in the fp32 bit domain without forming
// the code (RN presets):
//   * normal range (biased exponent >= 1): the rounded mantissa field fr << (23-fb) is OR-ed under
//     the input's own exponent field -- fr = 2^fb lands on exponent bit 23, which is the reference's
//     OR-merge (carry kept for even exponent fields, lost for odd ones);
//   * below 2^(1-bias): the single subnormal binade comes from the 9-entry table, anything below
//     2^-bias is zero.
// qb: fp32 bits of the value (sign ignored, mantissa cut to 15 bits here). No saturation.
// qdq_mag_normal returns the normal-range result and the rounding sum that qdq_mag_subrange needs.
template <class F>
MXQ_HD uint32_t qdq_mag_normal(uint32_t qb, uint32_t* sum_out, const F& f) {
    constexpr int fb = F{}.fb(), eb = F{}.eb();
    static_assert(fb >= 1 && fb <= 3 && eb <= 5, "table-driven subnormal path covers the built-in presets");
    constexpr uint32_t cbits = (uint32_t)(127 + 23 - fb) << 23;           // 2^(23-fb)
    // mantissa cut to 15 bits, tagged with exponent 0, rounded half-to-even to fb bits by the add:
    // the sum's bits are cbits + 2^fb + fr, fr in [0, 2^fb]
    const uint32_t sum = f32_bits(add_rn(bits_f32((qb & 0x007FFF00u) | 0x3F800000u), bits_f32(cbits)));
    *sum_out = sum;
    // (sum << (23-fb)) = 2^23 + (fr << (23-fb)) modulo 2^32; written as a multiply-add for the FMA pipe
    const uint32_t z = sum * (uint32_t)rt_pow2_shift(fb) - 0x800000u;
    (void)f;
    return (qb & 0x7F800000u) | z;
}
// |q| < 2^(1-bias): the subnormal binade from the table, zero below it
template <class F>
MXQ_HD uint32_t qdq_mag_subrange(uint32_t qb, uint32_t sum, const F& f) {
    constexpr int fb = F{}.fb(), eb = F{}.eb();
    constexpr int bias = (1 << (eb - 1)) - 1;
    constexpr uint32_t cbits = (uint32_t)(127 + 23 - fb) << 23;
    const uint32_t idx4 = sum * (uint32_t)rt_k(1) - (cbits + (1u << fb)) * 4u;              // 4 * fr (modulo 2^32)
    uint32_t c0 = (uint32_t)(subnormal_table<fb>() >> idx4) & 0xFu;
    c0 = __builtin_fabsf(bits_f32(qb)) < bits_f32((uint32_t)(127 - bias) << 23) ? 0u : c0;  // below the binade: zero
    (void)f;
    return f32_bits(mul_rn(bits_f32(c0 * (uint32_t)rt_pow2_shift(fb)), bits_f32((uint32_t)(254 - bias) << 23)));
}
template <class F>
MXQ_HD uint32_t qdq_mag_bits(uint32_t qb, const F& f) {
    uint32_t sum;
    uint32_t y = qdq_mag_normal(qb, &sum, f);
    if (is_subrange(qb, f)) y = qdq_mag_subrange(qb, sum, f);
    return y;
}

template <class F>
MXQ_HD uint32_t qdq_f32_fast(uint32_t u, const F& f) {
    constexpr int fb = F{}.fb(), eb = F{}.eb();
    constexpr int bias = (1 << (eb - 1)) - 1;
    uint32_t a = u & 0x7FFFFFFFu;
    uint32_t s = f32_bits(add_rn(bits_f32(u), 0.0f));                     // sign bit: set for x < 0 only
    if (a >= 0x7F800000u) {                       // Inf / NaN: rare; same rule as encode_f32_fast
        const bool is_nan = a > 0x7F800000u;
        a = (126u << 23) | (is_nan ? ((a & 0x7FFFFFu) | 0x400000u) : 0u);
        s = is_nan ? 0u : u;
    }
    uint32_t y = qdq_mag_bits(a, f);
    constexpr int emax = F{}.fin() ? (1 << eb) - 1 : (1 << eb) - 2;
    constexpr uint32_t ymax = ((uint32_t)(emax - bias + 127) << 23) | (((1u << fb) - 1u) << (23 - fb));
    y = y > ymax ? ymax : y;                      // saturate (emax is odd: a carry at emax was already dropped)
    return y | (s & 0x80000000u);
}

// ---------------------------------------------------------------------------------------------
// MXFP shared exponent (mxfp/fake.py:43-50).
//   amax_bits : max over the block of |x| bit patterns compared as unsigned integers
//               (any NaN compares above Inf, which compares above every finite value)
// Returns se in [-127, 128]; *scale_byte is what the reference stores (0 for an all-flushed block)
// ---------------------------------------------------------------------------------------------
MXQ_HD int log2_roundup_count(int e) {
    // number of fp32 values just below 2^(e+1) whose floor(log2f()) is e+1 (correctly rounded log2f)
    int mag;
    if (e >= 1) mag = e; else if (e <= -3) mag = -e - 1; else return 0;
    int m = 0;
    while ((2 << m) <= mag) ++m;
    // floor(2^m * ln 2) for m = 0..6 is 0, 1, 2, 5, 11, 22, 44 (one byte each)
    return (int)((0x2C160B05020100ull >> (8 * m)) & 0xFFu);
}

template <class F>
MXQ_HD int shared_exponent(uint32_t amax_bits, const F& f, uint32_t* scale_byte) {
    const int emax_b = fmt_emax(f) - fmt_bias(f);
    const uint32_t E = amax_bits >> 23;
    int se;
    if (amax_bits == 0u || E == 255u) se = 128;      // log2 -> -Inf/Inf/NaN -> INT_MIN, wraps, clamps
    else if (E == 0u) se = -127;
    else {
        const int e = (int)E - 127;
        const int M = (int)(amax_bits & 0x7FFFFFu);
        int l = e;
        if (M > 0x7FFFFF - 64 && (0x7FFFFF - M) < log2_roundup_count(e)) l = e + 1;
        se = l - emax_b;
        if (se < -127) se = -127;
    }
    *scale_byte = (E == 0u) ? 0u : (uint32_t)(se + 127);
    return se;
}

// Element of an MXFP block: code of fp32(x / 2^se) (mxfp/fake.py:54-57 + minifloat extract).
// Generic version (any mode / format); the quotient is formed in integer arithmetic.
template <class F>
MXQ_HD uint32_t mx_encode(uint32_t u, int se, const F& f) {
    const uint32_t a = u & 0x7FFFFFFFu;
    const int E = (int)(a >> 23);
    if (E == 0) return 0u;                              // flushed input -> +0.0
    uint32_t q;
    if (E == 255) {
        // finite divisor keeps Inf/NaN; 2^128 overflows to Inf: Inf/Inf is the default NaN
        if (se == 128) q = (a > 0x7F800000u) ? (u | 0x400000u) : 0xFFC00000u;
        else q = (a > 0x7F800000u) ? (u | 0x400000u) : u;
    } else if (se == 128) {
        q = u & 0x80000000u;                            // finite / Inf = signed zero
    } else {
        const int Eq = E - se;
        if (Eq >= 255) q = (u & 0x80000000u) | 0x7F800000u;     // cannot happen for a block maximum
        else if (Eq >= 1) q = (u & 0x80000000u) | ((uint32_t)Eq << 23) | (a & 0x7FFFFFu);
        else {
            // quotient is an fp32 subnormal or zero: the encoder flushes it, only "non-zero and
            // negative" survives as the sign bit. Non-zero iff it is above 2^-150 (ties to even).
            const bool nonzero = Eq > -23 || (Eq == -23 && (a & 0x7FFFFFu) != 0);
            q = (u & 0x80000000u) | (nonzero ? 1u : 0u);
        }
    }
    return encode_f32(q, f) & 0xFFu;
}

// Flush-to-zero of subnormal operands: x * 1.0 with the .ftz modifier (sign is kept).
MXQ_HD float flush_subnormal(float x) {
#if defined(__CUDA_ARCH__)
    float r;
    asm("mul.ftz.f32 %0, %1, 0f3F800000;" : "=f"(r) : "f"(x));
    return r;
#else
    return ((f32_bits(x) & 0x7F800000u) == 0u) ? bits_f32(f32_bits(x) & 0x80000000u) : x;
#endif
}
// Fast MXFP element encode (RN presets, finite block).
//   inv_scale = 2^-se as an fp32 value (se in [-127, 127] for a finite block).
// The quotient is formed by a real fp32 multiply (exact for a power of two, rounded like the
// reference's division when it lands in the subnormal range), so "bits above 0x80000000" says
// exactly "negative and non-zero after the reference's flush".
// mx_quotient_bits: the quotient plus (+0.0), so that its sign bit alone says "negative and non-zero".
MXQ_HD uint32_t mx_quotient_bits(uint32_t u, float inv_scale) {
    return f32_bits(add_rn(mul_rn(flush_subnormal(bits_f32(u & 0xFFFFFF00u)), inv_scale), 0.0f));
}
template <class F>
MXQ_HD uint32_t mx_encode_fast(uint32_t u, float inv_scale, const F& f) {
    const uint32_t qb = mx_quotient_bits(u, inv_scale);
    const uint32_t code = (uint32_t)encode_mag_fp(qb, f);
    return code | ((qb >> (31 - f.eb() - f.fb())) & (1u << (f.eb() + f.fb())));
}

// Fast fused MXFP quantize-dequantize of one element of a finite block (RN presets): the quantised
// quotient, built in the fp32 bit domain, times 2^se; the sign is that of the non-zero quotient.
template <class F>
MXQ_HD uint32_t mx_qdq_fast(uint32_t u, float inv_scale, float scale, const F& f) {
    const uint32_t qb = mx_quotient_bits(u, inv_scale);
    return f32_bits(mul_rn(bits_f32(qdq_mag_bits(qb, f)), scale)) | (qb & 0x80000000u);
}

// MXFP compose of one element (mxfp/fake.py:71-78): decode(code) * 2^(scale-127) in fp32.
template <class F>
MXQ_HD uint32_t mx_decode(uint32_t code, float scale_f, const F& f) {
    const uint32_t v = decode_f32_fast(code, f);
    uint32_t y = f32_bits(mul_rn(bits_f32(v), scale_f));
    // 0 * Inf: the reference's host yields the negative default NaN; an element NaN keeps its sign
    if ((y & 0x7FFFFFFFu) > 0x7F800000u) y = ((v & 0x7FFFFFFFu) > 0x7F800000u) ? (v | 0x400000u) : 0xFFC00000u;
    return y;
}

}  // namespace mxq
