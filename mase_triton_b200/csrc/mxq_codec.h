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
// Fast encode core for round-to-nearest formats with exp_bits <= 7.
//   ar = |x| bits minus ((127 - bias) << 23), as a signed integer: its "exponent field" is the
//        biased minifloat exponent ye (possibly negative), its low 23 bits the fp32 mantissa.
// Returns the unsigned magnitude code, WITHOUT the overflow clamp (callers that can overflow
// apply it) and without sign / flush / Inf / NaN handling.
// ---------------------------------------------------------------------------------------------
template <class F>
MXQ_HD int encode_mag_rn(int ar, const F& f) {
    const int fb = f.fb();
    const int sh = 23 - fb;
    // mantissa: drop the low 8 bits, round half-to-even at bit sh; a carry stays inside fr
    const int t = ar & 0x007FFF00;
    const int lsb = (ar >> (sh - 8)) & 0x100;
    const int fr = (t + (((1 << (sh - 9)) - 1) << 8) + lsb) >> sh;          // 0 .. 2^fb
    // exponent field shifted into place; OR (not add) keeps the reference's lost carry
    int code = ((ar >> sh) & ~((1 << fb) - 1)) | fr;
    // ye < 0 leaves a negative number here: underflow -> 0
    code = code < 0 ? 0 : code;
    // ye == 0: the single subnormal binade
    if ((unsigned)ar < 0x00800000u && fr != 0) code = (fr | (1 << fb)) >> 1;
    return code;
}

// Minifloat encode, fast path (RN, exp_bits <= 7): full semantics incl. overflow, Inf/NaN, flush.
template <class F>
MXQ_HD uint32_t encode_f32_fast(uint32_t u, const F& f) {
    const int eb = f.eb(), fb = f.fb();
    const int bias = fmt_bias(f), emax = fmt_emax(f);
    uint32_t a = u & 0x7FFFFFFFu;
    const uint32_t sign = 1u << (eb + fb);
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
    if (a < 0x00800000u)                          // fp32 zero / subnormal: flushed, keeps x<0
        return ((u >> 31) && a != 0) ? sign : 0u;
    int code = encode_mag_rn((int)a - ((127 - bias) << 23), f);
    const int cmax = (emax << fb) | ((1 << fb) - 1);
    // ye > emax saturates; ye == emax with a rounding carry already lost it through the OR
    if ((int)(a >> 23) - 127 + bias > emax) code = cmax;
    return (uint32_t)code | ((u >> 31) ? sign : 0u);
}

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

// Fast MXFP element encode (RN, finite block, -127 <= se <= 127):
//   rebase = (se + 127 - bias) << 23 precomputed per block.
template <class F>
MXQ_HD uint32_t mx_encode_fast(uint32_t u, int rebase, const F& f) {
    const uint32_t a = u & 0x7FFFFFFFu;
    const int ar = (int)a - rebase;
    int code = encode_mag_rn(ar, f);
    const bool normal_in = a >= 0x00800000u;
    // the quotient's own exponent field is (ar >> 23) + 127 - bias; it is non-zero in fp32 iff
    // that exceeds -23, or equals -23 with a non-zero mantissa
    const bool q_nonzero = ar > (fmt_bias(f) - 150) * (1 << 23);
    if (!normal_in) code = 0;
    if ((u >> 31) && normal_in && q_nonzero) code |= 1 << (f.eb() + f.fb());
    return (uint32_t)code & 0xFFu;
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
