// CPU harness around mase_triton_b200/csrc/mxq_codec.h: runs, on the host, exactly the
// element arithmetic the CUDA kernels use, so it can be compared with the oracle
// without a GPU. Built by tests/test_codec_host.py with g++.
#include <stdint.h>

#include "../../mase_triton_b200/csrc/mxq_codec.h"

using namespace mxq;

template <class Fn>
static bool with_preset(int eb, int fb, int fin, int rm, Fn&& fn) {
    if (rm != RM_RN || !fin) return false;
    if (eb == 4 && fb == 3) { fn(FmtCT<4, 3, true, RM_RN>{}); return true; }
    if (eb == 5 && fb == 2) { fn(FmtCT<5, 2, true, RM_RN>{}); return true; }
    if (eb == 2 && fb == 3) { fn(FmtCT<2, 3, true, RM_RN>{}); return true; }
    if (eb == 3 && fb == 2) { fn(FmtCT<3, 2, true, RM_RN>{}); return true; }
    if (eb == 2 && fb == 1) { fn(FmtCT<2, 1, true, RM_RN>{}); return true; }
    return false;
}

// returns 1 when the fast (compile-time format) path was used
extern "C" int hc_minifloat_encode(const uint32_t* bits, uint16_t* out, int64_t n, int eb, int fb, int fin, int rm, int fast) {
    if (fast && with_preset(eb, fb, fin, rm, [&](auto f) { for (int64_t i = 0; i < n; ++i) out[i] = (uint16_t)encode_f32_fast(bits[i], f); }))
        return 1;
    FmtRT f{eb, fb, fin, rm};
    for (int64_t i = 0; i < n; ++i) out[i] = (uint16_t)encode_f32(bits[i], f);
    return 0;
}

extern "C" int hc_minifloat_qdq(const uint32_t* bits, uint32_t* out, int64_t n, int eb, int fb, int fin, int rm, int fast) {
    if (fast && with_preset(eb, fb, fin, rm, [&](auto f) { for (int64_t i = 0; i < n; ++i) out[i] = qdq_f32_fast(bits[i], f); }))
        return 1;
    FmtRT f{eb, fb, fin, rm};
    for (int64_t i = 0; i < n; ++i) out[i] = decode_f32(encode_f32(bits[i], f), f);
    return 0;
}

extern "C" int hc_minifloat_decode(const uint16_t* codes, uint32_t* out, int64_t n, int eb, int fb, int fin, int fast) {
    if (fast && with_preset(eb, fb, fin, RM_RN, [&](auto f) { for (int64_t i = 0; i < n; ++i) out[i] = decode_f32_fast(codes[i], f); }))
        return 1;
    FmtRT f{eb, fb, fin, 0};
    for (int64_t i = 0; i < n; ++i) out[i] = decode_f32(codes[i], f);
    return 0;
}

template <class F>
static void mx_extract_blocks(const uint32_t* bits, uint8_t* scales, uint8_t* el, int64_t nb, int B, const F& f, bool fast) {
    for (int64_t b = 0; b < nb; ++b) {
        uint32_t amax = 0;
        for (int j = 0; j < B; ++j) { const uint32_t a = bits[b * B + j] & 0x7FFFFFFFu; amax = a > amax ? a : amax; }
        uint32_t sbyte;
        const int se = shared_exponent(amax, f, &sbyte);
        scales[b] = (uint8_t)sbyte;
        const bool special = amax >= 0x7F800000u;
        // 2^-se; an all-flushed block (se = 128 or -127) encodes to zeros with any finite factor
        const float inv = bits_f32((amax >> 23) == 0u ? 0x3F800000u : (uint32_t)(127 - se) << 23);
        for (int j = 0; j < B; ++j) {
            const uint32_t u = bits[b * B + j];
            if constexpr (F::kStatic) el[b * B + j] = (uint8_t)((fast && !special) ? mx_encode_fast(u, inv, f) : mx_encode(u, se, f));
            else el[b * B + j] = (uint8_t)mx_encode(u, se, f);
        }
    }
}

extern "C" int hc_mxfp_extract(const uint32_t* bits, uint8_t* scales, uint8_t* el, int64_t n, int B, int eb, int fb, int fin, int rm, int fast) {
    if (fast && with_preset(eb, fb, fin, rm, [&](auto f) { mx_extract_blocks(bits, scales, el, n / B, B, f, true); })) return 1;
    mx_extract_blocks(bits, scales, el, n / B, B, FmtRT{eb, fb, fin, rm}, false);
    return 0;
}

template <class F>
static void mx_compose_blocks(const uint8_t* scales, const uint8_t* el, uint32_t* out, int64_t nb, int B, const F& f, bool fast) {
    for (int64_t b = 0; b < nb; ++b) {
        const uint32_t s = scales[b];
        const float sf = bits_f32(s == 0u ? 0x00400000u : (s << 23));
        for (int j = 0; j < B; ++j) {
            const uint32_t c = el[b * B + j];
            if (fast && s != 255u) out[b * B + j] = f32_bits(mul_rn(bits_f32(decode_f32_fast(c, f)), sf));
            else out[b * B + j] = mx_decode(c, sf, f);
        }
    }
}

extern "C" int hc_mxfp_compose(const uint8_t* scales, const uint8_t* el, uint32_t* out, int64_t n, int B, int eb, int fb, int fin, int fast) {
    if (fast && with_preset(eb, fb, fin, RM_RN, [&](auto f) { mx_compose_blocks(scales, el, out, n / B, B, f, true); })) return 1;
    mx_compose_blocks(scales, el, out, n / B, B, FmtRT{eb, fb, fin, 0}, false);
    return 0;
}

extern "C" int hc_log2_roundup_count(int e) { return log2_roundup_count(e); }

// fused quantize-dequantize of 32-blocks with the kernels' fast arithmetic (finite blocks) and the
// generic encode + decode for blocks holding Inf/NaN
template <class F>
static void mx_qdq_blocks(const uint32_t* bits, uint32_t* out, int64_t nb, int B, const F& f) {
    for (int64_t b = 0; b < nb; ++b) {
        uint32_t amax = 0;
        for (int j = 0; j < B; ++j) { const uint32_t a = bits[b * B + j] & 0x7FFFFFFFu; amax = a > amax ? a : amax; }
        uint32_t sbyte;
        const int se = shared_exponent(amax, f, &sbyte);
        const bool special = amax >= 0x7F800000u;
        const float inv = bits_f32((amax >> 23) == 0u ? 0x3F800000u : (uint32_t)(127 - se) << 23);
        const float sf = bits_f32(sbyte == 0u ? 0x00400000u : (sbyte << 23));
        for (int j = 0; j < B; ++j) {
            const uint32_t u = bits[b * B + j];
            out[b * B + j] = special ? mx_decode(mx_encode(u, se, f), sf, f) : mx_qdq_fast(u, inv, sf, f);
        }
    }
}

extern "C" int hc_mxfp_qdq(const uint32_t* bits, uint32_t* out, int64_t n, int B, int eb, int fb, int fin, int rm) {
    return with_preset(eb, fb, fin, rm, [&](auto f) { mx_qdq_blocks(bits, out, n / B, B, f); }) ? 1 : 0;
}
