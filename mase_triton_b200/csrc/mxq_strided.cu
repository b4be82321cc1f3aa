// MXFP kernels for blocks that do NOT run along the contiguous dimension.
//
// The tensor is seen as [outer, D, inner] (row-major, contiguous); the 32-element blocks run
// along D, so the elements of one block sit `inner` elements apart.  The reference first moves
// the block dimension last with a permute + copy (src/mase_triton/mxfp/helpers.py:4-20) and then
// quantises the flat result; these kernels read the original layout directly and write
//   elements : [(o * inner + i) * D + j]        (the order the permuted copy would have had)
//   scales   : [(o * inner + i) * (D / 32) + j / 32]
// so the bytes are identical to the reference's and the extra 2 x sizeof(x) B/element pass is gone.
//
// One thread owns one column i (two adjacent columns for 16-bit inputs) of one block: it reads its
// 32 values with 32 row-strided accesses that are coalesced across the lanes of the warp, reduces
// the block maximum in registers (no shuffles), and writes its 32 code bytes with two 16-byte
// stores.  A CTA of 256 threads covers 4 consecutive blocks (128 rows) of 64 or 128 columns, so the
// four 32-byte code runs of one column form one 128-byte line.
#include "mxq_device.cuh"

namespace mxq {

constexpr int kStridedQdqMinBlocks = 2;   // resident CTAs per SM asked of the fused kernel (caps its registers)

constexpr int kRowBlocks = 4;          // blocks along D per CTA
constexpr int kColThreads = kThreads / kRowBlocks;

struct StridedGeom {
    int64_t D, inner;
    uint32_t tiles_i, tiles_j;
};

template <int CPT, class K>
__device__ __forceinline__ uint32_t column_bits(uint32_t raw, int col) {
    if constexpr (K::size == 4) return raw;
    else if constexpr (std::is_same<K, KBF16>::value) {
        if constexpr (CPT == 2) return col ? (raw & 0xFFFF0000u) : (raw << 16);
        else return raw << 16;
    } else {
        return K::to_bits(CPT == 2 ? ((raw >> (16 * col)) & 0xFFFFu) : (raw & 0xFFFFu));
    }
}

template <class K, int CPT>
__device__ __forceinline__ uint32_t load_cols(const char* p) {
    if constexpr (K::size * CPT == 4) return __ldcs(reinterpret_cast<const unsigned int*>(p));
    else return (uint32_t)__ldcs(reinterpret_cast<const unsigned short*>(p));
}

// fp32 bits of max |x| down each column of a thread (any NaN wins); packed 16-bit maxima when a
// thread holds two columns per word
template <int CPT, class K>
__device__ __forceinline__ void column_absmax(const uint32_t (&raw)[32], uint32_t (&amax)[CPT]) {
    if constexpr (CPT == 2 && std::is_same<K, KBF16>::value) {
        __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw[0]));
#pragma unroll
        for (int k = 1; k < 32; ++k) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw[k])));
        const uint32_t mw = *reinterpret_cast<uint32_t*>(&m);
        amax[0] = mw << 16;
        amax[1] = mw & 0xFFFF0000u;
    } else if constexpr (CPT == 2) {
        __half2 m = __habs2(*reinterpret_cast<const __half2*>(&raw[0]));
#pragma unroll
        for (int k = 1; k < 32; ++k) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __half2*>(&raw[k])));
        const float2 mf = __half22float2(m);
        amax[0] = __float_as_uint(mf.x);
        amax[1] = __float_as_uint(mf.y);
    } else {
        float m = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) m = max_abs_nan(m, __uint_as_float(column_bits<CPT, K>(raw[k], 0)));
        amax[0] = __float_as_uint(m);
    }
}

// the CPT results of one row of a thread -> memory; PLAIN promises that none is NaN
template <class K, int CPT, bool PLAIN>
__device__ __forceinline__ void store_row(char* d, const uint32_t (&y)[CPT]) {
    if constexpr (K::size == 4) {
        __stcs(reinterpret_cast<unsigned int*>(d), y[0]);
    } else if constexpr (CPT == 2) {
        uint32_t w;
        if constexpr (PLAIN && std::is_same<K, KBF16>::value) {
            const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(y[0]), __uint_as_float(y[1]));
            w = *reinterpret_cast<const uint32_t*>(&hh);
        } else if constexpr (PLAIN) {
            const __half2 hh = __floats2half2_rn(__uint_as_float(y[0]), __uint_as_float(y[1]));
            w = *reinterpret_cast<const uint32_t*>(&hh);
        } else {
            w = K::from_bits(y[0]) | (K::from_bits(y[1]) << 16);
        }
        __stcs(reinterpret_cast<unsigned int*>(d), w);
    } else {
        __stcs(reinterpret_cast<unsigned short*>(d), (unsigned short)K::from_bits(y[0]));
    }
}

// decomposes the CTA index into (column tile, block tile, outer index) and returns false for
// threads that fall outside the tensor
template <int CPT>
__device__ __forceinline__ bool strided_position(const StridedGeom& g, int64_t& o, int64_t& jb, int64_t& i0) {
    const uint32_t bid = blockIdx.x;
    const uint32_t ti = bid % g.tiles_i;
    const uint32_t r = bid / g.tiles_i;
    const uint32_t tj = r % g.tiles_j;
    o = r / g.tiles_j;
    const int c = threadIdx.x % kColThreads, rb = threadIdx.x / kColThreads;
    i0 = ((int64_t)ti * kColThreads + c) * CPT;
    jb = (int64_t)tj * kRowBlocks + rb;
    return i0 < g.inner && jb * 32 < g.D;
}

template <class KIn, class F, int CPT, int MODE>
__global__ void __launch_bounds__(kThreads, MODE == MODE_QDQ ? kStridedQdqMinBlocks : 1) mxfp_strided_quant_kernel(const void* __restrict__ x, uint8_t* __restrict__ scales,
                                                                      uint8_t* __restrict__ elements, void* __restrict__ out,
                                                                      StridedGeom g, F f) {
    int64_t o, jb, i0;
    if (!strided_position<CPT>(g, o, jb, i0)) return;
    const int64_t row_bytes = g.inner * KIn::size;
    const int64_t first = ((o * g.D + jb * 32) * g.inner + i0) * KIn::size;
    const char* src = reinterpret_cast<const char*>(x) + first;
    uint32_t raw[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) raw[k] = load_cols<KIn, CPT>(src + k * row_bytes);

    uint32_t h[CPT];
    {
        uint32_t amax[CPT];
        column_absmax<CPT, KIn>(raw, amax);
#pragma unroll
        for (int col = 0; col < CPT; ++col) h[col] = block_header(amax[col], f);
    }
    bool special = false;
#pragma unroll
    for (int col = 0; col < CPT; ++col) special = special || (h[col] & 1u);

    if constexpr (MODE == MODE_CODES) {
#pragma unroll
        for (int col = 0; col < CPT; ++col) {
            const int64_t colidx = o * g.inner + i0 + col;
            scales[colidx * (g.D / 32) + jb] = (uint8_t)(h[col] >> 8);
            uint32_t words[8];
            if (!(h[col] & 1u)) {
                const float inv = __uint_as_float(h[col] & 0x7F800000u);
#pragma unroll
                for (int k4 = 0; k4 < 32; k4 += 4) {
                    uint32_t qb[4], mag[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        qb[k] = mx_quotient_bits(column_bits<CPT, KIn>(raw[k4 + k], col), inv);
                        mag[k] = (uint32_t)encode_mag_fp(qb[k], f);
                    }
                    words[k4 >> 2] = pack4_codes(mag, qb, f);
                }
            } else {
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    const uint32_t code = mx_encode(column_bits<CPT, KIn>(raw[k], col), 128, f);
                    if ((k & 3) == 0) words[k >> 2] = code; else words[k >> 2] |= code << (8 * (k & 3));
                }
            }
            uint4* d = reinterpret_cast<uint4*>(elements + colidx * g.D + jb * 32);
            __stcs(d, make_uint4(words[0], words[1], words[2], words[3]));
            __stcs(d + 1, make_uint4(words[4], words[5], words[6], words[7]));
        }
    } else {
        // results leave row by row, both columns of a thread in one store
        char* dst = reinterpret_cast<char*>(out) + first;
        float inv[CPT], sf[CPT];
        int se[CPT];
#pragma unroll
        for (int col = 0; col < CPT; ++col) {
            inv[col] = __uint_as_float(h[col] & 0x7F800000u);
            sf[col] = scale_from_byte((h[col] >> 8) & 0xFFu);
            se[col] = (h[col] & 1u) ? 128 : 127 - (int)((h[col] >> 23) & 0xFFu);
        }
        const float unbias = __uint_as_float((uint32_t)(254 - fmt_bias(f)) << 23);
        if (!special) {
#pragma unroll
            for (int k = 0; k < 32; ++k) {
                uint32_t y[CPT];
#pragma unroll
                for (int col = 0; col < CPT; ++col) {
                    // code then decode (cheaper here than the bit-domain form, whose sub-range test would
                    // be a branch in each of the 32 x CPT unrolled element slots)
                    const uint32_t qb = mx_quotient_bits(column_bits<CPT, KIn>(raw[k], col), inv[col]);
                    const uint32_t mag = (uint32_t)encode_mag_fp(qb, f);
                    const float v = __fmul_rn(__uint_as_float((uint32_t)((int)mag * rt_k(0)) << (23 - f.fb())), unbias);
                    y[col] = __float_as_uint(__fmul_rn(v, sf[col])) | (qb & 0x80000000u);
                }
                store_row<KIn, CPT, true>(dst + k * row_bytes, y);
            }
        } else {
            // a column of this thread holds Inf/NaN: element-by-element generic arithmetic for the pair
#pragma unroll
            for (int k = 0; k < 32; ++k) {
                uint32_t y[CPT];
#pragma unroll
                for (int col = 0; col < CPT; ++col)
                    y[col] = mx_decode(mx_encode(column_bits<CPT, KIn>(raw[k], col), se[col], f), sf[col], f);
                store_row<KIn, CPT, false>(dst + k * row_bytes, y);
            }
        }
    }
}

template <class KOut, class F, int CPT>
__global__ void __launch_bounds__(kThreads) mxfp_strided_compose_kernel(const uint8_t* __restrict__ scales,
                                                                        const uint8_t* __restrict__ elements,
                                                                        void* __restrict__ out, StridedGeom g, F f) {
    int64_t o, jb, i0;
    if (!strided_position<CPT>(g, o, jb, i0)) return;
    const int64_t row_bytes = g.inner * KOut::size;
    uint32_t words[CPT][8];
    uint32_t sb[CPT];
#pragma unroll
    for (int col = 0; col < CPT; ++col) {
        const int64_t colidx = o * g.inner + i0 + col;
        const uint4* s = reinterpret_cast<const uint4*>(elements + colidx * g.D + jb * 32);
        const uint4 a = __ldcs(s), b = __ldcs(s + 1);
        words[col][0] = a.x; words[col][1] = a.y; words[col][2] = a.z; words[col][3] = a.w;
        words[col][4] = b.x; words[col][5] = b.y; words[col][6] = b.z; words[col][7] = b.w;
        sb[col] = __ldg(scales + colidx * (g.D / 32) + jb);
    }
    char* dst = reinterpret_cast<char*>(out) + ((o * g.D + jb * 32) * g.inner + i0) * KOut::size;
    bool plain = true;
#pragma unroll
    for (int col = 0; col < CPT; ++col) plain = plain && (sb[col] != 255u);
    float sf[CPT];
#pragma unroll
    for (int col = 0; col < CPT; ++col) sf[col] = scale_from_byte(sb[col]);
    if (plain) {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            uint32_t y[CPT];
#pragma unroll
            for (int col = 0; col < CPT; ++col) {
                const uint32_t code = (words[col][k >> 2] >> (8 * (k & 3))) & 0xFFu;
                y[col] = __float_as_uint(__fmul_rn(__uint_as_float(decode_f32_fast(code, f)), sf[col]));
            }
            store_row<KOut, CPT, true>(dst + k * row_bytes, y);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            uint32_t y[CPT];
#pragma unroll
            for (int col = 0; col < CPT; ++col) y[col] = mx_decode((words[col][k >> 2] >> (8 * (k & 3))) & 0xFFu, sf[col], f);
            store_row<KOut, CPT, false>(dst + k * row_bytes, y);
        }
    }
}

// true when the strided kernels cover the problem; fills the geometry
static bool strided_geometry(int64_t outer, int64_t D, int64_t inner, int B, int cpt, StridedGeom* g) {
    if (B != 32 || outer <= 0 || D <= 0 || inner <= 0 || D % 32 != 0) return false;
    const int64_t ti = (inner + (int64_t)kColThreads * cpt - 1) / ((int64_t)kColThreads * cpt);
    const int64_t tj = (D / 32 + kRowBlocks - 1) / kRowBlocks;
    if (ti >= (1ll << 31) || tj >= (1ll << 31) || outer * ti * tj >= (1ll << 31)) return false;
    g->D = D; g->inner = inner; g->tiles_i = (uint32_t)ti; g->tiles_j = (uint32_t)tj;
    return true;
}

// two columns per thread need an even inner extent and a 4-byte aligned base
static int columns_per_thread(int dtype, const void* p, int64_t inner) {
    return (dtype != MXQ_F32 && inner % 2 == 0 && reinterpret_cast<uintptr_t>(p) % 4 == 0) ? 2 : 1;
}

}  // namespace mxq

using namespace mxq;

template <int MODE>
static int strided_quant(const void* x, int x_dtype, uint8_t* scales, uint8_t* elements, void* out, int64_t outer, int64_t D,
                         int64_t inner, int B, int eb, int fb, int fin, int rm, cudaStream_t st) {
    const int cpt = columns_per_thread(x_dtype, x, inner);
    StridedGeom g;
    if (!strided_geometry(outer, D, inner, B, cpt, &g)) return MXQ_ESIZE;
    if (MODE == MODE_CODES && reinterpret_cast<uintptr_t>(elements) % 16 != 0) return MXQ_ESIZE;
    if (MODE == MODE_QDQ && cpt == 2 && reinterpret_cast<uintptr_t>(out) % 4 != 0) return MXQ_ESIZE;
    int rc = MXQ_OK;
    const unsigned grid = (unsigned)(outer * g.tiles_i * g.tiles_j);
    bool done = false;
    with_kind(x_dtype, [&](auto kin) {
        using KIn = decltype(kin);
        done = with_preset(eb, fb, fin, rm, [&](auto f) {
            using F = decltype(f);
            if constexpr (KIn::size == 4) {
                mxfp_strided_quant_kernel<KIn, F, 1, MODE><<<grid, kThreads, 0, st>>>(x, scales, elements, out, g, f);
            } else {
                if (cpt == 2) mxfp_strided_quant_kernel<KIn, F, 2, MODE><<<grid, kThreads, 0, st>>>(x, scales, elements, out, g, f);
                else mxfp_strided_quant_kernel<KIn, F, 1, MODE><<<grid, kThreads, 0, st>>>(x, scales, elements, out, g, f);
            }
            rc = check_launch();
        });
    });
    return done ? rc : MXQ_ESIZE;
}

extern "C" int mxq_mxfp_extract_strided(const void* x, int x_dtype, uint8_t* scales, uint8_t* elements, int64_t outer,
                                        int64_t D, int64_t inner, int B, int eb, int fb, int is_finite, int rm, void* stream) {
    if (outer < 0 || D < 0 || inner < 0 || B <= 0 || !valid_dtype(x_dtype) || !valid_mx_element(eb, fb, rm)) return MXQ_EINVAL;
    if (outer * D * inner == 0) return MXQ_OK;
    if (!x || !scales || !elements) return MXQ_EINVAL;
    return strided_quant<MODE_CODES>(x, x_dtype, scales, elements, nullptr, outer, D, inner, B, eb, fb, is_finite, rm, (cudaStream_t)stream);
}

extern "C" int mxq_mxfp_qdq_strided(const void* x, int x_dtype, void* out, int out_dtype, int64_t outer, int64_t D,
                                    int64_t inner, int B, int eb, int fb, int is_finite, int rm, void* stream) {
    if (outer < 0 || D < 0 || inner < 0 || B <= 0 || !valid_dtype(x_dtype) || !valid_dtype(out_dtype) || !valid_mx_element(eb, fb, rm)) return MXQ_EINVAL;
    if (outer * D * inner == 0) return MXQ_OK;
    if (!x || !out) return MXQ_EINVAL;
    if (out_dtype != x_dtype) return MXQ_ESIZE;
    return strided_quant<MODE_QDQ>(x, x_dtype, nullptr, nullptr, out, outer, D, inner, B, eb, fb, is_finite, rm, (cudaStream_t)stream);
}

extern "C" int mxq_mxfp_compose_strided(const uint8_t* scales, const uint8_t* elements, void* out, int out_dtype, int64_t outer,
                                        int64_t D, int64_t inner, int B, int eb, int fb, int is_finite, void* stream) {
    if (outer < 0 || D < 0 || inner < 0 || B <= 0 || !valid_dtype(out_dtype) || !valid_mx_element(eb, fb, 0)) return MXQ_EINVAL;
    if (outer * D * inner == 0) return MXQ_OK;
    if (!scales || !elements || !out) return MXQ_EINVAL;
    const int cpt = columns_per_thread(out_dtype, out, inner);
    StridedGeom g;
    if (!strided_geometry(outer, D, inner, B, cpt, &g) || reinterpret_cast<uintptr_t>(elements) % 16 != 0) return MXQ_ESIZE;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)(outer * g.tiles_i * g.tiles_j);
    int rc = MXQ_OK;
    bool done = false;
    with_kind(out_dtype, [&](auto kout) {
        using KOut = decltype(kout);
        done = with_preset(eb, fb, is_finite, RM_RN, [&](auto f) {
            using F = decltype(f);
            if constexpr (KOut::size == 4) {
                mxfp_strided_compose_kernel<KOut, F, 1><<<grid, kThreads, 0, st>>>(scales, elements, out, g, f);
            } else {
                if (cpt == 2) mxfp_strided_compose_kernel<KOut, F, 2><<<grid, kThreads, 0, st>>>(scales, elements, out, g, f);
                else mxfp_strided_compose_kernel<KOut, F, 1><<<grid, kThreads, 0, st>>>(scales, elements, out, g, f);
            }
            rc = check_launch();
        });
    });
    return done ? rc : MXQ_ESIZE;
}
