// Bandwidth-bound kernels of libmxq for sm_100a: minifloat extract / compose /
// quantize-dequantize and MXFP extract / compose / quantize-dequantize.
//
// Layout in HBM (all row-major, contiguous):
//   x, out      : n floating elements (fp32 / bf16 / fp16)
//   codes       : n uint16 (minifloat)            elements : n uint8 (MXFP, one code per byte)
//   scales      : n / block_size uint8 (E8M0), block j covers elements [j*B, (j+1)*B)
//
// Fast kernels: every lane moves 16 bytes of the wider side per access (128-bit
// loads/stores, a warp covers 512 contiguous bytes), keeps U independent
// accesses in flight, and for MXFP reduces the block maximum of |x| bit patterns
// with warp shuffles over the 4 or 8 lanes that share a 32-element block.
// Generic kernels (any block size, any exp/frac split, any rounding mode, any
// alignment) trade speed for coverage.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "../../include/mxq.h"
#include "mxq_codec.h"
#include "mxq_internal.h"

namespace mxq {

// ------------------------------------------------------------------------------------------------
// storage kinds: how one element is held in memory and how it maps to fp32 bits
// ------------------------------------------------------------------------------------------------
struct KF32 {
    static constexpr int size = 4;
    static __device__ __forceinline__ uint32_t to_bits(uint32_t raw) { return raw; }
    static __device__ __forceinline__ uint32_t from_bits(uint32_t b) { return b; }
};
struct KBF16 {
    static constexpr int size = 2;
    static __device__ __forceinline__ uint32_t to_bits(uint32_t raw) { return raw << 16; }
    static __device__ __forceinline__ uint32_t from_bits(uint32_t b) {
        // NaN narrows to 0xFFFF as x86 PyTorch does; everything else rounds half to even
        if ((b & 0x7FFFFFFFu) > 0x7F800000u) return 0xFFFFu;
        return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(b)));
    }
};
struct KF16 {
    static constexpr int size = 2;
    static __device__ __forceinline__ uint32_t to_bits(uint32_t raw) {
        return __float_as_uint(__half2float(__ushort_as_half((unsigned short)raw)));
    }
    static __device__ __forceinline__ uint32_t from_bits(uint32_t b) {
        if ((b & 0x7FFFFFFFu) > 0x7F800000u)   // keep sign, quiet, keep the top payload bits
            return ((b >> 16) & 0x8000u) | 0x7E00u | ((b >> 13) & 0x1FFu);
        return (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(b)));
    }
};
struct KU16 { static constexpr int size = 2; };
struct KU8 { static constexpr int size = 1; };

// A pack of BYTES bytes moved with one memory instruction.
template <int BYTES> struct Pack { uint32_t w[BYTES / 4]; };

template <int BYTES>
__device__ __forceinline__ Pack<BYTES> load_pack(const void* p) {
    Pack<BYTES> r;
    if constexpr (BYTES == 16) { uint4 v = __ldcs(reinterpret_cast<const uint4*>(p)); r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w; }
    else if constexpr (BYTES == 8) { uint2 v = __ldcs(reinterpret_cast<const uint2*>(p)); r.w[0] = v.x; r.w[1] = v.y; }
    else { r.w[0] = __ldcs(reinterpret_cast<const unsigned int*>(p)); }
    return r;
}
template <int BYTES>
__device__ __forceinline__ void store_pack(void* p, const Pack<BYTES>& r) {
    if constexpr (BYTES == 16) __stcs(reinterpret_cast<uint4*>(p), make_uint4(r.w[0], r.w[1], r.w[2], r.w[3]));
    else if constexpr (BYTES == 8) __stcs(reinterpret_cast<uint2*>(p), make_uint2(r.w[0], r.w[1]));
    else __stcs(reinterpret_cast<unsigned int*>(p), r.w[0]);
}
// raw element i of a pack whose elements are ESZ bytes wide
template <int ESZ, int BYTES>
__device__ __forceinline__ uint32_t pack_get(const Pack<BYTES>& p, int i) {
    if constexpr (ESZ == 4) return p.w[i];
    else if constexpr (ESZ == 2) return (p.w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
    else return (p.w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
}
template <int ESZ, int BYTES>
__device__ __forceinline__ void pack_set(Pack<BYTES>& p, int i, uint32_t v) {
    if constexpr (ESZ == 4) p.w[i] = v;
    else if constexpr (ESZ == 2) { if (i & 1) p.w[i >> 1] |= v << 16; else p.w[i >> 1] = v & 0xFFFFu; }
    else { if (i & 3) p.w[i >> 2] |= (v & 0xFFu) << (8 * (i & 3)); else p.w[i >> 2] = v & 0xFFu; }
}
// fp32 bits of element i of a pack of floating elements of kind K
template <class K, int BYTES>
__device__ __forceinline__ uint32_t pack_bits(const Pack<BYTES>& p, int i) {
    if constexpr (K::size == 4) return p.w[i];
    else if constexpr (std::is_same<K, KBF16>::value) return (i & 1) ? (p.w[i >> 1] & 0xFFFF0000u) : (p.w[i >> 1] << 16);
    else return K::to_bits(pack_get<2>(p, i));
}

template <class K> __device__ __forceinline__ uint32_t load_elem_bits(const void* base, int64_t i) {
    if constexpr (K::size == 4) return reinterpret_cast<const uint32_t*>(base)[i];
    else return K::to_bits(reinterpret_cast<const uint16_t*>(base)[i]);
}
template <class K> __device__ __forceinline__ void store_elem_bits(void* base, int64_t i, uint32_t bits) {
    if constexpr (K::size == 4) reinterpret_cast<uint32_t*>(base)[i] = bits;
    else reinterpret_cast<uint16_t*>(base)[i] = (uint16_t)K::from_bits(bits);
}

constexpr int kThreads = 256;

// ------------------------------------------------------------------------------------------------
// minifloat: vectorised element-wise kernel. Op maps (raw in) -> (raw out).
// ------------------------------------------------------------------------------------------------
template <int IN_SZ, int OUT_SZ, int V, int U, class Op>
__global__ void __launch_bounds__(kThreads) ew_vec_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                          int64_t n_vec, Op op) {
    const int64_t tile = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;
    Pack<V * IN_SZ> p[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t idx = tile + j * kThreads;
        if (idx < n_vec) p[j] = load_pack<V * IN_SZ>(reinterpret_cast<const char*>(in) + idx * (V * IN_SZ));
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t idx = tile + j * kThreads;
        if (idx < n_vec) {
            Pack<V * OUT_SZ> o;
#pragma unroll
            for (int i = 0; i < V; ++i) pack_set<OUT_SZ>(o, i, op(pack_get<IN_SZ>(p[j], i)));
            store_pack<V * OUT_SZ>(reinterpret_cast<char*>(out) + idx * (V * OUT_SZ), o);
        }
    }
}

// scalar version for tails and unaligned buffers
template <int IN_SZ, int OUT_SZ, class Op>
__global__ void __launch_bounds__(kThreads) ew_scalar_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                             int64_t first, int64_t n, Op op) {
    const int64_t i = first + (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    uint32_t raw;
    if constexpr (IN_SZ == 4) raw = reinterpret_cast<const uint32_t*>(in)[i];
    else raw = reinterpret_cast<const uint16_t*>(in)[i];
    const uint32_t r = op(raw);
    if constexpr (OUT_SZ == 4) reinterpret_cast<uint32_t*>(out)[i] = r;
    else reinterpret_cast<uint16_t*>(out)[i] = (uint16_t)r;
}

template <class KIn, class F, bool FAST> struct ExtractOp {
    F f;
    __device__ __forceinline__ uint32_t operator()(uint32_t raw) const {
        const uint32_t u = KIn::to_bits(raw);
        if constexpr (FAST) return encode_f32_fast(u, f); else return encode_f32(u, f);
    }
};
template <class KOut, class F, bool FAST> struct ComposeOp {
    F f;
    __device__ __forceinline__ uint32_t operator()(uint32_t raw) const {
        if constexpr (FAST) return KOut::from_bits(decode_f32_fast(raw, f)); else return KOut::from_bits(decode_f32(raw, f));
    }
};
template <class KIn, class KOut, class F, bool FAST> struct QdqOp {
    F f;
    __device__ __forceinline__ uint32_t operator()(uint32_t raw) const {
        const uint32_t u = KIn::to_bits(raw);
        if constexpr (FAST) return KOut::from_bits(decode_f32_fast(encode_f32_fast(u, f), f));
        else return KOut::from_bits(decode_f32(encode_f32(u, f), f));
    }
};

template <int IN_SZ, int OUT_SZ, class Op>
static int launch_ew(const void* in, void* out, int64_t n, Op op, cudaStream_t st) {
    constexpr int WIDE = IN_SZ > OUT_SZ ? IN_SZ : OUT_SZ;
    constexpr int V = 16 / WIDE;
    constexpr int U = 4;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) % (V * IN_SZ)) == 0) && ((reinterpret_cast<uintptr_t>(out) % (V * OUT_SZ)) == 0);
    const int64_t n_vec = aligned ? n / V : 0;
    if (n_vec > 0) {
        const int64_t grid = (n_vec + kThreads * U - 1) / (kThreads * U);
        ew_vec_kernel<IN_SZ, OUT_SZ, V, U, Op><<<(unsigned)grid, kThreads, 0, st>>>(in, out, n_vec, op);
    }
    const int64_t first = n_vec * V;
    if (first < n) {
        const int64_t grid = (n - first + kThreads - 1) / kThreads;
        ew_scalar_kernel<IN_SZ, OUT_SZ, Op><<<(unsigned)grid, kThreads, 0, st>>>(in, out, first, n, op);
    }
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// MXFP, block size 32: fast kernels
// ------------------------------------------------------------------------------------------------
// Per-block header computed once per block by one lane and handed to the others by shuffle:
//   bits 31..23 : (se + 127 - bias), the exponent rebase of the element encoder
//   bit  0      : block holds Inf/NaN (generic path)
//   bits 15..8  : the E8M0 scale byte
template <class F>
__device__ __forceinline__ uint32_t block_header(uint32_t amax_bits, const F& f) {
    uint32_t sbyte;
    const int se = shared_exponent(amax_bits, f, &sbyte);
    const uint32_t special = amax_bits >= 0x7F800000u ? 1u : 0u;
    return ((uint32_t)(se + 127 - fmt_bias(f)) << 23) | (sbyte << 8) | special;
}

__device__ __forceinline__ float scale_from_byte(uint32_t s) {
    // 2^(s-127): s = 0 is the fp32 subnormal 2^-127, s = 255 overflows to +Inf
    return __uint_as_float(s == 0u ? 0x00400000u : (s << 23));
}

template <class KIn, class KOut, class F, int U, bool WRITE_CODES>
__global__ void __launch_bounds__(kThreads) mxfp_b32_quant_kernel(const void* __restrict__ x, uint8_t* __restrict__ scales,
                                                                  uint8_t* __restrict__ elements, void* __restrict__ out,
                                                                  int64_t n_vec, F f) {
    constexpr int V = 16 / KIn::size;     // elements per lane per access: 4 (fp32) or 8 (16-bit)
    constexpr int G = 32 / V;             // lanes that share one 32-element block: 8 or 4
    static_assert(U <= G, "one lane of the group per in-flight access");
    const int lane = threadIdx.x & 31;
    const int sub = lane & (G - 1);
    const int64_t tile = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;

    Pack<16> p[U];
    uint32_t amax[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t idx = tile + j * kThreads;
        if (idx < n_vec) p[j] = load_pack<16>(reinterpret_cast<const char*>(x) + idx * 16);
        else p[j] = Pack<16>{{0u, 0u, 0u, 0u}};
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        uint32_t m = 0;
#pragma unroll
        for (int i = 0; i < V; ++i) m = max(m, pack_bits<KIn>(p[j], i) & 0x7FFFFFFFu);
#pragma unroll
        for (int o = 1; o < G; o <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        amax[j] = m;
    }
    // lane `sub` of each group derives the header of access `sub`
    uint32_t mine = amax[0];
#pragma unroll
    for (int j = 1; j < U; ++j) mine = (sub == j) ? amax[j] : mine;
    const uint32_t hdr = block_header(mine, f);
    if (WRITE_CODES && sub < U) {
        const int64_t idx = tile + sub * kThreads;
        if (idx < n_vec) scales[idx / G] = (uint8_t)(hdr >> 8);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const uint32_t h = __shfl_sync(0xFFFFFFFFu, hdr, (lane & ~(G - 1)) + j);
        const int64_t idx = tile + j * kThreads;
        if (idx >= n_vec) continue;
        uint32_t code[V];
        if (!(h & 1u)) {
            const int rebase = (int)(h & 0xFF800000u);
#pragma unroll
            for (int i = 0; i < V; ++i) code[i] = mx_encode_fast(pack_bits<KIn>(p[j], i), rebase, f);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) code[i] = mx_encode(pack_bits<KIn>(p[j], i), 128, f);
        }
        if constexpr (WRITE_CODES) {
            Pack<V> o;
#pragma unroll
            for (int i = 0; i < V; ++i) pack_set<1>(o, i, code[i]);
            store_pack<V>(elements + idx * V, o);
        } else {
            const uint32_t sb = (h >> 8) & 0xFFu;
            const float sf = scale_from_byte(sb);
            constexpr int OB = V * KOut::size;      // 16 or 32 bytes per lane
            Pack<(OB > 16 ? 16 : OB)> o[OB > 16 ? 2 : 1];
#pragma unroll
            for (int i = 0; i < V; ++i) {
                uint32_t y;
                if (sb != 255u) y = __float_as_uint(__fmul_rn(__uint_as_float(decode_f32_fast(code[i], f)), sf));
                else y = mx_decode(code[i], sf, f);
                constexpr int per = (OB > 16 ? 16 : OB) / KOut::size;
                pack_set<KOut::size>(o[i / per], i % per, KOut::from_bits(y));
            }
            char* dst = reinterpret_cast<char*>(out) + idx * OB;
            store_pack<(OB > 16 ? 16 : OB)>(dst, o[0]);
            if constexpr (OB > 16) store_pack<16>(dst + 16, o[1]);
        }
    }
}

template <class KOut, class F, int U>
__global__ void __launch_bounds__(kThreads) mxfp_b32_compose_kernel(const uint8_t* __restrict__ scales,
                                                                    const uint8_t* __restrict__ elements,
                                                                    void* __restrict__ out, int64_t n_vec, F f) {
    constexpr int V = 16 / KOut::size;    // 4 or 8 elements per lane per access
    constexpr int G = 32 / V;
    const int64_t tile = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;
    Pack<V> c[U];
    uint32_t sb[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t idx = tile + j * kThreads;
        if (idx < n_vec) {
            c[j] = load_pack<V>(elements + idx * V);
            sb[j] = __ldg(scales + idx / G);
        }
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t idx = tile + j * kThreads;
        if (idx >= n_vec) continue;
        const float sf = scale_from_byte(sb[j]);
        Pack<16> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const uint32_t code = pack_get<1>(c[j], i);
            uint32_t y;
            if (sb[j] != 255u) y = __float_as_uint(__fmul_rn(__uint_as_float(decode_f32_fast(code, f)), sf));
            else y = mx_decode(code, sf, f);
            pack_set<KOut::size>(o, i, KOut::from_bits(y));
        }
        store_pack<16>(reinterpret_cast<char*>(out) + idx * 16, o);
    }
}

// ------------------------------------------------------------------------------------------------
// MXFP, generic: any block size / format / rounding mode / alignment. One thread per block.
// ------------------------------------------------------------------------------------------------
template <class KIn, class KOut, bool WRITE_CODES>
__global__ void __launch_bounds__(kThreads) mxfp_generic_quant_kernel(const void* __restrict__ x, uint8_t* __restrict__ scales,
                                                                      uint8_t* __restrict__ elements, void* __restrict__ out,
                                                                      int64_t n_blocks, int B, FmtRT f) {
    const int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (b >= n_blocks) return;
    const int64_t base = b * B;
    uint32_t amax = 0;
    for (int j = 0; j < B; ++j) amax = max(amax, load_elem_bits<KIn>(x, base + j) & 0x7FFFFFFFu);
    uint32_t sbyte;
    const int se = shared_exponent(amax, f, &sbyte);
    if constexpr (WRITE_CODES) scales[b] = (uint8_t)sbyte;
    const float sf = scale_from_byte(sbyte);
    for (int j = 0; j < B; ++j) {
        const uint32_t code = mx_encode(load_elem_bits<KIn>(x, base + j), se, f);
        if constexpr (WRITE_CODES) elements[base + j] = (uint8_t)code;
        else store_elem_bits<KOut>(out, base + j, mx_decode(code, sf, f));
    }
}

template <class KOut>
__global__ void __launch_bounds__(kThreads) mxfp_generic_compose_kernel(const uint8_t* __restrict__ scales,
                                                                        const uint8_t* __restrict__ elements,
                                                                        void* __restrict__ out, int64_t n, int B, FmtRT f) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    const float sf = scale_from_byte(scales[i / B]);
    store_elem_bits<KOut>(out, i, mx_decode(elements[i], sf, f));
}

// ------------------------------------------------------------------------------------------------
// host-side dispatch
// ------------------------------------------------------------------------------------------------
static bool valid_dtype(int dt) { return dt == MXQ_F32 || dt == MXQ_BF16 || dt == MXQ_F16; }
static bool valid_minifloat(int eb, int fb, int rm) { return eb > 0 && fb > 0 && eb + fb < 16 && rm >= 0 && rm <= 3; }
static bool valid_mx_element(int eb, int fb, int rm) { return eb > 0 && fb > 0 && eb + fb <= 7 && rm >= 0 && rm <= 3; }

// calls fn(FmtCT<..>{}) when (eb, fb, fin, rm) is one of the built-in round-to-nearest presets
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
template <class Fn>
static void with_kind(int dt, Fn&& fn) {
    if (dt == MXQ_F32) fn(KF32{}); else if (dt == MXQ_BF16) fn(KBF16{}); else fn(KF16{});
}

}  // namespace mxq

using namespace mxq;

extern "C" int mxq_minifloat_extract(const void* x, int x_dtype, uint16_t* codes, int64_t n, int eb, int fb,
                                     int is_finite, int rm, void* stream) {
    if (n < 0 || !valid_dtype(x_dtype) || !valid_minifloat(eb, fb, rm)) return MXQ_EINVAL;
    if (n == 0) return MXQ_OK;
    if (!x || !codes) return MXQ_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MXQ_OK;
    with_kind(x_dtype, [&](auto kin) {
        using KIn = decltype(kin);
        const bool fast = with_preset(eb, fb, is_finite, rm, [&](auto f) {
            rc = launch_ew<KIn::size, 2>(x, codes, n, ExtractOp<KIn, decltype(f), true>{f}, st);
        });
        if (!fast) rc = launch_ew<KIn::size, 2>(x, codes, n, ExtractOp<KIn, FmtRT, false>{FmtRT{eb, fb, is_finite, rm}}, st);
    });
    return rc;
}

extern "C" int mxq_minifloat_compose(const uint16_t* codes, void* out, int out_dtype, int64_t n, int eb, int fb,
                                     int is_finite, void* stream) {
    if (n < 0 || !valid_dtype(out_dtype) || !valid_minifloat(eb, fb, 0)) return MXQ_EINVAL;
    if (n == 0) return MXQ_OK;
    if (!codes || !out) return MXQ_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MXQ_OK;
    with_kind(out_dtype, [&](auto kout) {
        using KOut = decltype(kout);
        const bool fast = with_preset(eb, fb, is_finite, RM_RN, [&](auto f) {
            rc = launch_ew<2, KOut::size>(codes, out, n, ComposeOp<KOut, decltype(f), true>{f}, st);
        });
        if (!fast) rc = launch_ew<2, KOut::size>(codes, out, n, ComposeOp<KOut, FmtRT, false>{FmtRT{eb, fb, is_finite, 0}}, st);
    });
    return rc;
}

extern "C" int mxq_minifloat_qdq(const void* x, int x_dtype, void* out, int out_dtype, int64_t n, int eb, int fb,
                                 int is_finite, int rm, void* stream) {
    if (n < 0 || !valid_dtype(x_dtype) || !valid_dtype(out_dtype) || !valid_minifloat(eb, fb, rm)) return MXQ_EINVAL;
    if (n == 0) return MXQ_OK;
    if (!x || !out) return MXQ_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MXQ_OK;
    with_kind(x_dtype, [&](auto kin) {
        using KIn = decltype(kin);
        with_kind(out_dtype, [&](auto kout) {
            using KOut = decltype(kout);
            const bool fast = with_preset(eb, fb, is_finite, rm, [&](auto f) {
                rc = launch_ew<KIn::size, KOut::size>(x, out, n, QdqOp<KIn, KOut, decltype(f), true>{f}, st);
            });
            if (!fast)
                rc = launch_ew<KIn::size, KOut::size>(x, out, n, QdqOp<KIn, KOut, FmtRT, false>{FmtRT{eb, fb, is_finite, rm}}, st);
        });
    });
    return rc;
}

namespace mxq {
template <bool WRITE_CODES>
static int mxfp_quant_dispatch(const void* x, int x_dtype, uint8_t* scales, uint8_t* elements, void* out, int out_dtype,
                               int64_t n, int B, int eb, int fb, int fin, int rm, cudaStream_t st) {
    int rc = MXQ_OK;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                         (WRITE_CODES ? (reinterpret_cast<uintptr_t>(elements) % 16 == 0) : (reinterpret_cast<uintptr_t>(out) % 16 == 0));
    bool done = false;
    if (B == 32 && aligned) {
        with_kind(x_dtype, [&](auto kin) {
            using KIn = decltype(kin);
            auto go = [&](auto kout) {
                using KOut = decltype(kout);
                done = with_preset(eb, fb, fin, rm, [&](auto f) {
                    constexpr int V = 16 / KIn::size;
                    constexpr int U = 4;
                    const int64_t n_vec = n / V;
                    const int64_t grid = (n_vec + kThreads * U - 1) / (kThreads * U);
                    mxfp_b32_quant_kernel<KIn, KOut, decltype(f), U, WRITE_CODES><<<(unsigned)grid, kThreads, 0, st>>>(
                        x, scales, elements, out, n_vec, f);
                    rc = check_launch();
                });
            };
            if constexpr (WRITE_CODES) go(KF32{});
            else if (out_dtype == x_dtype) go(kin);   // fused fast path: same dtype in and out
        });
    }
    if (!done) {
        const int64_t nb = n / B;
        const int64_t grid = (nb + kThreads - 1) / kThreads;
        FmtRT f{eb, fb, fin, rm};
        with_kind(x_dtype, [&](auto kin) {
            using KIn = decltype(kin);
            if constexpr (WRITE_CODES) {
                mxfp_generic_quant_kernel<KIn, KF32, true><<<(unsigned)grid, kThreads, 0, st>>>(x, scales, elements, out, nb, B, f);
            } else {
                with_kind(out_dtype, [&](auto kout) {
                    mxfp_generic_quant_kernel<KIn, decltype(kout), false><<<(unsigned)grid, kThreads, 0, st>>>(x, scales, elements, out, nb, B, f);
                });
            }
        });
        rc = check_launch();
    }
    return rc;
}
}  // namespace mxq

extern "C" int mxq_mxfp_extract(const void* x, int x_dtype, uint8_t* scales, uint8_t* elements, int64_t n, int B,
                                int eb, int fb, int is_finite, int rm, void* stream) {
    if (n < 0 || B <= 0 || n % B != 0 || !valid_dtype(x_dtype) || !valid_mx_element(eb, fb, rm)) return MXQ_EINVAL;
    if (n == 0) return MXQ_OK;
    if (!x || !scales || !elements) return MXQ_EINVAL;
    return mxfp_quant_dispatch<true>(x, x_dtype, scales, elements, nullptr, MXQ_F32, n, B, eb, fb, is_finite, rm, (cudaStream_t)stream);
}

extern "C" int mxq_mxfp_qdq(const void* x, int x_dtype, void* out, int out_dtype, int64_t n, int B, int eb, int fb,
                            int is_finite, int rm, void* stream) {
    if (n < 0 || B <= 0 || n % B != 0 || !valid_dtype(x_dtype) || !valid_dtype(out_dtype) || !valid_mx_element(eb, fb, rm)) return MXQ_EINVAL;
    if (n == 0) return MXQ_OK;
    if (!x || !out) return MXQ_EINVAL;
    return mxfp_quant_dispatch<false>(x, x_dtype, nullptr, nullptr, out, out_dtype, n, B, eb, fb, is_finite, rm, (cudaStream_t)stream);
}

extern "C" int mxq_mxfp_compose(const uint8_t* scales, const uint8_t* elements, void* out, int out_dtype, int64_t n,
                                int B, int eb, int fb, int is_finite, void* stream) {
    if (n < 0 || B <= 0 || n % B != 0 || !valid_dtype(out_dtype) || !valid_mx_element(eb, fb, 0)) return MXQ_EINVAL;
    if (n == 0) return MXQ_OK;
    if (!scales || !elements || !out) return MXQ_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MXQ_OK;
    bool done = false;
    const bool aligned = (reinterpret_cast<uintptr_t>(elements) % 8 == 0) && (reinterpret_cast<uintptr_t>(out) % 16 == 0);
    with_kind(out_dtype, [&](auto kout) {
        using KOut = decltype(kout);
        if (B == 32 && aligned) {
            done = with_preset(eb, fb, is_finite, RM_RN, [&](auto f) {
                constexpr int V = 16 / KOut::size;
                constexpr int U = 4;
                const int64_t n_vec = n / V;
                const int64_t grid = (n_vec + kThreads * U - 1) / (kThreads * U);
                mxfp_b32_compose_kernel<KOut, decltype(f), U><<<(unsigned)grid, kThreads, 0, st>>>(scales, elements, out, n_vec, f);
                rc = check_launch();
            });
        }
        if (!done) {
            const int64_t grid = (n + kThreads - 1) / kThreads;
            mxfp_generic_compose_kernel<KOut><<<(unsigned)grid, kThreads, 0, st>>>(scales, elements, out, n, B, FmtRT{eb, fb, is_finite, 0});
            rc = check_launch();
        }
    });
    return rc;
}
