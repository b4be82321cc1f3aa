// Device-side building blocks shared by the bandwidth-bound kernels of libmxq: storage kinds,
// 128-bit packs, the per-block header of the MXFP quantisers and the format dispatch helpers.
#pragma once
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
        // a NaN keeps its sign and payload (quieted), as the x86 conversion does; the GPU's own
        // conversion would return the canonical 0x7FFFFFFF
        if ((raw & 0x7FFFu) > 0x7C00u) return ((raw & 0x8000u) << 16) | 0x7FC00000u | ((raw & 0x3FFu) << 13);
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
// the same with the default cache policy: for data the next kernel reads right away (a GEMM operand), which should
// stay in L2 instead of being marked for early eviction
template <int BYTES>
__device__ __forceinline__ void store_pack_keep(void* p, const Pack<BYTES>& r) {
    if constexpr (BYTES == 16) *reinterpret_cast<uint4*>(p) = make_uint4(r.w[0], r.w[1], r.w[2], r.w[3]);
    else if constexpr (BYTES == 8) *reinterpret_cast<uint2*>(p) = make_uint2(r.w[0], r.w[1]);
    else *reinterpret_cast<unsigned int*>(p) = r.w[0];
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

// Programmatic dependent launch.  A kernel started with launch_overlapped() may become resident while the kernel before
// it in the stream is still draining its last CTAs; it calls grid_dependency_sync() before it touches memory: that
// lets the kernel after it do the same in turn, then waits until the kernels before it have completed and their
// writes are visible.  Launch latency and the ramp of a grid then hide behind the tail of the previous one, which is
// 3 us of an 18 us kernel.  After a kernel launched the plain way the wait returns at once.
__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <class... KArgs, class... Args>
static cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------------------------------------
// helpers shared by the fast kernels
// ------------------------------------------------------------------------------------------------
// Per-block header computed once per block by one lane and handed to the others by shuffle:
//   bits 30..23 : exponent field of 2^-se, so (header & 0x7F800000) IS the fp32 factor 2^-se
//   bits 15..8  : the E8M0 scale byte
//   bit  0      : block holds Inf/NaN (generic path)
template <class F>
__device__ __forceinline__ uint32_t block_header(uint32_t amax_bits, const F& f) {
    uint32_t sbyte;
    const int se = shared_exponent(amax_bits, f, &sbyte);
    const uint32_t special = amax_bits >= 0x7F800000u ? 1u : 0u;
    // an all-flushed block (exponent field 0) encodes to zeros whatever the factor: use 1.0
    const uint32_t inv_field = ((amax_bits >> 23) == 0u || special) ? 127u : (uint32_t)(127 - se);
    return (inv_field << 23) | (sbyte << 8) | special;
}

__device__ __forceinline__ float scale_from_byte(uint32_t s) {
    // 2^(s-127): s = 0 is the fp32 subnormal 2^-127, s = 255 overflows to +Inf
    return __uint_as_float(s == 0u ? 0x00400000u : (s << 23));
}

__device__ __forceinline__ float max_abs_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(fabsf(a)), "f"(fabsf(b)));
    return r;
}

// fp32 bits of max |x| over the V elements of a 16-byte pack; any NaN wins
template <class K>
__device__ __forceinline__ uint32_t pack_absmax_bits(const Pack<16>& p) {
    if constexpr (K::size == 4) {
        const float m = max_abs_nan(max_abs_nan(__uint_as_float(p.w[0]), __uint_as_float(p.w[1])),
                                    max_abs_nan(__uint_as_float(p.w[2]), __uint_as_float(p.w[3])));
        return __float_as_uint(m);
    } else if constexpr (std::is_same<K, KBF16>::value) {
        __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&p.w[0]));
#pragma unroll
        for (int i = 1; i < 4; ++i) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&p.w[i])));
        const uint32_t mw = *reinterpret_cast<uint32_t*>(&m);
        return __float_as_uint(max_abs_nan(__uint_as_float(mw << 16), __uint_as_float(mw & 0xFFFF0000u)));
    } else {
        __half2 m = __habs2(*reinterpret_cast<const __half2*>(&p.w[0]));
#pragma unroll
        for (int i = 1; i < 4; ++i) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __half2*>(&p.w[i])));
        const float2 mf = __half22float2(m);
        return __float_as_uint(max_abs_nan(mf.x, mf.y));
    }
}

// V fp32 results -> V * K::size bytes at dst. `plain` promises that no result is NaN, so the
// packed hardware conversions can be used for 16-bit outputs.
template <class K, int V>
__device__ __forceinline__ void store_results(void* dst, const uint32_t (&y)[V], bool plain) {
    if constexpr (K::size == 4) {
#pragma unroll
        for (int i = 0; i < V; i += 4) {
            Pack<16> o{{y[i], y[i + 1], y[i + 2], y[i + 3]}};
            store_pack<16>(reinterpret_cast<char*>(dst) + 4 * i, o);
        }
    } else {
        Pack<2 * V> o;
        if (plain) {
#pragma unroll
            for (int i = 0; i < V; i += 2) {
                if constexpr (std::is_same<K, KBF16>::value) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(y[i]), __uint_as_float(y[i + 1]));
                    o.w[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                } else {
                    const __half2 h = __floats2half2_rn(__uint_as_float(y[i]), __uint_as_float(y[i + 1]));
                    o.w[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) pack_set<2>(o, i, K::from_bits(y[i]));
        }
        store_pack<2 * V>(dst, o);
    }
}

// four magnitude codes (one per byte) plus the sign bits taken from the top bytes of the quotients
template <class F>
__device__ __forceinline__ uint32_t pack4_codes(const uint32_t* mag, const uint32_t* qb, const F& f) {
    constexpr int sp = F{}.eb() + F{}.fb();                 // sign position inside the code byte
    uint32_t w = (uint32_t)((int)mag[3] * rt_k(4) + ((int)mag[2] * rt_k(3) + ((int)mag[1] * rt_k(2) + (int)mag[0])));
    const uint32_t s01 = __byte_perm(qb[0], qb[1], 0x0073);
    const uint32_t s23 = __byte_perm(qb[2], qb[3], 0x0073);
    const uint32_t sg = __byte_perm(s01, s23, 0x5410);
    if constexpr (sp == 7) w |= sg & 0x80808080u;
    else w |= (sg >> (7 - sp)) & (0x01010101u << sp);
    (void)f;
    return w;
}

// what an MXFP quantiser writes
constexpr int MODE_QDQ = 0;      // dequantised values (fused quantize_dequantize)
constexpr int MODE_CODES = 1;    // reference scales + element codes

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
