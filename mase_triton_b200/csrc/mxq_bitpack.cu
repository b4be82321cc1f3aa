// Dense bit packing of MXFP element codes for storage: the reference keeps one code per byte
// (`elements`, uint8, src/mase_triton/mxfp/fake.py:57-59) although a code has only
// 1 + exp_bits + frac_bits significant bits.  These kernels pack n codes of `bits` bits (4, 6 or 8)
// into n * bits / 8 bytes, little-endian (code i occupies bits [i * bits, (i + 1) * bits) of the
// stream), and unpack them again: FP4 weights shrink to a half, FP6 weights to three quarters.
// Both directions are bandwidth-bound: one thread moves 16 codes (16 bytes unpacked; 8 / 12 / 16 packed).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mxq.h"
#include "mxq_internal.h"

namespace mxq {

constexpr int kPackThreads = 256;

// 16 codes (one per byte of c[0..4)) -> BITS * 2 bytes
template <int BITS>
__device__ __forceinline__ void pack16(const uint32_t (&c)[4], uint32_t (&o)[4]) {
    if constexpr (BITS == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = c[i];
    } else if constexpr (BITS == 4) {
        // bytes b0..b3 of a word -> nibbles: (b0 | b1 << 4) | (b2 | b3 << 4) << 8
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t h[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint32_t w = c[2 * i + k] & 0x0F0F0F0Fu;
                const uint32_t t = w | (w >> 4);                     // byte 0: b0 | b1 << 4; byte 2: b2 | b3 << 4
                h[k] = (t & 0xFFu) | ((t >> 8) & 0xFF00u);
            }
            o[i] = h[0] | (h[1] << 16);
        }
        o[2] = o[3] = 0u;
    } else {
        // four 6-bit codes -> 24 bits; four such groups -> three words
        uint32_t g[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = c[i] & 0x3F3F3F3Fu;
            g[i] = (w & 0x3Fu) | ((w >> 2) & 0xFC0u) | ((w >> 4) & 0x3F000u) | ((w >> 6) & 0xFC0000u);
        }
        o[0] = g[0] | (g[1] << 24);
        o[1] = (g[1] >> 8) | (g[2] << 16);
        o[2] = (g[2] >> 16) | (g[3] << 8);
        o[3] = 0u;
    }
}

template <int BITS>
__device__ __forceinline__ void unpack16(const uint32_t (&p)[4], uint32_t (&c)[4]) {
    if constexpr (BITS == 8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = p[i];
    } else if constexpr (BITS == 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t h = (p[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;          // four nibbles
            c[i] = (h & 0xFu) | ((h & 0xF0u) << 4) | ((h & 0xF00u) << 8) | ((h & 0xF000u) << 12);
        }
    } else {
        uint32_t g[4];
        g[0] = p[0] & 0xFFFFFFu;
        g[1] = ((p[0] >> 24) | (p[1] << 8)) & 0xFFFFFFu;
        g[2] = ((p[1] >> 16) | (p[2] << 16)) & 0xFFFFFFu;
        g[3] = (p[2] >> 8) & 0xFFFFFFu;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            c[i] = (g[i] & 0x3Fu) | ((g[i] & 0xFC0u) << 2) | ((g[i] & 0x3F000u) << 4) | ((g[i] & 0xFC0000u) << 6);
    }
}

// one thread per 16 codes; n is a multiple of 16
template <int BITS, bool PACK>
__global__ void __launch_bounds__(kPackThreads) bitpack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t n_groups) {
    const int64_t g = (int64_t)blockIdx.x * kPackThreads + threadIdx.x;
    if (g >= n_groups) return;
    constexpr int PB = 2 * BITS;                         // packed bytes per 16 codes
    uint32_t a[4] = {0u, 0u, 0u, 0u}, b[4];
    if constexpr (PACK) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + g * 16);
        a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
        pack16<BITS>(a, b);
        uint32_t* d = reinterpret_cast<uint32_t*>(dst + g * PB);
#pragma unroll
        for (int i = 0; i < PB / 4; ++i) d[i] = b[i];
    } else {
        const uint32_t* s = reinterpret_cast<const uint32_t*>(src + g * PB);
#pragma unroll
        for (int i = 0; i < PB / 4; ++i) a[i] = s[i];
        unpack16<BITS>(a, b);
        *reinterpret_cast<uint4*>(dst + g * 16) = make_uint4(b[0], b[1], b[2], b[3]);
    }
}

template <bool PACK>
static int launch_bitpack(const uint8_t* src, uint8_t* dst, int64_t n, int bits, cudaStream_t st) {
    const int64_t groups = n / 16;
    const unsigned grid = (unsigned)((groups + kPackThreads - 1) / kPackThreads);
    if (bits == 4) bitpack_kernel<4, PACK><<<grid, kPackThreads, 0, st>>>(src, dst, groups);
    else if (bits == 6) bitpack_kernel<6, PACK><<<grid, kPackThreads, 0, st>>>(src, dst, groups);
    else bitpack_kernel<8, PACK><<<grid, kPackThreads, 0, st>>>(src, dst, groups);
    return check_launch();
}

}  // namespace mxq

using namespace mxq;

static bool bitpack_args_ok(const void* a, const void* b, int64_t n, int bits) {
    return a && b && n > 0 && (bits == 4 || bits == 6 || bits == 8) &&
           (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) % 16 == 0;
}

extern "C" int64_t mxq_packed_bytes(int64_t n, int bits) {
    if (n < 0 || n % 16 != 0 || !(bits == 4 || bits == 6 || bits == 8)) return MXQ_EINVAL;
    return n / 16 * 2 * bits;
}

extern "C" int mxq_pack_codes(const uint8_t* codes, uint8_t* packed, int64_t n, int bits, void* stream) {
    if (n == 0) return MXQ_OK;
    if (!bitpack_args_ok(codes, packed, n, bits)) return MXQ_EINVAL;
    if (n % 16 != 0) return MXQ_ESIZE;
    return launch_bitpack<true>(codes, packed, n, bits, (cudaStream_t)stream);
}

extern "C" int mxq_unpack_codes(const uint8_t* packed, uint8_t* codes, int64_t n, int bits, void* stream) {
    if (n == 0) return MXQ_OK;
    if (!bitpack_args_ok(codes, packed, n, bits)) return MXQ_EINVAL;
    if (n % 16 != 0) return MXQ_ESIZE;
    return launch_bitpack<false>(packed, codes, n, bits, (cudaStream_t)stream);
}
