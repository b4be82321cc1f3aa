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
#include "mxq_device.cuh"

namespace mxq {

// ------------------------------------------------------------------------------------------------
// minifloat: vectorised element-wise kernel.
//   KIn / KOut : storage kinds (KF32 / KBF16 / KF16 floating, KU16 codes)
//   Op         : maps the fp32 bits of a floating input (or the raw code of a KU16 input) to the
//                fp32 bits of a floating output (or the raw code of a KU16 output)
//   PLAIN      : the op never yields NaN, so 16-bit outputs may use the packed conversions
// ------------------------------------------------------------------------------------------------
template <class K, int BYTES>
__device__ __forceinline__ uint32_t pack_elem(const Pack<BYTES>& p, int i) {
    if constexpr (std::is_same<K, KU16>::value) return pack_get<2>(p, i);
    else return pack_bits<K>(p, i);
}

template <class KIn, class KOut, int V, int U, bool PLAIN, bool FULL, class Op>
__device__ __forceinline__ void ew_tile(const char* __restrict__ src, char* __restrict__ dst, int64_t left, const Op& op) {
    // src / dst already point at this thread's first vector; `left` = vectors from there to the end
    constexpr int IB = V * KIn::size, OB = V * KOut::size;
    Pack<IB> p[U];
#pragma unroll
    for (int j = 0; j < U; ++j)
        if (FULL || j * kThreads < left) p[j] = load_pack<IB>(src + (size_t)j * kThreads * IB);
#pragma unroll
    for (int j = 0; j < U; ++j) {
        if (!FULL && j * kThreads >= left) continue;
        uint32_t y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) y[i] = op(pack_elem<KIn>(p[j], i));
        char* d = dst + (size_t)j * kThreads * OB;
        if constexpr (std::is_same<KOut, KU16>::value) {
            Pack<OB> o;
#pragma unroll
            for (int i = 0; i < V; ++i) pack_set<2>(o, i, y[i]);
            store_pack<OB>(d, o);
        } else {
            store_results<KOut, V>(d, y, PLAIN);
        }
    }
}

template <class KIn, class KOut, int V, int U, bool PLAIN, class Op>
__global__ void __launch_bounds__(kThreads) ew_vec_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                          int64_t n_vec, Op op) {
    grid_dependency_sync();
    const int64_t first = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;
    const char* src = reinterpret_cast<const char*>(in) + first * (V * KIn::size);
    char* dst = reinterpret_cast<char*>(out) + first * (V * KOut::size);
    if ((int64_t)(blockIdx.x + 1) * (kThreads * U) <= n_vec) ew_tile<KIn, KOut, V, U, PLAIN, true>(src, dst, 0, op);
    else ew_tile<KIn, KOut, V, U, PLAIN, false>(src, dst, n_vec - first, op);
}

// scalar version for tails and unaligned buffers
template <class KIn, class KOut, class Op>
__global__ void __launch_bounds__(kThreads) ew_scalar_kernel(const void* __restrict__ in, void* __restrict__ out,
                                                             int64_t first, int64_t n, Op op) {
    const int64_t i = first + (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    uint32_t v;
    if constexpr (std::is_same<KIn, KU16>::value) v = reinterpret_cast<const uint16_t*>(in)[i];
    else v = load_elem_bits<KIn>(in, i);
    const uint32_t r = op(v);
    if constexpr (std::is_same<KOut, KU16>::value) reinterpret_cast<uint16_t*>(out)[i] = (uint16_t)r;
    else store_elem_bits<KOut>(out, i, r);
}

template <class F, bool FAST> struct ExtractOp {
    F f;
    __device__ __forceinline__ uint32_t operator()(uint32_t u) const {
        if constexpr (FAST) return encode_f32_fast(u, f); else return encode_f32(u, f);
    }
};
template <class F, bool FAST> struct ComposeOp {
    F f;
    __device__ __forceinline__ uint32_t operator()(uint32_t code) const {
        if constexpr (FAST) return decode_f32_fast(code, f); else return decode_f32(code, f);
    }
};
template <class F, bool FAST> struct QdqOp {
    F f;
    __device__ __forceinline__ uint32_t operator()(uint32_t u) const {
        if constexpr (FAST) return qdq_f32_fast(u, f);
        else return decode_f32(encode_f32(u, f), f);
    }
};

template <class KIn, class KOut, bool PLAIN, class Op>
static int launch_ew(const void* in, void* out, int64_t n, Op op, cudaStream_t st) {
    constexpr int WIDE = KIn::size > KOut::size ? KIn::size : KOut::size;
    constexpr int V = 16 / WIDE;
    constexpr int U = 4;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) % (V * KIn::size)) == 0) && ((reinterpret_cast<uintptr_t>(out) % (V * KOut::size)) == 0);
    const int64_t n_vec = aligned ? n / V : 0;
    if (n_vec > 0) {
        const int64_t grid = (n_vec + kThreads * U - 1) / (kThreads * U);
        const cudaError_t e = launch_overlapped(ew_vec_kernel<KIn, KOut, V, U, PLAIN, Op>, (unsigned)grid, kThreads, st, in, out, n_vec, op);
        if (e != cudaSuccess) { set_last_cuda_error(e); return MXQ_ELAUNCH; }
    }
    const int64_t first = n_vec * V;
    if (first < n) {
        const int64_t grid = (n - first + kThreads - 1) / kThreads;
        ew_scalar_kernel<KIn, KOut, Op><<<(unsigned)grid, kThreads, 0, st>>>(in, out, first, n, op);
    }
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// MXFP, block size 32: fast kernels
// ------------------------------------------------------------------------------------------------


// Geometry of the scale-factor chunks of a [rows, K] left operand (see mxq_gemm.cu): the block index is
// split into (row, K block) with a multiply-shift division by K/32.
struct PackGeom {
    uint32_t kbpr;     // K / 32
    uint32_t magic;    // ceil(2^(31+shift) / kbpr)
    uint32_t shift;
    uint32_t KT;       // ceil(K / 128)
};

__device__ __forceinline__ uint32_t sf_chunk_offset(uint32_t blk, const PackGeom& g) {
    const uint32_t r = (uint32_t)(((uint64_t)blk * g.magic) >> (31 + g.shift));     // blk / kbpr for blk < 2^31
    const uint32_t kb = blk - r * g.kbpr;
    const uint32_t lr = r & 255u, rr = lr & 127u;
    return (((r >> 8) * g.KT + (kb >> 2)) * 2u + (lr >> 7)) * 512u + (rr & 31u) * 16u + (rr >> 5) * 4u + (kb & 3u);
}

// ------------------------------------------------------------------------------------------------
// MXFP4 (E2M1) elements of bf16 inputs, two elements per 32-bit word on the packed bf16 units.
// The quotient q = |x| * 2^-se is exact in bf16 for a power-of-two factor (below 2^-126 it only has
// to stay below 0.625), and q < 8 for a finite block.  Per word:
//   * q >= 1: the 7-bit mantissa, tagged with exponent 0, plus 63.0 is 64 + (m - 1) rounded half to
//     even to a multiple of 0.5, so the sum's bits are those of 64.0 plus fr in {0, 1, 2}; fr << 6
//     OR-ed under q's own exponent field is the quantised quotient in bf16 (fr = 2 lands on the
//     exponent's low bit: the reference's OR-merge, minifloat/fake.py:70, carry lost for odd fields);
//     the code is that pattern shifted down, re-biased with one XOR;
//   * q < 1: the single subnormal binade (:56-60) leaves code 1 (0.5) above 0.625 and zero below.
// An element is kept (else it is +0) when it is not a flushed input and its fp32 quotient does not
// round to zero: |x| > max(2^(se-150), largest subnormal), one packed comparison against a
// per-block constant; the sign bit rides along with the kept ones.
// This is ~8 integer-pipe instructions per element instead of ~13 for the generic codec.
// ------------------------------------------------------------------------------------------------
struct E2M1Block {
    uint32_t inv2;    // 2^-se in both halves
    uint32_t sf2;     // 2^se in both halves (fused form)
    uint32_t ts2;     // keep threshold in both halves
};

__device__ __forceinline__ E2M1Block e2m1_block(uint32_t h) {
    E2M1Block b;
    const uint32_t sb = (h >> 8) & 0xFFu;
    b.inv2 = ((h >> 16) & 0x7F80u) * 0x10001u;
    b.sf2 = (sb == 0u ? 0x0040u : (sb << 7)) * 0x10001u;
    b.ts2 = (uint32_t)max(((int)sb - 150) * 128, 0x7F) * 0x10001u;
    return b;
}

__device__ __forceinline__ __nv_bfloat162 bf2(uint32_t w) { return *reinterpret_cast<__nv_bfloat162*>(&w); }
__device__ __forceinline__ uint32_t bf2_bits(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// one 16-byte access of a lane (8 bf16 inputs) of a finite block -> 8 code bytes or 8 bf16 results
template <bool VALUES>
__device__ __forceinline__ void e2m1_bf16_quantise(const Pack<16>& p, const E2M1Block& b, uint32_t* out) {
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = p.w[i];
        const uint32_t aw = w & 0x7FFF7FFFu;
        const __nv_bfloat162 q = __hmul2(bf2(aw), bf2(b.inv2));
        const uint32_t qb = bf2_bits(q);
        const uint32_t keep = __hgt2_mask(bf2(aw), bf2(b.ts2));
        // normal range: rounded mantissa field under q's exponent field
        const uint32_t sum = bf2_bits(__hadd2(bf2((qb & 0x007F007Fu) | 0x3F803F80u), bf2(0x427C427Cu)));      // + 63.0
        const uint32_t z = sum * (uint32_t)rt_k(9) - 0x42804280u * 64u;        // (sum - bits(64.0)) << 6 per half, as one multiply-add
        const uint32_t y = (qb & 0x7F807F80u) | z;
        const uint32_t lt1 = __hlt2_mask(q, bf2(0x3F803F80u));                  // q < 1
        const uint32_t gt = __hgt2_mask(q, bf2(0x3F203F20u));                   // q > 0.625
        if constexpr (VALUES) {
            const uint32_t v = (lt1 & gt & 0x3F003F00u) | (~lt1 & y);            // 0.5 / 0 below 1, else the quantised quotient
            const uint32_t o = bf2_bits(__hmul2(bf2(v), bf2(b.sf2)));
            r[i] = ((o & 0x7FFF7FFFu) | (w & 0x80008000u)) & keep;
        } else {
            const uint32_t cn = ((y >> 6) ^ 0x00040004u) & 0x00070007u;          // (E << 1 | fr) - 252, modulo 8
            const uint32_t c = (lt1 & gt & 0x00010001u) | (~lt1 & cn);
            r[i] = (c | ((w >> 12) & 0x00080008u)) & keep;
        }
    }
    if constexpr (VALUES) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = r[i];
    } else {
        out[0] = __byte_perm(r[0], r[1], 0x6420);
        out[1] = __byte_perm(r[2], r[3], 0x6420);
    }
}

// ------------------------------------------------------------------------------------------------
// The same idea for the other element formats (E4M3, E5M2, E2M3, E3M2) of bf16 inputs: two elements
// per 32-bit word on the packed bf16 units.  For a quotient q = |x| * 2^-se (exact in bf16):
//   * normal range (biased exponent >= 1): the 7-bit mantissa, tagged with exponent 0, plus 2^(7-fb)
//     rounds half to even to fb fraction bits, so the sum's low bits are 2^fb + fr with fr in
//     [0, 2^fb]; the code is q's exponent field, re-biased by flipping its bit eb-1 (127 - bias is
//     2^(eb-1) modulo 2^eb), with fr OR-ed in -- fr = 2^fb lands on the exponent's low bit, which is the
//     reference's OR-merge with its lost carry (minifloat/fake.py:70-75); the dequantised value is fr
//     OR-ed under q's own exponent field;
//   * below 2^(1-bias): the single subnormal binade (fake.py:56-60) encodes as (fr | 2^fb) >> 1 unless
//     fr is zero, anything below 2^-bias as zero.  For the 8-bit formats such elements are rare and the lanes of a
//     warp skip this part together when none of them has one;
//   * an element is kept (else it is +0) when it is not a flushed input and its fp32 quotient does not
//     round to zero: one packed comparison against a per-block threshold; the sign rides along.
// A bf16 input has 7 mantissa bits, so the reference's cut to 15 bits (fake.py:45) changes nothing.
// ------------------------------------------------------------------------------------------------
template <class F> struct PkFmt {
    static constexpr int EB = F{}.eb(), FB = F{}.fb();
    static constexpr int BIAS = (1 << (EB - 1)) - 1;
    static constexpr uint32_t rep(uint32_t half) { return half * 0x10001u; }
    static constexpr uint32_t ROUND_C = rep((uint32_t)(127 + 7 - FB) << 7);                      // 2^(7-fb)
    static constexpr uint32_t SUM_BASE = rep(((uint32_t)(127 + 7 - FB) << 7) + (1u << FB));      // bits of 2^(7-fb) with mantissa field 2^fb
    static constexpr uint32_t EXP_FLIP = rep((1u << (EB - 1)) << FB);
    static constexpr uint32_t MAG_MASK = rep((1u << (EB + FB)) - 1u);
    static constexpr uint32_t EXP_MASK = rep(((1u << EB) - 1u) << FB);
    static constexpr uint32_t FR_ONE = rep(1u << FB);
    static constexpr uint32_t SUB_MASK = rep((2u << FB) - 1u);
    static constexpr uint32_t SIGN_BIT = rep(1u << (EB + FB));
    static constexpr uint32_t NORMAL_MIN = rep((uint32_t)(128 - BIAS) << 7);                     // 2^(1-bias)
    static constexpr uint32_t BINADE_MIN = rep((uint32_t)(127 - BIAS) << 7);                     // 2^-bias
    static constexpr uint32_t REBIAS = rep((uint32_t)(254 - BIAS) << 7);                         // 2^(127-bias)
    static constexpr bool RARE_SUBRANGE = EB >= 4;       // block maximum >= 2^(emax-bias): elements 2^14 (E4M3) / 2^29 (E5M2) below it
};

// one 16-byte access of a lane (8 bf16 inputs) of a finite block.
// VALUES: 8 bf16 results in out[0..4); else 8 magnitude+sign code bytes in out[0..2)
template <class F, bool VALUES>
__device__ __forceinline__ void pk_bf16_quantise(const Pack<16>& p, const E2M1Block& b, uint32_t* out) {
    using P = PkFmt<F>;
    uint32_t qb[4], fr[4], res[4];
    uint32_t any_sub = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t aw = p.w[i] & 0x7FFF7FFFu;
        qb[i] = bf2_bits(__hmul2(bf2(aw), bf2(b.inv2)));
        const uint32_t sum = bf2_bits(__hadd2(bf2((qb[i] & 0x007F007Fu) | 0x3F803F80u), bf2(P::ROUND_C)));
        fr[i] = sum - P::SUM_BASE;                                           // 0 .. 2^fb in each half
        if constexpr (VALUES) res[i] = (qb[i] & 0x7F807F80u) | (fr[i] << (7 - P::FB));
        else res[i] = (((qb[i] >> (7 - P::FB)) ^ P::EXP_FLIP) & P::EXP_MASK) | fr[i];
        any_sub |= __hlt2_mask(bf2(qb[i]), bf2(P::NORMAL_MIN));
    }
    if (!P::RARE_SUBRANGE || __any_sync(__activemask(), any_sub != 0u)) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lt = __hlt2_mask(bf2(qb[i]), bf2(P::NORMAL_MIN));
            const uint32_t ge = __hge2_mask(bf2(qb[i]), bf2(P::BINADE_MIN));
            // (fr | 2^fb) >> 1 when the rounded mantissa field is not zero (fake.py:58), zero otherwise and below the binade
            const uint32_t nz = (((fr[i] + 0x7FFF7FFFu) >> 15) & 0x00010001u) * 0xFFFFu;
            const uint32_t sub = ((fr[i] | P::FR_ONE) >> 1) & P::SUB_MASK & ge & nz;
            if constexpr (VALUES) {
                // sub * 2^(1-bias-fb): the field placed at the top of a bf16 mantissa is sub * 2^(-fb-126)
                const uint32_t v = bf2_bits(__hmul2(bf2(sub << (7 - P::FB)), bf2(P::REBIAS)));
                res[i] = (lt & v) | (~lt & res[i]);
            } else {
                res[i] = (lt & sub) | (~lt & res[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = p.w[i];
        const uint32_t keep = __hgt2_mask(bf2(w & 0x7FFF7FFFu), bf2(b.ts2));
        if constexpr (VALUES) {
            const uint32_t o = bf2_bits(__hmul2(bf2(res[i]), bf2(b.sf2)));
            res[i] = ((o & 0x7FFF7FFFu) | (w & 0x80008000u)) & keep;
        } else {
            res[i] = (res[i] | ((w >> (15 - P::EB - P::FB)) & P::SIGN_BIT)) & keep;
        }
    }
    if constexpr (VALUES) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = res[i];
    } else {
        out[0] = __byte_perm(res[0], res[1], 0x6420);
        out[1] = __byte_perm(res[2], res[3], 0x6420);
    }
}

// ------------------------------------------------------------------------------------------------
// bf16 inputs: what the lanes of a block share, and the short form of the quantiser for the 8-bit formats.
//   * every lane keeps the packed maximum AND minimum of its eight |x| (NaN wins the maximum); the maxima are
//     reduced over the block's lanes as packed pairs, the two halves are only compared on the lane that derives the header;
//   * that lane also derives the packed constants the block's lanes need and hands them over in one word:
//     2^-se and a second bf16 threshold (its own per format, see bf16_block_word);
//   * E4M3 / E5M2: when every |x| of the lanes that vote together is at least 2^(1-bias+se) -- no element in the
//     sub-range, none flushed or rounding to zero, which is nearly always so for these formats -- the code is
//     built from the SIGNED quotient with no per-element case analysis: exponent field and rounded fraction
//     OR-ed per word, the re-bias (one XOR) and the sign bits (one byte gather) applied to four packed codes
//     at a time.  Otherwise the lanes take pk_bf16_quantise, which handles every case.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void bf16_abs_range(const Pack<16>& p, uint32_t& mx2, uint32_t& mn2) {
    const __nv_bfloat162 a0 = __habs2(bf2(p.w[0])), a1 = __habs2(bf2(p.w[1])), a2 = __habs2(bf2(p.w[2])), a3 = __habs2(bf2(p.w[3]));
    mx2 = bf2_bits(__hmax2_nan(__hmax2_nan(a0, a1), __hmax2_nan(a2, a3)));
    mn2 = bf2_bits(__hmin2(__hmin2(a0, a1), __hmin2(a2, a3)));
}

// fp32 bits of the larger half of a packed pair of bf16 magnitudes; NaN wins (as 15-bit patterns the magnitudes
// order like integers, NaN above Inf above every finite value)
__device__ __forceinline__ uint32_t bf16x2_max_bits(uint32_t m2) {
    return max(m2 & 0xFFFFu, m2 >> 16) << 16;
}

// block_header for the maximum of bf16 inputs (fp32 bits with 16 zero low bits): such a maximum is never among the
// last floats below a power of two, so the round-up of the reference's log2 (shared_exponent) cannot apply and the
// shared exponent is the exponent field minus the format's largest exponent
template <class F>
__device__ __forceinline__ uint32_t block_header_bf16(uint32_t amax_bits, const F& f) {
    const int emax_b = fmt_emax(f) - fmt_bias(f);
    const uint32_t E = amax_bits >> 23;
    const uint32_t special = E == 255u ? 1u : 0u;
    const int se = max((int)E - 127 - emax_b, -127);
    const uint32_t sbyte = E == 0u ? 0u : (special ? 255u : (uint32_t)(se + 127));
    const uint32_t inv_field = (E == 0u || special) ? 127u : (uint32_t)(127 - se);
    return (inv_field << 23) | (sbyte << 8) | special;
}

// Low half: bf16 bits of 2^-se.  High half, by format: E2M1 -- the keep threshold (e2m1_block's ts2); E4M3 / E5M2 --
// 2^(1-bias+se), the smallest |x| of the short form (+Inf, i.e. never, for blocks so small that flushed inputs
// could lie above it); others: unused.  Bit 31: the block holds Inf / NaN.
template <class F>
__device__ __forceinline__ uint32_t bf16_block_word(uint32_t hdr) {
    const int sb = (int)((hdr >> 8) & 0xFFu);
    uint32_t second = 0u;
    if constexpr (F{}.eb() == 2 && F{}.fb() == 1) {
        second = (uint32_t)max((sb - 150) * 128, 0x7F);
    } else if constexpr (PkFmt<F>::RARE_SUBRANGE) {
        const int e = sb + 1 - PkFmt<F>::BIAS;
        second = e >= 2 ? (uint32_t)e << 7 : 0x7F80u;
    }
    return ((hdr >> 16) & 0x7F80u) | (second << 16) | (hdr << 31);
}

// short form (see above): 8 bf16 inputs of a lane -> 8 code bytes (out[0..2)) or 8 bf16 results (out[0..4))
template <class F, bool VALUES>
__device__ __forceinline__ void pk_bf16_quantise_normal(const Pack<16>& p, uint32_t inv2, uint32_t sf2, uint32_t* out) {
    using P = PkFmt<F>;
    static_assert(P::EB + P::FB == 7, "the sign gather assumes 8-bit codes");
    uint32_t qb[4], r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qb[i] = bf2_bits(__hmul2(bf2(p.w[i]), bf2(inv2)));                  // signed quotient
        const uint32_t sum = bf2_bits(__hadd2(bf2((qb[i] & 0x007F007Fu) | 0x3F803F80u), bf2(P::ROUND_C)));
        if constexpr (VALUES) {
            // (sum - SUM_BASE) << (7 - fb) as one multiply-add; OR-ed under the quotient's sign and exponent, times 2^se
            const uint32_t z = sum * (uint32_t)rt_k(P::FB == 3 ? 10 : 11) - P::SUM_BASE * (1u << (7 - P::FB));
            r[i] = bf2_bits(__hmul2(bf2((qb[i] & 0xFF80FF80u) | z), bf2(sf2)));
        } else {
            const uint32_t fr = sum * (uint32_t)rt_k(0) - P::SUM_BASE;       // 0 .. 2^fb in each half
            r[i] = ((qb[i] >> (7 - P::FB)) & P::EXP_MASK) | fr;             // exponent field not re-biased yet
        }
    }
    if constexpr (VALUES) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = r[i];
    } else {
        constexpr uint32_t FLIP4 = ((1u << (P::EB - 1)) << P::FB) * 0x01010101u;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t mag4 = __byte_perm(r[2 * i], r[2 * i + 1], 0x6420) ^ FLIP4;
            const uint32_t sgn4 = __byte_perm(qb[2 * i], qb[2 * i + 1], 0x7531);        // the halves' upper bytes: sign on top
            out[i] = mag4 | (sgn4 & 0x80808080u);
        }
    }
}

// One 16-byte access of a lane of a finite block, every format: picks the short form where it applies.
// `w2` is the block word, `mn2` this lane's packed minimum, `h` the block header (only read on the full path).
template <class F, bool VALUES>
__device__ __forceinline__ void bf16_quantise_access(const Pack<16>& p, uint32_t w2, uint32_t mn2, uint32_t h, uint32_t sf2, uint32_t* out) {
    const uint32_t inv2 = __byte_perm(w2, 0u, 0x1010);
    const uint32_t second2 = __byte_perm(w2, 0u, 0x3232);
    if constexpr (F{}.eb() == 2 && F{}.fb() == 1) {
        // (a vote that skips the keep threshold when no lane holds an element at or below it was measured: no gain)
        E2M1Block b;
        b.inv2 = inv2; b.sf2 = sf2; b.ts2 = second2;
        e2m1_bf16_quantise<VALUES>(p, b, out);
    } else if constexpr (PkFmt<F>::RARE_SUBRANGE) {
        const bool any_below = __any_sync(__activemask(), __hlt2_mask(bf2(mn2), bf2(second2)) != 0u);
        if (!any_below) pk_bf16_quantise_normal<F, VALUES>(p, inv2, sf2, out);
        else pk_bf16_quantise<F, VALUES>(p, e2m1_block(h), out);
    } else {
        pk_bf16_quantise<F, VALUES>(p, e2m1_block(h), out);
    }
}

// bf16 inputs: the tile of mxfp_b32_quant_kernel (8 elements per lane per access, 4 lanes per block)
template <class F, int U, int MODE, bool FULL>
__device__ __forceinline__ void mxfp_b32_quant_tile_bf16(const char* __restrict__ src, uint8_t* __restrict__ scales,
                                                         char* __restrict__ dst, int64_t first, int64_t left, const F& f) {
    constexpr bool WRITE_CODES = (MODE != MODE_QDQ);
    constexpr int V = 8, G = 4;
    static_assert(U <= G, "one lane of the group per in-flight access");
    constexpr int OB = WRITE_CODES ? V : 16;
    const int lane = threadIdx.x & 31;
    const int sub = lane & (G - 1);

    Pack<16> p[U];
    uint32_t mx2[U], mn2[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        if (FULL || j * kThreads < left) p[j] = load_pack<16>(src + (size_t)j * kThreads * 16);
        else p[j] = Pack<16>{{0u, 0u, 0u, 0u}};
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        bf16_abs_range(p[j], mx2[j], mn2[j]);
#pragma unroll
        for (int o = 1; o < G; o <<= 1) mx2[j] = bf2_bits(__hmax2_nan(bf2(mx2[j]), bf2(__shfl_xor_sync(0xFFFFFFFFu, mx2[j], o))));
    }
    // lane `sub` of each group derives the header and the block word of access `sub`
    uint32_t mine = mx2[0];
#pragma unroll
    for (int j = 1; j < U; ++j) mine = (sub == j) ? mx2[j] : mine;
    const uint32_t hdr = block_header_bf16(bf16x2_max_bits(mine), f);
    const uint32_t word = bf16_block_word<F>(hdr);
    const uint32_t sb = (hdr >> 8) & 0xFFu;
    const uint32_t sf2_mine = (sb == 0u ? 0x0040u : (sb << 7)) * 0x10001u;
    if (MODE == MODE_CODES && sub < U && (FULL || sub * kThreads < left))
        scales[(first + sub * kThreads) / G] = (uint8_t)sb;
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int owner = (lane & ~(G - 1)) + j;
        const uint32_t h = __shfl_sync(0xFFFFFFFFu, hdr, owner);
        const uint32_t w2 = __shfl_sync(0xFFFFFFFFu, word, owner);
        uint32_t sf2 = 0u;
        if constexpr (MODE == MODE_QDQ) sf2 = __shfl_sync(0xFFFFFFFFu, sf2_mine, owner);
        if (!FULL && j * kThreads >= left) continue;
        char* d = dst + (size_t)j * kThreads * OB;
        if (!(h & 1u)) {
            if constexpr (MODE == MODE_QDQ) {
                Pack<16> o;
                bf16_quantise_access<F, true>(p[j], w2, mn2[j], h, sf2, o.w);
                store_pack<16>(d, o);
            } else {
                Pack<V> o;
                bf16_quantise_access<F, false>(p[j], w2, mn2[j], h, sf2, o.w);
                store_pack<V>(d, o);
            }
        } else {
            // Inf / NaN block: the generic codec with the reference's fixed exponent
            uint32_t code[V];
#pragma unroll
            for (int i = 0; i < V; ++i) code[i] = mx_encode(pack_bits<KBF16>(p[j], i), 128, f);
            if constexpr (WRITE_CODES) {
                Pack<V> o;
#pragma unroll
                for (int i = 0; i < V; ++i) pack_set<1>(o, i, code[i]);
                store_pack<V>(d, o);
            } else {
                const float sf = scale_from_byte((h >> 8) & 0xFFu);
                uint32_t y[V];
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = mx_decode(code[i], sf, f);
                store_results<KBF16, V>(d, y, false);
            }
        }
    }
}

// fp32 inputs, E4M3 / E5M2 codes: the short form of the element encode, as pk_bf16_quantise_normal.  When every
// |x| of the lanes that vote together is at least 2^(1-bias+se) (`lim`), nothing is flushed, in the sub-range or
// rounding to zero, so four codes are: exponent field (low eb bits, re-biased later) OR rounded fraction per
// element from the SIGNED quotient, packed, re-biased with one XOR, signs gathered from the quotients' top bytes.
template <class F>
__device__ __forceinline__ uint32_t f32_codes4_normal(const uint32_t* x_bits, float inv, const F& f) {
    constexpr int fb = F{}.fb(), eb = F{}.eb();
    constexpr uint32_t cbits = (uint32_t)(127 + 23 - fb) << 23;           // 2^(23-fb)
    uint32_t qb[4], mag[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qb[i] = __float_as_uint(__fmul_rn(__uint_as_float(x_bits[i]), inv));
        // the reference's cut of the mantissa to 15 bits (minifloat/fake.py:45) commutes with the exact scaling
        const float m = __uint_as_float((qb[i] & 0x007FFF00u) | 0x3F800000u);
        const uint32_t fr = (uint32_t)mad_add((int)__float_as_uint(__fadd_rn(m, __uint_as_float(cbits))), -(int)(cbits + (1u << fb)));
        mag[i] = ((qb[i] >> (23 - fb)) & (((1u << eb) - 1u) << fb)) | fr;
    }
    return pack4_codes(mag, qb, f) ^ (((1u << (eb - 1)) << fb) * 0x01010101u);
}

// per-block bound of the short form as fp32 bits, from the block header (+Inf: never)
template <class F>
__device__ __forceinline__ uint32_t short_form_limit_bits(uint32_t hdr) {
    const int e = (int)((hdr >> 8) & 0xFFu) + 1 - PkFmt<F>::BIAS;
    return (uint32_t)(e >= 2 ? e : 255) << 23;
}

__device__ __forceinline__ float f32x4_absmin(const Pack<16>& p) {
    return fminf(fminf(fabsf(__uint_as_float(p.w[0])), fabsf(__uint_as_float(p.w[1]))),
                 fminf(fabsf(__uint_as_float(p.w[2])), fabsf(__uint_as_float(p.w[3]))));
}

template <class KIn, class F, int U, int MODE, bool FULL>
__device__ __forceinline__ void mxfp_b32_quant_tile(const char* __restrict__ src, uint8_t* __restrict__ scales,
                                                    char* __restrict__ dst, int64_t first, int64_t left, const F& f) {
    constexpr bool WRITE_CODES = (MODE != MODE_QDQ);
    constexpr int V = 16 / KIn::size;     // elements per lane per access: 4 (fp32) or 8 (16-bit)
    // fp32 inputs have issue slots to spare for the bookkeeping of the warp-level sub-range skip and
    // gain from it (0.72 -> 0.79 of the HBM peak for MXFP8 extract); for 16-bit inputs, with twice the
    // elements per byte moved, the bookkeeping costs more than the skipped table lookups save
    constexpr bool kWarpSkip = (KIn::size == 4);
    constexpr int G = 32 / V;             // lanes that share one 32-element block: 8 or 4
    static_assert(U <= G, "one lane of the group per in-flight access");
    constexpr int OB = WRITE_CODES ? V : 16;
    const int lane = threadIdx.x & 31;
    const int sub = lane & (G - 1);

    Pack<16> p[U];
    uint32_t amax[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        if (FULL || j * kThreads < left) p[j] = load_pack<16>(src + (size_t)j * kThreads * 16);
        else p[j] = Pack<16>{{0u, 0u, 0u, 0u}};
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        float m = __uint_as_float(pack_absmax_bits<KIn>(p[j]));
#pragma unroll
        for (int o = 1; o < G; o <<= 1) m = max_abs_nan(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        amax[j] = __float_as_uint(m);
    }
    // lane `sub` of each group derives the header of access `sub`
    uint32_t mine = amax[0];
#pragma unroll
    for (int j = 1; j < U; ++j) mine = (sub == j) ? amax[j] : mine;
    const uint32_t hdr = block_header(mine, f);
    // fp32 inputs, 8-bit element codes: the short form where no element of the voting lanes is below its block's bound
    constexpr bool kShortForm = (MODE == MODE_CODES) && KIn::size == 4 && PkFmt<F>::RARE_SUBRANGE;
    uint32_t lim_mine = 0u;
    if constexpr (kShortForm) lim_mine = short_form_limit_bits<F>(hdr);
    if (MODE == MODE_CODES && sub < U && (FULL || sub * kThreads < left))
        scales[(first + sub * kThreads) / G] = (uint8_t)(hdr >> 8);
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const uint32_t h = __shfl_sync(0xFFFFFFFFu, hdr, (lane & ~(G - 1)) + j);
        uint32_t lim = 0u;
        if constexpr (kShortForm) lim = __shfl_sync(0xFFFFFFFFu, lim_mine, (lane & ~(G - 1)) + j);
        if (!FULL && j * kThreads >= left) continue;
        char* d = dst + (size_t)j * kThreads * OB;
        if constexpr (kShortForm) {
            if (!(h & 1u)) {
                const bool any_below = __any_sync(__activemask(), f32x4_absmin(p[j]) < __uint_as_float(lim));
                if (!any_below) {
                    Pack<V> o;
                    o.w[0] = f32_codes4_normal(p[j].w, __uint_as_float(h & 0x7F800000u), f);
                    store_pack<V>(d, o);
                    continue;
                }
            }
        }
        if constexpr (MODE == MODE_QDQ) {
            if (!(h & 1u)) {
                const float inv = __uint_as_float(h & 0x7F800000u);
                const float sf = scale_from_byte((h >> 8) & 0xFFu);       // never 255 for a finite block
                uint32_t y[V];
                if constexpr (kWarpSkip) {
                    uint32_t qb[V], sum[V];
                    uint32_t sub = 0;                          // bit i: element i lies below the normal range
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        qb[i] = mx_quotient_bits(pack_bits<KIn>(p[j], i), inv);
                        y[i] = qdq_mag_normal(qb[i], &sum[i], f);
                        sub |= is_subrange(qb[i], f) ? (1u << i) : 0u;
                    }
                    // the lanes that sit here together skip the table path when none of them has such an element
                    if (__any_sync(__activemask(), sub != 0u)) {
#pragma unroll
                        for (int i = 0; i < V; ++i)
                            if (sub & (1u << i)) y[i] = qdq_mag_subrange(qb[i], sum[i], f);
                    }
#pragma unroll
                    for (int i = 0; i < V; ++i) y[i] = __float_as_uint(__fmul_rn(__uint_as_float(y[i]), sf)) | (qb[i] & 0x80000000u);
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) y[i] = mx_qdq_fast(pack_bits<KIn>(p[j], i), inv, sf, f);
                }
                store_results<KIn, V>(d, y, true);
                continue;
            }
        }
        if (!(h & 1u)) {
            const float inv = __uint_as_float(h & 0x7F800000u);
            uint32_t qb[V], mag[V];
#pragma unroll
            if constexpr (kWarpSkip) {
                uint32_t sub = 0;                              // bit i: element i lies below the normal range
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    qb[i] = mx_quotient_bits(pack_bits<KIn>(p[j], i), inv);
                    mag[i] = (uint32_t)encode_mag_normal(qb[i], f);
                    sub |= is_subrange(qb[i], f) ? (1u << i) : 0u;
                }
                // with wide-exponent formats few elements are that small relative to their block maximum:
                // the lanes that sit here together skip the table path when none of them has one
                if (__any_sync(__activemask(), sub != 0u)) {
#pragma unroll
                    for (int i = 0; i < V; ++i)
                        if (sub & (1u << i)) mag[i] = (uint32_t)subrange_code((int)mag[i], f);
                }
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    qb[i] = mx_quotient_bits(pack_bits<KIn>(p[j], i), inv);
                    mag[i] = (uint32_t)encode_mag_fp(qb[i], f);
                }
            }
            if constexpr (WRITE_CODES) {
                Pack<V> o;
#pragma unroll
                for (int i = 0; i < V; i += 4) o.w[i >> 2] = pack4_codes(&mag[i], &qb[i], f);
                store_pack<V>(d, o);
            }
        } else {
            uint32_t code[V];
#pragma unroll
            for (int i = 0; i < V; ++i) code[i] = mx_encode(pack_bits<KIn>(p[j], i), 128, f);
            if constexpr (WRITE_CODES) {
                Pack<V> o;
#pragma unroll
                for (int i = 0; i < V; ++i) pack_set<1>(o, i, code[i]);
                store_pack<V>(d, o);
            } else {
                const float sf = scale_from_byte((h >> 8) & 0xFFu);
                uint32_t y[V];
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = mx_decode(code[i], sf, f);
                store_results<KIn, V>(d, y, false);
            }
        }
    }
}

template <class KIn, class F, int U, int MODE>
__global__ void __launch_bounds__(kThreads) mxfp_b32_quant_kernel(const void* __restrict__ x, uint8_t* __restrict__ scales,
                                                                  uint8_t* __restrict__ elements, void* __restrict__ out,
                                                                  int64_t n_vec, F f) {
    grid_dependency_sync();
    constexpr int V = 16 / KIn::size;
    const int64_t first = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;
    const char* src = reinterpret_cast<const char*>(x) + first * 16;
    char* dst = MODE != MODE_QDQ ? reinterpret_cast<char*>(elements) + first * V : reinterpret_cast<char*>(out) + first * 16;
    const bool full = (int64_t)(blockIdx.x + 1) * (kThreads * U) <= n_vec;
    if constexpr (std::is_same<KIn, KBF16>::value) {
        if (full) mxfp_b32_quant_tile_bf16<F, U, MODE, true>(src, scales, dst, first, 0, f);
        else mxfp_b32_quant_tile_bf16<F, U, MODE, false>(src, scales, dst, first, n_vec - first, f);
    } else {
        if (full) mxfp_b32_quant_tile<KIn, F, U, MODE, true>(src, scales, dst, first, 0, f);
        else mxfp_b32_quant_tile<KIn, F, U, MODE, false>(src, scales, dst, first, n_vec - first, f);
    }
}

template <class KOut, class F, int U>
__global__ void __launch_bounds__(kThreads) mxfp_b32_compose_kernel(const uint8_t* __restrict__ scales,
                                                                    const uint8_t* __restrict__ elements,
                                                                    void* __restrict__ out, int64_t n_vec, F f) {
    grid_dependency_sync();
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
        const bool plain = sb[j] != 255u;
        uint32_t y[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const uint32_t code = pack_get<1>(c[j], i);
            if (plain) y[i] = __float_as_uint(__fmul_rn(__uint_as_float(decode_f32_fast(code, f)), sf));
            else y[i] = mx_decode(code, sf, f);
        }
        store_results<KOut, V>(reinterpret_cast<char*>(out) + idx * 16, y, plain);
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
            rc = launch_ew<KIn, KU16, true>(x, codes, n, ExtractOp<decltype(f), true>{f}, st);
        });
        if (!fast) rc = launch_ew<KIn, KU16, false>(x, codes, n, ExtractOp<FmtRT, false>{FmtRT{eb, fb, is_finite, rm}}, st);
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
            rc = launch_ew<KU16, KOut, true>(codes, out, n, ComposeOp<decltype(f), true>{f}, st);
        });
        if (!fast) rc = launch_ew<KU16, KOut, false>(codes, out, n, ComposeOp<FmtRT, false>{FmtRT{eb, fb, is_finite, 0}}, st);
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
                rc = launch_ew<KIn, KOut, true>(x, out, n, QdqOp<decltype(f), true>{f}, st);
            });
            if (!fast)
                rc = launch_ew<KIn, KOut, false>(x, out, n, QdqOp<FmtRT, false>{FmtRT{eb, fb, is_finite, rm}}, st);
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
                    const cudaError_t e = launch_overlapped(mxfp_b32_quant_kernel<KIn, decltype(f), U, WRITE_CODES ? MODE_CODES : MODE_QDQ>,
                                                            (unsigned)grid, kThreads, st, x, scales, elements, out, n_vec, f);
                    if (e != cudaSuccess) set_last_cuda_error(e);
                    rc = e == cudaSuccess ? check_launch() : MXQ_ELAUNCH;
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
                const cudaError_t e = launch_overlapped(mxfp_b32_compose_kernel<KOut, decltype(f), U>, (unsigned)grid, kThreads, st, scales, elements,
                                                        out, n_vec, f);
                if (e != cudaSuccess) set_last_cuda_error(e);
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

// Per-tensor minifloat (FP8 E4M3 / E5M2, round to nearest, is_finite) quantisation of a [M, K]
// activation straight into the tensor-core operand layout: hardware FP8 codes and left-operand scale
// chunks holding 2^0 (2^1 for a 32-element group that contains the reference's saturated E4M3 480 or
// an E5M2 top-binade value, whose codes are halved).  One lane per 16 input bytes; the 4 or 8 lanes
// of a 32-element group agree on the re-bias with shuffles.
template <class KIn, class F>
__global__ void __launch_bounds__(kThreads) minifloat_hwpack_kernel(const void* __restrict__ x, uint8_t* __restrict__ hw_codes,
                                                                    uint8_t* __restrict__ hw_sf, int64_t n_vec, F f, PackGeom geom) {
    constexpr int V = 16 / KIn::size;
    constexpr int G = 32 / V;
    const int64_t idx = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const bool active = idx < n_vec;                 // whole groups are active or not: n_vec is a multiple of G
    const int lane = threadIdx.x & 31;
    Pack<16> p = active ? load_pack<16>(reinterpret_cast<const char*>(x) + idx * 16) : Pack<16>{{0u, 0u, 0u, 0u}};
    constexpr uint32_t hw_max = (F{}.eb() == 4) ? 0x7Eu : 0x7Bu;
    uint32_t code[V];
    uint32_t bad = 0;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        code[i] = encode_f32_fast(pack_bits<KIn>(p, i), f);          // sign at bit 7 for the 8-bit formats
        bad |= ((code[i] & 0x7Fu) > hw_max) ? 1u : 0u;
    }
#pragma unroll
    for (int o = 1; o < G; o <<= 1) bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, o);
    if (!active) return;
    Pack<V> out;
#pragma unroll
    for (int i = 0; i < V; ++i) {
        uint32_t mag = code[i] & 0x7Fu;
        if (bad) mag = (mag >= (2u << f.fb())) ? mag - (1u << f.fb()) : (mag + ((mag >> 1) & 1u)) >> 1;
        pack_set<1>(out, i, mag | (code[i] & 0x80u));
    }
    store_pack_keep<V>(hw_codes + idx * V, out);
    if ((lane & (G - 1)) == 0) hw_sf[sf_chunk_offset((uint32_t)(idx / G), geom)] = (uint8_t)(bad ? 128u : 127u);
}

// Four hardware magnitude+sign code bytes of a block that is stored with its scale raised by one: every
// magnitude becomes the code of half the value -- exponent minus one for codes with exponent >= 2, a
// round-half-to-even shift for the two lowest binades -- on all four bytes of the word at once.
template <int FB>
__device__ __forceinline__ uint32_t halve_codes4(uint32_t c) {
    constexpr uint32_t ONE = 0x01010101u;
    const uint32_t mag = c & 0x7F7F7F7Fu;
    // per byte: 0xFF where mag >= 2 << FB (adding 0x80 - (2 << FB) carries into bit 7 exactly then)
    const uint32_t big = (((mag + ONE * (0x80u - (2u << FB))) >> 7) & ONE) * 0xFFu;
    const uint32_t normal = mag - (big & (ONE << FB));                       // no borrow: those bytes are >= 2 << FB
    const uint32_t small = ((mag + ((mag >> 1) & ONE)) >> 1) & 0x7F7F7F7Fu;   // bytes < 2 << FB: no carry out of the byte
    return (big & normal) | (~big & small) | (c & 0x80808080u);
}

// ------------------------------------------------------------------------------------------------
// Activation -> tensor-core left operand in one pass (MXFP8 elements): hardware codes [M, K] and the scale
// factors in the chunked order of mxq_gemm.cu.  A flat pass over x like the extract kernel (a lane owns 16
// bytes per access, four accesses in flight, the 4 or 8 lanes of a 32-element block reduce its maximum with
// shuffles; bf16 inputs take the packed two-per-word quantiser), plus:
//   * a block holding a magnitude the hardware format reads as NaN/Inf (reference E4M3 0x7F, reference E5M2
//     exponent 31) is stored as (scale + 1, elements / 2), four code bytes per instruction;
//   * the scale bytes of four consecutive blocks of a row are adjacent in their chunk, so one lane gathers them
//     with shuffles and stores one 32-bit word instead of four scattered bytes (K % 128 == 0).
// ------------------------------------------------------------------------------------------------
template <class KIn, class F, bool WORDS>
__global__ void __launch_bounds__(kThreads) mx_quant_pack_flat_kernel(const void* __restrict__ x, uint8_t* __restrict__ hw_codes,
                                                                      uint8_t* __restrict__ hw_sf, int64_t n_vec, PackGeom geom) {
    constexpr int V = 16 / KIn::size;              // elements per lane per access: 8 or 4
    constexpr int G = 32 / V;                      // lanes that share a 32-element block: 4 or 8
    constexpr int U = 4;
    const int lane = threadIdx.x & 31;
    const int sub = lane & (G - 1);
    const int64_t first = (int64_t)blockIdx.x * (kThreads * U) + threadIdx.x;
    const F f{};
    constexpr uint32_t probe = (F{}.eb() == 4) ? 0x01010101u : 0x04040404u;    // carry out of the magnitude byte: a code the hardware reads as NaN / Inf
    // E2M1: the codes are stored two per byte (the 4-bit x 4-bit GEMM's operand); every E2M1 code is one the hardware has
    constexpr bool NIB = (F{}.eb() == 2 && F{}.fb() == 1);
    constexpr bool BF16 = std::is_same<KIn, KBF16>::value;
    Pack<16> p[U];
    uint32_t amax[U], amin[U];             // bf16: packed pairs (see bf16_abs_range); else fp32 bits of the maximum
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int64_t vec = first + (int64_t)j * kThreads;
        p[j] = vec < n_vec ? load_pack<16>(reinterpret_cast<const char*>(x) + vec * 16) : Pack<16>{{0u, 0u, 0u, 0u}};
    }
#pragma unroll
    for (int j = 0; j < U; ++j) {
        if constexpr (BF16) {
            bf16_abs_range(p[j], amax[j], amin[j]);
#pragma unroll
            for (int o = 1; o < G; o <<= 1) amax[j] = bf2_bits(__hmax2_nan(bf2(amax[j]), bf2(__shfl_xor_sync(0xFFFFFFFFu, amax[j], o))));
        } else {
            float m = __uint_as_float(pack_absmax_bits<KIn>(p[j]));
#pragma unroll
            for (int o = 1; o < G; o <<= 1) m = max_abs_nan(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            amax[j] = __float_as_uint(m);
            amin[j] = 0u;
        }
    }
    // lane `sub` of each group derives the header of access `sub` (U <= G)
    uint32_t mine = amax[0];
#pragma unroll
    for (int j = 1; j < U; ++j) mine = (sub == j) ? amax[j] : mine;
    uint32_t hdr;
    if constexpr (BF16) hdr = block_header_bf16(bf16x2_max_bits(mine), f);
    else hdr = block_header(mine, f);
    constexpr bool F32 = KIn::size == 4;
    // the second per-block word: bf16 -- see bf16_block_word; fp32 -- the bound of the short form
    const uint32_t word = BF16 ? bf16_block_word<F>(hdr) : (F32 ? short_form_limit_bits<F>(hdr) : 0u);
    uint32_t sb_of[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const int owner = (lane & ~(G - 1)) + j;
        const uint32_t h = __shfl_sync(0xFFFFFFFFu, hdr, owner);
        uint32_t w2 = 0u;
        if constexpr (BF16 || F32) w2 = __shfl_sync(0xFFFFFFFFu, word, owner);
        const int64_t vec = first + (int64_t)j * kThreads;
        Pack<V> o;
        uint32_t sbyte = (h >> 8) & 0xFFu;
        uint32_t bad = 0;                       // non-zero: a code of this lane is one the hardware reads as NaN / Inf
        if (!(h & 1u)) {
            if constexpr (BF16) {
                bf16_quantise_access<F, false>(p[j], w2, amin[j], h, 0u, o.w);
            } else {
                const float inv = __uint_as_float(h & 0x7F800000u);
                bool short_form = false;
                if constexpr (F32 && PkFmt<F>::RARE_SUBRANGE) short_form = !__any_sync(__activemask(), f32x4_absmin(p[j]) < __uint_as_float(w2));
                if (short_form) {
                    o.w[0] = f32_codes4_normal(p[j].w, inv, f);
                } else {
                    uint32_t qb[V], mag[V];
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        qb[i] = mx_quotient_bits(pack_bits<KIn>(p[j], i), inv);
                        mag[i] = (uint32_t)encode_mag_fp(qb[i], f);
                    }
#pragma unroll
                    for (int i = 0; i < V; i += 4) o.w[i >> 2] = pack4_codes(&mag[i], &qb[i], f);
                }
            }
            if constexpr (!NIB) {
#pragma unroll
                for (int i = 0; i < V / 4; ++i) bad |= ((o.w[i] & 0x7F7F7F7Fu) + probe) & 0x80808080u;
            }
        } else {
            // Inf/NaN block: scale byte 255 is NaN for the tensor cores too; the codes do not matter
#pragma unroll
            for (int i = 0; i < V / 4; ++i) o.w[i] = 0u;
            sbyte = 255u;
        }
        // the lanes of a block agree with xor-shuffles that every lane of the warp executes (a vote with a mask per
        // group compiles to a loop over the groups); lanes of Inf/NaN blocks contribute nothing
        if constexpr (!NIB) {
#pragma unroll
            for (int w = 1; w < G; w <<= 1) bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, w);
            if (bad != 0u) {
#pragma unroll
                for (int i = 0; i < V / 4; ++i) o.w[i] = halve_codes4<F{}.fb()>(o.w[i]);
                if (sbyte < 255u) sbyte += 1u;
            }
            if (vec < n_vec) store_pack_keep<V>(hw_codes + vec * V, o);
        } else {
            // four code bytes -> two bytes of nibbles (element 2i in the low nibble of byte i)
            uint32_t nib = 0u;
#pragma unroll
            for (int i = 0; i < V / 4; ++i) {
                uint32_t t = o.w[i] & 0x0F0F0F0Fu;
                t |= t >> 4;
                nib |= ((t & 0xFFu) | ((t >> 8) & 0xFF00u)) << (16 * i);
            }
            if (vec < n_vec) {
                if constexpr (V == 8) *reinterpret_cast<uint32_t*>(hw_codes + vec * 4) = nib;
                else *reinterpret_cast<uint16_t*>(hw_codes + vec * 2) = (uint16_t)nib;
            }
        }
        sb_of[j] = sbyte;
    }
    // lane `sub` of each group stores the scale byte of access `sub`, so that the position in the chunked array is
    // worked out once per lane instead of once per access
    uint32_t sb_mine = sb_of[0];
#pragma unroll
    for (int j = 1; j < U; ++j) sb_mine = (sub == j) ? sb_of[j] : sb_mine;
    const int64_t vec_mine = first - sub + (int64_t)(sub < U ? sub : 0) * kThreads;      // first lane of the group, access `sub`
    const bool mine_ok = sub < U && vec_mine < n_vec;
    const uint32_t blk = (uint32_t)(vec_mine / G);
    if constexpr (WORDS) {
        // blocks blk .. blk + 3 (blk % 4 == 0: the groups 0..3 or 4..7 of the warp) are K blocks 0 .. 3 of one row and
        // one 128-column step; their bytes are adjacent in the chunk: gather them from the lanes G, 2G, 3G further on
        uint32_t w = sb_mine | (__shfl_down_sync(0xFFFFFFFFu, sb_mine, G) << 8);
        w |= __shfl_down_sync(0xFFFFFFFFu, w, 2 * G) << 16;
        if ((lane & (4 * G - 1)) < G && mine_ok) *reinterpret_cast<uint32_t*>(hw_sf + sf_chunk_offset(blk, geom)) = w;
    } else {
        if (mine_ok) hw_sf[sf_chunk_offset(blk, geom)] = (uint8_t)sb_mine;
    }
}

// Quantise a [M, K] activation to MXFP8 (32-element blocks along K) straight into the tensor-core
// operand layout of mxq_gemm.cu: hardware FP8 codes [M, K] and left-operand scale-factor chunks.
// One pass over x instead of extract + pack. Declared in mxq_internal.h; returns MXQ_ESIZE when the
// format / alignment is not covered so the caller can take the two-kernel route.
namespace mxq {
int quantize_pack_left_operand(const void* x, int x_dtype, int64_t M, int64_t K, int eb, int fb, uint8_t* hw_codes,
                               uint8_t* hw_sf, int64_t sf_bytes, int* hw_format, cudaStream_t st) {
    const bool e4m3 = (eb == 4 && fb == 3), e5m2 = (eb == 5 && fb == 2), e2m1 = (eb == 2 && fb == 1);
    if (!(e4m3 || e5m2 || e2m1) || K % 32 != 0 || M * K / 32 >= (1ll << 31)) return MXQ_ESIZE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hw_codes) | reinterpret_cast<uintptr_t>(hw_sf)) % 16 != 0) return MXQ_ESIZE;
    *hw_format = e2m1 ? 5 : (e5m2 ? 1 : 0);          // E2M1: packed nibbles, the left operand of the 4-bit x 4-bit GEMM
    // padding rows / K blocks of the chunked scale array must read as 2^0; none exist for whole tiles
    if ((M % 256 != 0 || K % 128 != 0) && cudaMemsetAsync(hw_sf, 127, (size_t)sf_bytes, st) != cudaSuccess) return check_launch();
    PackGeom g;
    g.kbpr = (uint32_t)(K / 32);
    g.shift = 0;
    while ((1u << g.shift) < g.kbpr) ++g.shift;
    g.magic = (uint32_t)((((uint64_t)1 << (31 + g.shift)) + g.kbpr - 1) / g.kbpr);
    g.KT = (uint32_t)((K + 127) / 128);
    const bool words = K % 128 == 0;
    int rc = MXQ_OK;
    with_kind(x_dtype, [&](auto kin) {
        using KIn = decltype(kin);
        constexpr int V = 16 / KIn::size;
        const int64_t n_vec = M * K / V;
        const unsigned grid = (unsigned)((n_vec + kThreads * 4 - 1) / (kThreads * 4));
        auto go = [&](auto fmt) {
            using F = decltype(fmt);
            if (words) mx_quant_pack_flat_kernel<KIn, F, true><<<grid, kThreads, 0, st>>>(x, hw_codes, hw_sf, n_vec, g);
            else mx_quant_pack_flat_kernel<KIn, F, false><<<grid, kThreads, 0, st>>>(x, hw_codes, hw_sf, n_vec, g);
        };
        if (e4m3) go(FmtCT<4, 3, true, RM_RN>{}); else if (e5m2) go(FmtCT<5, 2, true, RM_RN>{}); else go(FmtCT<2, 1, true, RM_RN>{});
        rc = check_launch();
    });
    return rc;
}

// The same for per-tensor minifloat codes (unit block scales); declared in mxq_internal.h.
int minifloat_quantize_pack_left_operand(const void* x, int x_dtype, int64_t M, int64_t K, int eb, int fb, uint8_t* hw_codes,
                                         uint8_t* hw_sf, int64_t sf_bytes, int* hw_format, cudaStream_t st) {
    const bool e4m3 = (eb == 4 && fb == 3), e5m2 = (eb == 5 && fb == 2);
    if (!(e4m3 || e5m2) || K % 32 != 0 || M * K / 32 >= (1ll << 31)) return MXQ_ESIZE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(hw_codes)) % 16 != 0) return MXQ_ESIZE;
    *hw_format = e5m2 ? 1 : 0;
    if (cudaMemsetAsync(hw_sf, 127, (size_t)sf_bytes, st) != cudaSuccess) return check_launch();
    PackGeom g;
    g.kbpr = (uint32_t)(K / 32);
    g.shift = 0;
    while ((1u << g.shift) < g.kbpr) ++g.shift;
    g.magic = (uint32_t)((((uint64_t)1 << (31 + g.shift)) + g.kbpr - 1) / g.kbpr);
    g.KT = (uint32_t)((K + 127) / 128);
    int rc = MXQ_OK;
    with_kind(x_dtype, [&](auto kin) {
        using KIn = decltype(kin);
        constexpr int V = 16 / KIn::size;
        const int64_t n_vec = M * K / V;
        const int64_t grid = (n_vec + kThreads - 1) / kThreads;
        if (e4m3)
            minifloat_hwpack_kernel<KIn, FmtCT<4, 3, true, RM_RN>><<<(unsigned)grid, kThreads, 0, st>>>(x, hw_codes, hw_sf, n_vec, FmtCT<4, 3, true, RM_RN>{}, g);
        else
            minifloat_hwpack_kernel<KIn, FmtCT<5, 2, true, RM_RN>><<<(unsigned)grid, kThreads, 0, st>>>(x, hw_codes, hw_sf, n_vec, FmtCT<5, 2, true, RM_RN>{}, g);
        rc = check_launch();
    });
    return rc;
}
}  // namespace mxq
