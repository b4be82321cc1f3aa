// Dequantise-in-the-loader GEMM for sm_100a: out[M,N] = X[M,K] * dequant(W)[N,K]^T (+ bias).
//
// This is the tensor-core path of the layer types whose operands are not both block-quantised codes:
// the activation is a dense bf16 / fp16 matrix (raw, or already fake-quantised by the element-wise
// kernels), the weight is either dense too or stays in memory as quantised codes that this kernel
// expands on the fly:
//   * SRC_RAW : W is a dense [N, K] matrix of the activation's dtype, brought in by TMA;
//   * SRC_MX  : W is an MXFP tensor as the reference stores it -- one code byte per element
//               [N, K] plus one E8M0 scale per 32 elements along K [N, K/32] (the `w_elements` /
//               `w_scales` of mase-triton's MXFPLinearPTQ, src/mase_triton/mxfp/layers.py:66-80);
//   * SRC_MF  : W is a per-tensor minifloat tensor, one uint16 code per element [N, K]
//               (`w_element` of MinifloatLinearPTQ, src/mase_triton/minifloat/layers.py).
// It replaces "compose the whole weight to a dense tensor, then call a library GEMM"
// (src/mase_triton/mxfp/functional/linear.py:10-33,67-116, minifloat/functional/linear.py:10-105):
// the dequantised weight never exists in HBM.
//
// Structure (one persistent CTA per SM, 256 x 256 output tile, K step 64):
//   warp 0      TMA producer: X tile (and a raw W tile) into a 128-byte-swizzled shared-memory ring;
//   warp 1      issues tcgen05.mma.kind::f16 (M=128, N=256, K=16), fp32 accumulators in tensor
//               memory (two 128 x 256 blocks = all 512 columns);
//   warps 2-5   epilogue: tcgen05.ld, bias, convert, staging in shared memory, TMA store (asynchronous:
//               the accumulator is handed back after the last tcgen05.ld, not after the global stores);
//   warps 6-13  dequantisers: each thread owns 16 consecutive K elements of four rows of the W tile; it reads
//               their code bytes (one 16-byte load per row) and scales three ring stages ahead (kept
//               in registers), expands them to bf16 / fp16 exactly as the reference's compose
//               does (decode * 2^(scale-127), rounded once to the operand dtype), write the
//               swizzled tile with 16-byte shared stores, make them visible to the tensor cores
//               (fence.proxy.async) and arrive on the stage's mbarrier next to the TMA bytes.
// Every mbarrier wait is bounded; a wait that runs out records a code in the caller's status word and
// the CTA unwinds (copies and MMAs in flight are waited for, tensor memory is freed).
#include "mxq_codec.h"
#include "mxq_tc.cuh"

namespace mxq {
namespace dq {

using namespace tc;

constexpr int BN = 256, BK = 64;                 // BK elements of 2 bytes = one 128-byte swizzle span
constexpr int B_BYTES = BN * BK * 2;             // 32 KiB
constexpr int BAR_BYTES = 256;
constexpr int TMEM_COLS = 512;
constexpr int DQ_WARPS = 8;
constexpr int DQ_THREADS = DQ_WARPS * 32;
constexpr int THREADS = 192 + DQ_THREADS;
constexpr int PF = 3;                            // ring stages of codes a dequantiser thread holds in registers
constexpr int SEGS = BK / 16;                    // a dequantiser thread expands 16 consecutive K elements of a row: 4 threads per row
constexpr int ROWS_PER_PASS = DQ_THREADS / SEGS; // 64 rows of the W tile per pass over the threads
constexpr int ROWS_PER_THREAD = BN / ROWS_PER_PASS;    // 4 rows (64 elements) per thread per stage

enum : int { SRC_RAW = 0, SRC_MX = 1, SRC_MF = 2 };

struct WSource {
    const void* codes;         // SRC_MX: uint8 [N, K]; SRC_MF: uint16 [N, K]
    const uint8_t* scales;     // SRC_MX: uint8 [N, K / 32]
    int eb, fb, fin;
};

template <int MH> struct Cfg {
    static constexpr int BM = 128 * MH;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;                      // multiple of 1024
    static constexpr int STAGES = MH == 2 ? 3 : 4;
    static constexpr int STAGING = 4 * EPI_SLOT_BYTES;                         // staging slots of the four epilogue warps
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING + BAR_BYTES + 1024;  // + slack to align the ring
};

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// ------------------------------------------------------------------------------------------------
// code -> operand dtype, eight elements (one 16-byte chunk of a tile row) at a time
// ------------------------------------------------------------------------------------------------
struct DqConsts {
    uint32_t mag_mask;      // (1 << (eb + fb)) - 1
    uint32_t sign_pos;      // eb + fb
    uint32_t up;            // 23 - fb: magnitude field -> top of an fp32 mantissa / bottom of its exponent
    float rebias;           // 2^(127 - bias)
    uint32_t top_exp;       // exponent field that decodes to Inf / NaN: all ones when !fin, 255 for 8 exponent bits (the value
                            // 2^128 overflows fp32 as it does in the reference's fp32 arithmetic), else 0xFFFFFFFF (never matches)
    uint32_t nan_mask;      // fraction bits that turn the Inf into a NaN (!fin only)
    // packed-bf16 route (MX codes -> bf16): field shifts inside a half word holding code << 8
    uint32_t mag_shift2, mag_mask2, sign_shift2, bias_;
};

__device__ __forceinline__ DqConsts dq_consts(int eb, int fb, int fin) {
    DqConsts c;
    const int bias = (1 << (eb - 1)) - 1;
    c.mag_mask = (1u << (eb + fb)) - 1u;
    c.sign_pos = (uint32_t)(eb + fb);
    c.up = (uint32_t)(23 - fb);
    c.rebias = __uint_as_float((uint32_t)(254 - bias) << 23);
    c.top_exp = !fin ? ((1u << eb) - 1u) : (eb == 8 ? 255u : 0xFFFFFFFFu);
    c.nan_mask = !fin ? ((1u << fb) - 1u) : 0u;
    c.mag_shift2 = (uint32_t)(1 + fb);
    c.mag_mask2 = (c.mag_mask << (7 - fb)) * 0x10001u;
    c.sign_shift2 = (uint32_t)(7 - eb - fb);
    c.bias_ = (uint32_t)bias;
    return c;
}

// one code -> fp32 value of the reference's decode (src/mase_triton/minifloat/fake.py:81-125), times `scale`
__device__ __forceinline__ float decode_scaled(uint32_t code, const DqConsts& c, float scale) {
    const uint32_t mag = code & c.mag_mask;
    float v = __fmul_rn(__uint_as_float(mag << c.up), c.rebias);      // exact: subnormal codes are fp32 subnormals here
    if ((mag >> (23 - c.up)) == c.top_exp) v = (mag & c.nan_mask) ? __uint_as_float(0x7FC00000u) : __uint_as_float(0x7F800000u);
    v = __fmul_rn(v, scale);
    return __uint_as_float(__float_as_uint(v) | ((code >> c.sign_pos) << 31));
}

template <int DT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (DT == MXQ_BF16) { const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&h); }
    else { const __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&h); }
}

// SRC_MX -> bf16, element format known at compile time: sixteen code bytes (one 16-byte load) and their block's
// scale byte -> sixteen bf16 values.  Two elements per 32-bit word on the packed bf16 units: a code shifted so
// that its exponent field sits at the bottom of bf16's exponent field and its fraction at the top of bf16's
// mantissa is the value times 2^(bias-127) (subnormal codes become bf16 subnormals, still exact); one multiply
// by 2^(scale-bias) restores the bias and applies the block scale, rounding once to bf16 exactly like the
// reference's fp32 product followed by .to(bfloat16).  Scales too large for that factor to be a finite bf16
// (and 255 = Inf) take a second multiply.
template <int EB, int FB>
__device__ __forceinline__ void dequant_mx16_bf16(const uint4& w, uint32_t sbyte, uint4& lo, uint4& hi) {
    constexpr uint32_t BIAS = (1u << (EB - 1)) - 1u;
    constexpr uint32_t MAG_MASK2 = (((1u << (EB + FB)) - 1u) << (7 - FB)) * 0x10001u;
    constexpr int SIGN_SHIFT = 7 - EB - FB;                           // 0 for the 8-bit formats
    const bool one_step = sbyte <= 127u + BIAS;
    const uint32_t f1 = (((one_step ? sbyte + 127u : 254u) - BIAS) << 7) * 0x10001u;
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t t = __byte_perm(words[j >> 1], 0u, (j & 1) ? 0x3424u : 0x1404u);     // code << 8 in each half
        const uint32_t sg = SIGN_SHIFT ? (t << SIGN_SHIFT) : t;
        const uint32_t v = ((t >> (1 + FB)) & MAG_MASK2) | (sg & 0x80008000u);
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&v), *reinterpret_cast<const __nv_bfloat162*>(&f1));
        o[j] = *reinterpret_cast<const uint32_t*>(&r);
    }
    if (!one_step) {
        const uint32_t f2 = (sbyte == 255u ? 0x7F80u : (sbyte << 7)) * 0x10001u;           // 2^(scale-127); here scale > 127
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&o[j]), *reinterpret_cast<const __nv_bfloat162*>(&f2));
            o[j] = *reinterpret_cast<const uint32_t*>(&r);
        }
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// SRC_MX, any dtype / format (fp32 arithmetic): eight code bytes (two words) and their block's scale byte -> eight DT elements
template <int DT>
__device__ __forceinline__ uint4 dequant_mx8(uint32_t w0, uint32_t w1, uint32_t sbyte, const DqConsts& c) {
    const float scale = __uint_as_float(sbyte == 0u ? 0x00400000u : (sbyte << 23));     // 255 -> +Inf as exp2(128) in fp32
    const uint32_t words[2] = {w0, w1};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t pair = words[j >> 1] >> (16 * (j & 1));
        o[j] = pack2<DT>(decode_scaled(pair & 0xFFu, c, scale), decode_scaled((pair >> 8) & 0xFFu, c, scale));
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// SRC_MF: eight uint16 codes -> eight DT elements
template <int DT>
__device__ __forceinline__ uint4 dequant_mf8(uint4 w, const DqConsts& c) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack2<DT>(decode_scaled(words[j] & 0xFFFFu, c, 1.0f), decode_scaled(words[j] >> 16, c, 1.0f));
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// what a dequantiser thread keeps in registers for one ring stage: the codes of its 16 elements in each of its
// 4 rows (+ the scale byte of the 32-element block they belong to)
template <int SRC> struct Staged;
template <> struct Staged<SRC_MX> { uint4 codes[ROWS_PER_THREAD]; uint32_t sb[ROWS_PER_THREAD]; };
template <> struct Staged<SRC_MF> { uint4 lo[ROWS_PER_THREAD], hi[ROWS_PER_THREAD]; };
template <> struct Staged<SRC_RAW> {};

// DT: MXQ_BF16 / MXQ_F16 (operand and output dtype); MH: 128-row accumulators per CTA tile; SRC: where W comes from
template <int DT, int MH, int SRC>
__global__ void __launch_bounds__(THREADS, 1)
dq_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const WSource wsrc,
               void* __restrict__ out, const BiasRef bias, int M, int N, int K, int bn, uint32_t idesc, int* status,
               const __grid_constant__ OutMaps omaps, int tma_out) {
    using C = Cfg<MH>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;
    uint8_t* ring_ptr = smem_raw + (ring - raw);
    // ring | staging slots of the epilogue | barriers
    const uint32_t bars = ring + STAGES * C::STAGE_BYTES + C::STAGING;   // full[S], empty[S], accum_full, tmem_empty[2], drain, tmem slot
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring_ptr + STAGES * C::STAGE_BYTES + C::STAGING + 8 * (2 * STAGES + 4));
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (2 * STAGES);
    auto tmem_empty_bar = [&](int h) { return bars + 8u * (2 * STAGES + 1 + h); };
    const uint32_t drain_bar = bars + 8u * (2 * STAGES + 3);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = (K + BK - 1) / BK;
    // bn: columns of the CTA tile (64, 128 or 256; always 256 when the weight is expanded by the dequantiser warps)
    const int MT = (M + C::BM - 1) / C::BM, NT = (N + bn - 1) / bn;
    const int num_tiles = MT * NT;

    if (threadIdx.x == 0) {
        // a stage is full when the TMA bytes have landed and (for quantised W) every dequantiser warp has written its rows
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1 + (SRC != SRC_RAW ? DQ_WARPS : 0)); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        mbar_init(tmem_empty_bar(0), 4);
        mbar_init(tmem_empty_bar(1), 4);
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        bool ok = true;
        uint32_t it = 0;
        const uint32_t tx_bytes = C::A_BYTES + (SRC == SRC_RAW ? (uint32_t)(bn * BK * 2) : 0u);
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int mt, nt;
            tile_coords(tile, MT, NT, mt, nt);
            for (int kt = 0; kt < KT && ok; ++kt, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES) ok = mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, status, ST_PRODUCER_TIMEOUT);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t st = ring + s * C::STAGE_BYTES;
                    mbar_expect_tx(full_bar(s), tx_bytes);
                    tma_load_2d(st, &map_a, kt * BK, mt * C::BM, full_bar(s));
                    if constexpr (SRC == SRC_RAW) tma_load_2d(st + C::A_BYTES, &map_b, kt * BK, nt * bn, full_bar(s));
                }
                __syncwarp();
            }
        }
        // copies started by this warp must have landed before the CTA gives its shared memory back; when W is
        // dequantised by other warps the barrier phase may stay open after a failure, so this wait is bounded too
        const uint32_t issued = it;
        for (uint32_t j = (issued > (uint32_t)STAGES ? issued - STAGES : 0u); j < issued; ++j)
            mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, ST_PRODUCER_TIMEOUT);
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        bool ok = true;
        uint32_t it = 0, tcount = 0;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
            for (int kt = 0; kt < KT && ok; ++kt, ++it) {
                const int s = it % STAGES;
                ok = mbar_wait(full_bar(s), (it / STAGES) & 1, status, ST_MMA_TIMEOUT);
                const uint32_t st = ring + s * C::STAGE_BYTES;
                const uint64_t b_desc = smem_desc(st + C::A_BYTES, 16, 1024, LAYOUT_SW128);
#pragma unroll
                for (int h = 0; h < MH; ++h) {
                    if (kt == 0 && tcount > 0 && ok) ok = mbar_wait(tmem_empty_bar(h), (tcount - 1) & 1, status, ST_MMA_TIMEOUT);
                    tc_fence_after();
                    if (ok && lane == 0) {
                        const uint64_t a_desc = smem_desc(st + h * 16384, 16, 1024, LAYOUT_SW128);
#pragma unroll
                        for (uint32_t k = 0; k < BK / 16; ++k)      // +32 bytes along K = +2 in the descriptor's address field
                            mma_f16(tmem_base + h * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt > 0 || k > 0) ? 1u : 0u);
                        if (h == MH - 1) mma_commit(empty_bar(s));
                    }
                    __syncwarp();
                }
            }
            if (lane == 0) mma_commit(accum_bar);
            __syncwarp();
        }
        if (!ok) {
            if (lane == 0) mma_commit(drain_bar);
            __syncwarp();
            mbar_wait(drain_bar, 0, nullptr, 0);
        }
    } else if (warp < 6) {
        // ---------------- epilogue ----------------
        const int q = warp & 3;
        uint8_t* slots = ring_ptr + STAGES * C::STAGE_BYTES + (warp - 2) * EPI_SLOT_BYTES;
        uint32_t turn = 0;
        bool ok = true;
        uint32_t tcount = 0;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
            int mt, nt;
            tile_coords(tile, MT, NT, mt, nt);
            ok = mbar_wait(accum_bar, tcount & 1, status, ST_EPILOGUE_TIMEOUT);
            tc_fence_after();
            if (!ok) break;
#pragma unroll
            for (int h = 0; h < MH; ++h) {
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + h * BN;
                if (tma_out) {
                    drain_accumulator_tma<DT>(taddr, bn / 32, false, 0, 1, bias, nt * bn, mt * C::BM + h * 128 + q * 32, M, N, slots, turn, omaps,
                                              tmem_empty_bar(h), lane);
                    continue;
                }
                const int row = mt * C::BM + h * 128 + q * 32 + lane;
#pragma unroll 1
                for (int c = 0; c < bn / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c == bn / 32 - 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_empty_bar(h));
                    }
                    store_chunk<DT, 32>(out, bias, r, row, nt * bn + c * 32, M, N, N, 0);
                }
            }
        }
        if (tma_out && lane == 0) bulk_wait_all();         // the stores issued by this warp have been written
    } else {
        // ---------------- dequantisers: W codes -> swizzled operand tile ----------------
        if constexpr (SRC != SRC_RAW) {
            const int t = threadIdx.x - 192;             // 0 .. 255
            const int seg = t & (SEGS - 1);              // 16-element segment of the 64-element K step this thread owns
            const int row_in = t / SEGS;                 // rows row_in + 64 j of the tile, j = 0 .. 3
            const DqConsts dc = dq_consts(wsrc.eb, wsrc.fb, wsrc.fin);
            const int my_tiles = (num_tiles > (int)blockIdx.x) ? (num_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
            const uint32_t total = (uint32_t)my_tiles * (uint32_t)KT;
            constexpr int CODE_BYTES = SRC == SRC_MX ? 1 : 2;
            Staged<SRC> buf[PF];

            // where the next stage to fetch comes from: advanced one K step at a time, so that the per-row addresses are
            // kept as running pointers and the (tile -> column tile) division happens once per tile
            int f_tile = blockIdx.x, f_kt = 0;
            const uint8_t* cptr[ROWS_PER_THREAD];
            const uint8_t* sptr[ROWS_PER_THREAD];
            uint32_t row_ok = 0;
            auto open_tile = [&]() {
                int mt, nt;
                tile_coords(f_tile, MT, NT, mt, nt);
                row_ok = 0;
#pragma unroll
                for (int j = 0; j < ROWS_PER_THREAD; ++j) {
                    const int64_t n = (int64_t)nt * BN + row_in + ROWS_PER_PASS * j;
                    if (n < N) row_ok |= 1u << j;
                    cptr[j] = reinterpret_cast<const uint8_t*>(wsrc.codes) + (n * K + seg * 16) * CODE_BYTES;
                    sptr[j] = wsrc.scales + n * (int64_t)(K / 32) + (seg >> 1);
                }
            };
            auto fetch = [&](Staged<SRC>& b) {                        // loads of one stage's codes; rows past N, columns past K read as zero codes
                const bool k_ok = f_kt * BK + seg * 16 < K;
#pragma unroll
                for (int j = 0; j < ROWS_PER_THREAD; ++j) {
                    const bool in = k_ok && ((row_ok >> j) & 1u);
                    if constexpr (SRC == SRC_MX) {
                        b.codes[j] = in ? __ldg(reinterpret_cast<const uint4*>(cptr[j])) : make_uint4(0u, 0u, 0u, 0u);
                        b.sb[j] = in ? (uint32_t)__ldg(sptr[j]) : 127u;
                    } else {
                        b.lo[j] = in ? __ldg(reinterpret_cast<const uint4*>(cptr[j])) : make_uint4(0u, 0u, 0u, 0u);
                        b.hi[j] = in ? __ldg(reinterpret_cast<const uint4*>(cptr[j]) + 1) : make_uint4(0u, 0u, 0u, 0u);
                    }
                    cptr[j] += BK * CODE_BYTES;
                    sptr[j] += BK / 32;
                }
                if (++f_kt == KT) {
                    f_kt = 0;
                    f_tile += gridDim.x;
                    if (f_tile < num_tiles) open_tile();
                }
            };
            auto expand = [&](uint32_t item, const Staged<SRC>& b, auto expand_mx16) -> bool {
                const int s = item % STAGES;
                if (item >= (uint32_t)STAGES && !mbar_wait(empty_bar(s), ((item / STAGES) & 1) ^ 1, status, ST_DEQUANT_TIMEOUT)) return false;
                uint8_t* tile_b = ring_ptr + s * C::STAGE_BYTES + C::A_BYTES;
#pragma unroll
                for (int j = 0; j < ROWS_PER_THREAD; ++j) {
                    const int r = row_in + ROWS_PER_PASS * j;
                    uint4 v0, v1;
                    if constexpr (SRC == SRC_MX) expand_mx16(b.codes[j], b.sb[j], v0, v1);
                    else { v0 = dequant_mf8<DT>(b.lo[j], dc); v1 = dequant_mf8<DT>(b.hi[j], dc); }
                    // 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r % 8) of that row
                    uint8_t* row = tile_b + r * 128;
                    *reinterpret_cast<uint4*>(row + (((2 * seg) ^ (r & 7)) << 4)) = v0;
                    *reinterpret_cast<uint4*>(row + (((2 * seg + 1) ^ (r & 7)) << 4)) = v1;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> visible to the MMA's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar(s));
                return true;
            };
            auto run = [&](auto expand_mx16) {
                if (total == 0) return;
                open_tile();
#pragma unroll
                for (int d = 0; d < PF; ++d)
                    if ((uint32_t)d < total) fetch(buf[d]);
                bool ok = true;
                for (uint32_t base = 0; base < total && ok; base += PF) {
#pragma unroll
                    for (int d = 0; d < PF; ++d) {
                        const uint32_t item = base + d;
                        if (item < total && ok) {
                            ok = expand(item, buf[d], expand_mx16);
                            if (ok && item + PF < total) fetch(buf[d]);
                        }
                    }
                }
            };
            auto generic = [&](const uint4& w, uint32_t sb, uint4& lo, uint4& hi) {
                lo = dequant_mx8<DT>(w.x, w.y, sb, dc);
                hi = dequant_mx8<DT>(w.z, w.w, sb, dc);
            };
            if constexpr (SRC == SRC_MX && DT == MXQ_BF16) {
                // the five MX element formats get their shifts and masks as immediates
                const int fmt = wsrc.eb * 8 + wsrc.fb;
                if (fmt == 4 * 8 + 3) run([](const uint4& w, uint32_t sb, uint4& lo, uint4& hi) { dequant_mx16_bf16<4, 3>(w, sb, lo, hi); });
                else if (fmt == 5 * 8 + 2) run([](const uint4& w, uint32_t sb, uint4& lo, uint4& hi) { dequant_mx16_bf16<5, 2>(w, sb, lo, hi); });
                else if (fmt == 3 * 8 + 2) run([](const uint4& w, uint32_t sb, uint4& lo, uint4& hi) { dequant_mx16_bf16<3, 2>(w, sb, lo, hi); });
                else if (fmt == 2 * 8 + 3) run([](const uint4& w, uint32_t sb, uint4& lo, uint4& hi) { dequant_mx16_bf16<2, 3>(w, sb, lo, hi); });
                else if (fmt == 2 * 8 + 1) run([](const uint4& w, uint32_t sb, uint4& lo, uint4& hi) { dequant_mx16_bf16<2, 1>(w, sb, lo, hi); });
                else run(generic);
            } else {
                run(generic);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

static bool make_map_16bit(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int box_rows, int dt) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, dt == MXQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims,
              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int DT, int MH, int SRC>
static int launch(const void* x, const void* w_raw, const WSource& wsrc, void* out, const void* bias, int M, int N, int K, int* status,
                  cudaStream_t st) {
    using C = Cfg<MH>;
    static bool attr_done[MAX_DEVICES] = {false};
    const cudaError_t e = raise_smem_limit(dq_gemm_kernel<DT, MH, SRC>, C::SMEM_BYTES, attr_done);
    if (e != cudaSuccess) { set_last_cuda_error(e); return MXQ_ELAUNCH; }
    // Dense operands: the tile width that finishes first by a simple model -- waves of tiles over the SMs times the
    // longer of a stage's MMAs (4 bn cycles for two 128-row halves, 2 bn for one) and its loads at the 69 bytes per clock
    // an SM takes in, plus the epilogue.  256 columns whenever the problem has tiles enough; narrower tiles put more SMs
    // to work on small problems (M = 256, N = 4096: 64 tiles of 64 columns instead of 16 of 256).
    int bn = BN;
    if (SRC == SRC_RAW) {
        const int mt = (M + C::BM - 1) / C::BM, kt = (K + BK - 1) / BK, sms = sm_count();
        double best = 1e300;
        for (int cand = BN; cand >= 64; cand >>= 1) {
            const int tiles = mt * ((N + cand - 1) / cand);
            const double mma = 2.0 * MH * cand, load = (C::A_BYTES + cand * BK * 2) / 69.0;
            const double cost = (double)((tiles + sms - 1) / sms) * (kt * (mma > load ? mma : load) + 24.0 * cand);
            if (cost < 0.97 * best) { best = cost; bn = cand; }          // a narrower tile has to win by 3 %
        }
    }
    CUtensorMap ma, mb;
    if (!make_map_16bit(&ma, x, M, K, C::BM, DT)) return MXQ_ELAUNCH;
    // a quantised W is read with plain loads; the kernel still takes a map argument, so give it a valid one
    if (!make_map_16bit(&mb, SRC == SRC_RAW ? w_raw : x, SRC == SRC_RAW ? N : M, K, SRC == SRC_RAW ? bn : C::BM, DT)) return MXQ_ELAUNCH;
    // instruction descriptor of kind::f16: fp32 accumulate, A/B format (0 fp16, 1 bf16), K-major operands, N >> 3, M >> 4
    const uint32_t fmt = DT == MXQ_BF16 ? 1u : 0u;
    const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const int tiles = ((M + C::BM - 1) / C::BM) * ((N + bn - 1) / bn);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    OutMaps omaps{};
    const int tma_out = make_out_maps(&omaps, out, M, N, N, DT) ? 1 : 0;     // else: stores from registers
    dq_gemm_kernel<DT, MH, SRC><<<grid, THREADS, C::SMEM_BYTES, st>>>(ma, mb, wsrc, out, bias, M, N, K, bn, idesc, status, omaps, tma_out);
    return check_launch();
}

template <int DT, int SRC>
static int launch_mh(const void* x, const void* w_raw, const WSource& wsrc, void* out, const void* bias, int M, int N, int K, int* status,
                     cudaStream_t st) {
    if (M <= 128) return launch<DT, 1, SRC>(x, w_raw, wsrc, out, bias, M, N, K, status, st);
    return launch<DT, 2, SRC>(x, w_raw, wsrc, out, bias, M, N, K, status, st);
}

template <int SRC>
static int launch_dt(int dtype, const void* x, const void* w_raw, const WSource& wsrc, void* out, const void* bias, int M, int N, int K,
                     int* status, cudaStream_t st) {
    if (dtype == MXQ_BF16) return launch_mh<MXQ_BF16, SRC>(x, w_raw, wsrc, out, bias, M, N, K, status, st);
    if (dtype == MXQ_F16) return launch_mh<MXQ_F16, SRC>(x, w_raw, wsrc, out, bias, M, N, K, status, st);
    return MXQ_ESIZE;             // fp32 operands are not a tensor-core format of this kernel
}

static bool dims_ok(int64_t M, int64_t N, int64_t K) { return M > 0 && N > 0 && K > 0 && M <= (1 << 30) && N <= (1 << 30) && K <= (1 << 30); }

}  // namespace dq
}  // namespace mxq

using namespace mxq;

extern "C" int mxq_dense_linear(const void* x, const void* w, int dtype, void* out, const void* bias, int64_t M, int64_t N, int64_t K,
                                int* status, void* stream) {
    if (!x || !w || !out || !dq::dims_ok(M, N, K)) return MXQ_EINVAL;
    if (K % 8 != 0) return MXQ_ESIZE;                                   // row pitch must be a whole number of 16-byte units
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) % 16 != 0) return MXQ_EINVAL;
    return dq::launch_dt<dq::SRC_RAW>(dtype, x, w, dq::WSource{}, out, bias, (int)M, (int)N, (int)K, status, (cudaStream_t)stream);
}

extern "C" int mxq_mxfp_weight_linear(const void* x, int dtype, const uint8_t* w_scales, const uint8_t* w_elements, int exp_bits,
                                      int frac_bits, void* out, const void* bias, int64_t M, int64_t N, int64_t K, int* status,
                                      void* stream) {
    if (!x || !w_scales || !w_elements || !out || !dq::dims_ok(M, N, K)) return MXQ_EINVAL;
    if (exp_bits <= 0 || frac_bits <= 0 || exp_bits + frac_bits > 7) return MXQ_EINVAL;
    if (K % 32 != 0) return MXQ_ESIZE;                                  // 32-element blocks along K
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 != 0 || reinterpret_cast<uintptr_t>(w_elements) % 16 != 0) return MXQ_EINVAL;
    const dq::WSource src{w_elements, w_scales, exp_bits, frac_bits, 1};
    return dq::launch_dt<dq::SRC_MX>(dtype, x, nullptr, src, out, bias, (int)M, (int)N, (int)K, status, (cudaStream_t)stream);
}

extern "C" int mxq_minifloat_weight_linear(const void* x, int dtype, const uint16_t* w_codes, int exp_bits, int frac_bits, int is_finite,
                                           void* out, const void* bias, int64_t M, int64_t N, int64_t K, int* status, void* stream) {
    if (!x || !w_codes || !out || !dq::dims_ok(M, N, K)) return MXQ_EINVAL;
    if (exp_bits <= 0 || frac_bits <= 0 || exp_bits + frac_bits >= 16) return MXQ_EINVAL;
    if (exp_bits > 8 || K % 8 != 0) return MXQ_ESIZE;                   // the decode places the exponent field inside fp32's
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(w_codes)) % 16 != 0) return MXQ_EINVAL;
    const dq::WSource src{w_codes, nullptr, exp_bits, frac_bits, is_finite ? 1 : 0};
    return dq::launch_dt<dq::SRC_MF>(dtype, x, nullptr, src, out, bias, (int)M, (int)N, (int)K, status, (cudaStream_t)stream);
}
