// Building blocks shared by the tensor-core GEMM kernels of libmxq (sm_100a): bounded mbarrier waits,
// TMA and bulk copies, tcgen05 shared-memory descriptors, tensor-memory loads, the epilogue's
// convert-and-store, the tile order of the persistent CTAs, and the per-device host set-up.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/mxq.h"
#include "mxq_codec.h"
#include "mxq_internal.h"

namespace mxq {
namespace tc {

// polls of one bounded wait; a test-only build shortens it so that a wait can be made to run out quickly
#ifdef MXQ_TEST_SPIN_LIMIT
constexpr uint32_t SPIN_LIMIT = MXQ_TEST_SPIN_LIMIT;
#else
constexpr uint32_t SPIN_LIMIT = 1u << 22;
#endif
constexpr int GROUP_M = 8;                       // tiles are dealt in groups of 8 row tiles x all column tiles

// status codes written to the caller's status word when a bounded wait runs out
enum : int { ST_OK = 0, ST_PRODUCER_TIMEOUT = 1, ST_MMA_TIMEOUT = 2, ST_EPILOGUE_TIMEOUT = 3, ST_FORWARD_TIMEOUT = 4, ST_DEQUANT_TIMEOUT = 5 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false (and a code in *status) when the phase never completes
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(32);
    }
    // plain store: the word may live in host memory mapped into the device; any one code is enough
    if (status) *reinterpret_cast<volatile int*>(status) = code;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// shared-memory matrix descriptors (tcgen05): start address, leading/stride byte offsets in 16-byte
// units, version 1, layout type in bits 61..63
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}
constexpr uint32_t LAYOUT_NONE = 0, LAYOUT_SW128 = 2;

__device__ __forceinline__ void tmem_cp_32x128b(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_mxf8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// both operands packed E2M1 nibbles (two per byte in shared memory), K = 64 per instruction, one E8M0 scale per 32
// elements: two scale bytes of each operand row per instruction, picked from the 32-bit column by the descriptor's ids
__device__ __forceinline__ void mma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
// 16 columns into r[0..16) (the last chunk of a tile whose width is an odd multiple of 16)
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// tile index -> (row tile, column tile): groups of GROUP_M row tiles sweep all column tiles, so the
// CTAs running at the same time share a few A tiles and re-use B tiles out of L2
__device__ __forceinline__ void tile_coords(int t, int MT, int NT, int& mt, int& nt) {
    const int per_group = GROUP_M * NT;
    const int g = t / per_group, r = t % per_group;
    const int gm = min(GROUP_M, MT - g * GROUP_M);
    mt = g * GROUP_M + r % gm;
    nt = r / gm;
}

// `out` is a row-major matrix with leading dimension ld; the tile's columns start at column `shift` of it.
// The bias an epilogue adds: N values of the output dtype, or -- `scales` set -- an MXFP-quantised bias as the reference
// stores it (N element-code bytes + one E8M0 scale per 32, src/mase_triton/mxfp/layers.py:85-95), decoded per column
// with the arithmetic and the rounding of compose_mxfp_tensor to the output dtype (src/mase_triton/mxfp/fake.py:62-79).
struct BiasRef {
    const void* ptr;
    const uint8_t* scales;
    int eb, fb;
    __host__ __device__ BiasRef(const void* p = nullptr) : ptr(p), scales(nullptr), eb(0), fb(0) {}
    __host__ __device__ BiasRef(const uint8_t* codes, const uint8_t* s, int e, int f) : ptr(codes), scales(s), eb(e), fb(f) {}
};

template <int OUT_DT>
__device__ __forceinline__ float bias_at(const BiasRef& bias, int col) {
    if (bias.scales != nullptr) {
        const uint32_t code = reinterpret_cast<const uint8_t*>(bias.ptr)[col];
        const uint32_t sb = bias.scales[col >> 5];
        const float v = __uint_as_float(mx_decode(code, __uint_as_float(sb == 0u ? 0x00400000u : (sb << 23)), FmtRT{bias.eb, bias.fb, 1, 0}));
        if constexpr (OUT_DT == MXQ_F32) return v;
        else if constexpr (OUT_DT == MXQ_BF16) return __bfloat162float(__float2bfloat16_rn(v));
        else return __half2float(__float2half_rn(v));
    }
    if constexpr (OUT_DT == MXQ_F32) return reinterpret_cast<const float*>(bias.ptr)[col];
    else if constexpr (OUT_DT == MXQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias.ptr)[col]);
    else return __half2float(reinterpret_cast<const __half*>(bias.ptr)[col]);
}

// W = 32 or 16: columns held in r[0..W)
template <int OUT_DT, int W>
__device__ __forceinline__ void store_chunk(void* __restrict__ out, const BiasRef& bias, const uint32_t (&r)[32],
                                            int row, int col0, int M, int N, int64_t ld, int64_t shift) {
    if (row >= M || col0 >= N) return;
    float v[W];
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = __uint_as_float(r[i]);
    const bool whole = (col0 + W <= N);
    if (bias.ptr != nullptr) {
#pragma unroll
        for (int i = 0; i < W; ++i)
            if (whole || col0 + i < N) v[i] += bias_at<OUT_DT>(bias, col0 + i);
    }
    if constexpr (OUT_DT == MXQ_F32) {
        float* o = reinterpret_cast<float*>(out) + (size_t)row * ld + shift + col0;
        if (whole && ((ld | shift) % 4 == 0)) {
#pragma unroll
            for (int i = 0; i < W; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i) if (col0 + i < N) o[i] = v[i];
        }
    } else {
        uint32_t pk[W / 2];
#pragma unroll
        for (int i = 0; i < W; i += 2) {
            if constexpr (OUT_DT == MXQ_BF16) { const __nv_bfloat162 h = __floats2bfloat162_rn(v[i], v[i + 1]); pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h); }
            else { const __half2 h = __floats2half2_rn(v[i], v[i + 1]); pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h); }
        }
        uint16_t* o = reinterpret_cast<uint16_t*>(out) + (size_t)row * ld + shift + col0;
        if (whole && ((ld | shift) % 8 == 0)) {
#pragma unroll
            for (int i = 0; i < W / 2; i += 4) *reinterpret_cast<uint4*>(o + 2 * i) = make_uint4(pk[i], pk[i + 1], pk[i + 2], pk[i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < W; ++i) if (col0 + i < N) o[i] = (uint16_t)(pk[i >> 1] >> (16 * (i & 1)));
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Asynchronous epilogue: tensor memory -> registers -> a small shared-memory staging slot -> TMA store.
// The warp never waits for global memory: it hands the accumulator back to the MMA warp as soon as its
// last tcgen05.ld has completed, and the bulk tensor stores drain behind it.  Two tcgen05.ld are kept
// in flight (the next chunk is requested before the current one is converted).  Rows past M and
// columns past N are clipped by the tensor map, so no bounds logic is needed.
// ------------------------------------------------------------------------------------------------
constexpr int EPI_SLOT_BYTES = 4096;             // staging per epilogue warp: two 2 KiB slots (16-bit out) or one 4 KiB slot (fp32)

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// the two output maps of a kernel: `main` = boxes of 64 bytes x 32 rows with the 64-byte swizzle, `tail` = boxes of
// 16 columns x 32 rows, unswizzled (16-bit outputs whose tile width is an odd multiple of 16)
struct OutMaps { CUtensorMap main, tail; };


// one chunk (W = 32 or 16 accumulator columns of this lane's row) -> staging slot -> TMA store at (col0, row0 + lane)
template <int OUT_DT, int W>
__device__ __forceinline__ void emit_chunk_tma(const uint32_t (&r)[32], const BiasRef& bias, int col0, int row0, int N, uint8_t* slot,
                                               const OutMaps& maps, int lane) {
    float v[W];
#pragma unroll
    for (int i = 0; i < W; ++i) v[i] = __uint_as_float(r[i]);
    if (bias.ptr != nullptr) {
#pragma unroll
        for (int i = 0; i < W; ++i) if (col0 + i < N) v[i] += bias_at<OUT_DT>(bias, col0 + i);
    }
    const uint32_t sw = (uint32_t)((lane >> 1) & 3);                 // 64-byte swizzle: 16-byte unit u of row r sits at unit u ^ ((r >> 1) & 3)
    if constexpr (OUT_DT == MXQ_F32) {
        // W floats = W / 16 boxes of 16 columns (64 bytes per row)
#pragma unroll
        for (int b = 0; b < W / 16; ++b) {
            uint8_t* box = slot + b * 2048 + lane * 64;
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u)
                *reinterpret_cast<float4*>(box + ((u ^ sw) << 4)) = make_float4(v[16 * b + 4 * u], v[16 * b + 4 * u + 1], v[16 * b + 4 * u + 2], v[16 * b + 4 * u + 3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < W / 16; ++b) tma_store_2d(&maps.main, col0 + 16 * b, row0, smem_u32(slot + b * 2048));
            bulk_commit();
        }
    } else {
        uint32_t pk[W / 2];
#pragma unroll
        for (int i = 0; i < W; i += 2) {
            if constexpr (OUT_DT == MXQ_BF16) { const __nv_bfloat162 h = __floats2bfloat162_rn(v[i], v[i + 1]); pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h); }
            else { const __half2 h = __floats2half2_rn(v[i], v[i + 1]); pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h); }
        }
        if constexpr (W == 32) {
            uint8_t* box = slot + lane * 64;
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u)
                *reinterpret_cast<uint4*>(box + ((u ^ sw) << 4)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        } else {
            uint8_t* box = slot + lane * 32;                         // 16 columns: 32 bytes per row, unswizzled
#pragma unroll
            for (uint32_t u = 0; u < 2; ++u)
                *reinterpret_cast<uint4*>(box + (u << 4)) = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(W == 32 ? &maps.main : &maps.tail, col0, row0, smem_u32(slot));
            bulk_commit();
        }
    }
}

// This warp's share of one accumulator: chunks first, first + step, ... of the n_chunks 32-column chunks (the last
// one 16 wide when tail16).  `taddr` = tensor-memory address of column 0 of the accumulator in this warp's lane
// quadrant; `slots` = this warp's EPI_SLOT_BYTES of staging (1024-byte aligned); `turn` alternates the two slots.
// Arrives on `release_bar` right after the last tensor-memory read.
template <int OUT_DT>
__device__ __forceinline__ void drain_accumulator_tma(uint32_t taddr, int n_chunks, bool tail16, int first, int step, const BiasRef& bias,
                                                      int col_base, int row0, int M, int N, uint8_t* slots, uint32_t& turn, const OutMaps& maps,
                                                      uint32_t release_bar, int lane) {
    constexpr bool TWO_SLOTS = OUT_DT != MXQ_F32;
    uint32_t ra[32], rb[32];
    auto request = [&](uint32_t (&r)[32], int c) {
        if (tail16 && c == n_chunks - 1) tmem_ld_32x32b_x16(taddr + c * 32, r);
        else tmem_ld_32x32b_x32(taddr + c * 32, r);
    };
    auto release = [&]() {                      // no tensor-memory read of this warp is outstanding any more
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(release_bar);
    };
    auto emit = [&](const uint32_t (&r)[32], int c) {
        if (row0 >= M || col_base + c * 32 >= N) return;             // nothing of this box lies inside the matrix
        // the slot about to be written must have been read by the store issued from it earlier
        if (lane == 0) { if constexpr (TWO_SLOTS) bulk_wait_read<1>(); else bulk_wait_read<0>(); }
        __syncwarp();
        uint8_t* slot = slots + (TWO_SLOTS ? (turn & 1u) * 2048u : 0u);
        ++turn;
        if (tail16 && c == n_chunks - 1) emit_chunk_tma<OUT_DT, 16>(r, bias, col_base + c * 32, row0, N, slot, maps, lane);
        else emit_chunk_tma<OUT_DT, 32>(r, bias, col_base + c * 32, row0, N, slot, maps, lane);
    };
    int c = first;
    if (c >= n_chunks) { release(); return; }
    request(ra, c);
    while (c < n_chunks) {
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int c1 = c + step;
        if (c1 < n_chunks) request(rb, c1); else release();
        emit(ra, c);
        if (c1 >= n_chunks) break;
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int c2 = c1 + step;
        if (c2 < n_chunks) request(ra, c2); else release();
        emit(rb, c1);
        c = c2;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Output maps of the asynchronous epilogue for a row-major [M, N] matrix of dtype `dt` with `ld` elements per row.
// False when the matrix cannot be described (base or row pitch not a multiple of 16 bytes): the caller then uses
// the epilogue that stores from registers.
static bool make_out_maps(OutMaps* maps, void* out, int64_t M, int64_t N, int64_t ld, int dt) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const int esz = dt == MXQ_F32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(out) % 16 != 0 || (ld * esz) % 16 != 0) return false;
    const CUtensorMapDataType type = dt == MXQ_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : (dt == MXQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)(ld * esz)};
    const cuuint32_t estr[2] = {1, 1};
    const cuuint32_t box_main[2] = {(cuuint32_t)(64 / esz), 32};
    const cuuint32_t box_tail[2] = {16, 32};
    if (fn(&maps->main, type, 2, out, dims, strides, box_main, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
    return fn(&maps->tail, type, 2, out, dims, strides, box_tail, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              dt == MXQ_F32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Unswizzled map of a row-major [M, N] matrix (`ld` elements per row) with boxes of box_cols x box_rows elements: whole
// row segments of a tile, for copies that only pass through shared memory.
static bool make_rows_map(CUtensorMap* map, void* base, int64_t M, int64_t N, int64_t ld, int dt, int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const int esz = dt == MXQ_F32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || (ld * esz) % 16 != 0 || box_cols > 256 || (box_cols * esz) % 16 != 0) return false;
    const CUtensorMapDataType type = dt == MXQ_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : (dt == MXQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)(ld * esz)};
    const cuuint32_t estr[2] = {1, 1};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    return fn(map, type, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per-device facts and one-time set-up (a process may drive several GPUs): the SM count, and for every
// kernel instantiation whether its dynamic shared-memory limit has been raised on that device.
constexpr int MAX_DEVICES = 64;
static std::mutex g_dev_mu;   // (one per translation unit that includes this header; each guards its own tables)

static int current_device() {
    int dev = 0;
    return (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < MAX_DEVICES) ? dev : -1;
}

static int sm_count() {
    static int n[MAX_DEVICES] = {0};
    const int dev = current_device();
    if (dev < 0) return 148;
    std::lock_guard<std::mutex> lock(g_dev_mu);
    if (n[dev] == 0 && (cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n[dev] <= 0)) n[dev] = 148;
    return n[dev];
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device (per-context) attribute
template <class Kernel>
static cudaError_t raise_smem_limit(Kernel kernel, int bytes, bool (&done)[MAX_DEVICES]) {
    const int dev = current_device();
    if (dev < 0) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_dev_mu);
    if (done[dev]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}

}  // namespace tc
}  // namespace mxq
