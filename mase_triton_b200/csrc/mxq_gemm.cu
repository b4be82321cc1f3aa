// Block-scaled MX GEMM for sm_100a: out[M,N] = dequant(A)[M,K] * dequant(B)[N,K]^T (+ bias).
//
// Both operands are MXFP tensors with 32-element blocks along K.  The kernel feeds the 5th-gen
// tensor cores directly with the quantised data:
//   * operand codes (one byte per element, OCP E4M3 or E5M2 as the hardware reads them) are staged
//     by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a shared-memory ring;
//   * the E8M0 block scales of a (tile rows) x 128(K) slab are 512-byte chunks brought in with a
//     bulk copy and moved shared -> tensor memory with tcgen05.cp;
//   * one elected thread issues tcgen05.mma.kind::mxf8f6f4.block_scale (M=128, N=bn, K=32); the
//     fp32 accumulators (one or two 128-lane x bn-column blocks) live in tensor memory;
//   * epilogue warps read them back with tcgen05.ld, add the bias and convert; eight of them stage 32 x 32 chunks in
//     shared memory and store with TMA (asynchronous: tensor memory goes back to the MMA warp before the stores land),
//     or four store from registers when the output cannot be described by a tensor map.
// Variants of the same kernel (template flags): the right operand as dense 6- / 4-bit codes that the copy engine
// spreads to bytes in shared memory; both operands as packed E2M1 nibbles on tcgen05.mma.kind::mxf4 (K = 64 per
// instruction, twice the arithmetic per byte staged); the all-gather of a column-parallel linear done by an extra
// warp that forwards every finished half tile to the peers with TMA.
// The CTA tile is 256 x bn (128 x bn when M <= 128) with bn = 224 by default: two accumulators fill
// the 512 TMEM columns and raise the flops per byte pulled from L2, which is what bounds this kernel.
// bn is a run-time value (a multiple of 16, at most 224) fixed when the right operand is packed, so a
// narrow layer can use the width that wastes the least padded work (1024 features: 5 tiles of 208).  CTAs are
// persistent (one per SM, tiles dealt round-robin in an L2-friendly order): the TMA producer runs
// ahead into the next tile while the epilogue drains tensor memory.
// Warp roles: warp 0 = TMA producer, warp 1 = MMA issuer (also owns the TMEM allocation),
// warps 2.. = epilogue (then the forwarding / copy-out warps of the gather-fused forms).  Every wait on an mbarrier is bounded; a wait that runs out records a
// code in the caller's status word and the CTA unwinds (TMEM is freed) instead of spinning.
//
// Operand layout in HBM (produced by the pack kernel in this file):
//   codes : [rows, K] bytes, K contiguous
//   sf    : [ceil(rows/T)][ceil(K/128)][2][512] bytes, T = 256 for the A operand and bn for B; chunk
//           h holds tile-local rows 128h .. 128h+127; inside a chunk the scale of local row r and
//           K block b (0..3) sits at (r % 32) * 16 + (r / 32) * 4 + b -- the order tcgen05.cp
//           (32x128b.warpx4) expects.
#include <cmath>

#include "mxq_codec.h"
#include "mxq_tc.cuh"

namespace mxq {
namespace gemm {

using namespace tc;

constexpr int BN_MAX = 224, BK = 128;            // widest right-operand tile (columns of the CTA tile)
constexpr int A_TILE_ROWS = 256;                 // rows per scale-factor tile of the A operand
constexpr int B_BYTES = BN_MAX * BK;             // 28 KiB reserved per stage, bn * 128 bytes of it used
constexpr int SF_REGION = 2048;                  // A chunks (<= 1024) + B chunks (1024) of one 128-element K step
constexpr int BAR_BYTES = 256;
constexpr int TMEM_COLS = 512;
constexpr int SFA_COL = 448, SFB_COL = 456;      // accumulators occupy columns [0, 448)
constexpr int SFA4_COL = 448, SFB4_COL = 464;    // 4-bit x 4-bit kernel: a stage holds two 128-element K steps of scales (8 columns each per operand)
constexpr int THREADS = 192;                     // TMA producer, MMA issuer, four epilogue warps (epilogue that stores from registers)
constexpr int EPI_TMA_WARPS = 8;                 // epilogue warps of the asynchronous (TMA-store) epilogue: two per TMEM lane quadrant
constexpr int THREADS_TMA = 64 + EPI_TMA_WARPS * 32;

// MXF4: both operands are packed E2M1 nibbles (kind::mxf4): a stage's 128 bytes per row are 256 elements of K, so it
// carries the scales of two 128-element K steps
template <int MH, bool MXF4 = false> struct Cfg {
    static constexpr int BM = 128 * MH;
    static constexpr int A_BYTES = BM * BK;
    static constexpr int K_PER_STAGE = MXF4 ? 2 * BK : BK;          // elements of K per stage
    static constexpr int SF_STEPS = MXF4 ? 2 : 1;                   // 128-element K steps of scales per stage
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_STEPS * SF_REGION;       // multiple of 1024
    static constexpr int STAGES = MH == 2 ? 3 : 4;
    static constexpr int TX_FIXED = A_BYTES + SF_STEPS * (MH * 512 + 1024);       // + the bytes of bn * BK codes of the right operand
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;   // + slack to align the ring
    static constexpr int SMEM_BYTES_TMA = SMEM_BYTES + EPI_TMA_WARPS * EPI_SLOT_BYTES;   // + staging of the asynchronous epilogue
};
constexpr int FWD_BUF_BYTES = 3584;              // one box of the forwarding warp: a few rows of a tile (8 x 224 16-bit values)
constexpr int FWD_BUFS = 2;                      // boxes with shared memory of their own; narrower tiles leave room for more:
constexpr int FWD_BUFS_MAX = 6;                  // the unused end of each stage's B region (bn < BN_MAX) holds one box

// Destinations of the gather-fused kernel: the [M, N] result goes, at column offset col0 of a
// row-major matrix with leading dimension ld, to every pointer in ptr[0..n): ptr[self] is this GPU's
// own output, the others are the peers' outputs mapped into this process.
constexpr int MAX_DEST = 8;
struct OutSpec {
    void* ptr[MAX_DEST];
    int n, self;
    int64_t ld, col0;
};
constexpr int FWD_WARPS = 4;                     // copy-out warps of the gather-fused kernel
constexpr int FWD_UNROLL = 4;                    // 16-byte units each copy-out lane keeps in flight
constexpr int STORED_BAR_OFF = 128, ACK_BAR_OFF = 144;   // two barriers each (one per accumulator), inside the BAR_BYTES region past the pipeline barriers
constexpr int FWD_BAR_OFF = 160;                 // one barrier per forwarding buffer

// Tensor maps of the gather-fused kernel whose forwarding is done by the copy engine: `src` reads this GPU's own
// output region back (boxes of box_rows rows x the tile width), dst[d] writes the same box into destination d.
struct FwdMaps {
    CUtensorMap src;
    CUtensorMap dst[MAX_DEST];
    int n, self, box_rows, box_bytes;
    int n_bufs;                                  // FWD_BUFS, or FWD_BUFS + the ring's stages when a box fits behind the B tile of a stage
};


// Copy-out of the gather-fused kernel: one tile of this GPU's output (just written by the epilogue
// warps, still in L2) is read back and stored into every peer's output, 16 bytes per lane, whole
// row segments per warp instruction.
template <int OUT_DT>
__device__ __forceinline__ void forward_tile(const OutSpec& outs, int fw, int lane, int row0, int rows, int col0, int cols) {
    constexpr int ESZ = OUT_DT == MXQ_F32 ? 4 : 2;
    constexpr int EPU = 16 / ESZ;                          // elements per 16-byte unit
    const int upr = cols / EPU;                            // units per row segment (cols is a multiple of EPU)
    const int total = rows * upr;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(outs.ptr[outs.self]);
    constexpr int UNROLL = FWD_UNROLL;
    for (int base = fw * 32 + lane; base < total; base += FWD_WARPS * 32 * UNROLL) {
        uint4 v[UNROLL];
        size_t off[UNROLL];
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            const int flat = base + j * FWD_WARPS * 32;
            if (flat < total) {
                const int row = flat / upr, u = flat - row * upr;
                off[j] = ((size_t)(row0 + row) * outs.ld + outs.col0 + col0 + u * EPU) * ESZ;
                v[j] = __ldcg(reinterpret_cast<const uint4*>(src + off[j]));
            }
        }
#pragma unroll
        for (int j = 0; j < UNROLL; ++j) {
            if (base + j * FWD_WARPS * 32 < total) {
                for (int d = 0; d < outs.n; ++d)
                    if (d != outs.self) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(outs.ptr[d]) + off[j]) = v[j];
            }
        }
    }
}

// OUT_DT: MXQ_F32 / MXQ_BF16 / MXQ_F16; MH: 128-row accumulators per CTA tile;
// EPI: EPI_REGS = four warps convert and store from registers, EPI_TMA = eight warps stage through shared memory and
//      store with TMA (asynchronous: tensor memory is handed back without waiting for global memory),
//      EPI_GATHER = EPI_REGS plus the copy-out warps of the gather-fused kernel;
// bn: columns of the CTA tile (multiple of 16, <= BN_MAX) = rows per scale-factor tile of the right operand
//      EPI_GATHER_TMA = EPI_TMA plus one forwarding warp: a single thread reads each finished half tile of the local
//      output back into small shared-memory boxes with TMA loads and stores every box to all peers with TMA stores
enum : int { EPI_REGS = 0, EPI_TMA = 1, EPI_GATHER = 2, EPI_GATHER_TMA = 3 };
template <int EPI> constexpr int kernel_threads() {
    return EPI == EPI_TMA ? THREADS_TMA : EPI == EPI_GATHER_TMA ? THREADS_TMA + 32 : THREADS + (EPI == EPI_GATHER ? FWD_WARPS * 32 : 0);
}
template <int EPI, int MH, bool MXF4 = false> constexpr int kernel_smem() {
    using C = Cfg<MH, MXF4>;
    return EPI == EPI_TMA ? C::SMEM_BYTES_TMA : EPI == EPI_GATHER_TMA ? C::SMEM_BYTES_TMA + FWD_BUFS * FWD_BUF_BYTES : C::SMEM_BYTES;
}

template <int OUT_DT, int MH, int EPI, bool MXF4 = false>
__global__ void __launch_bounds__(kernel_threads<EPI>(), 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, void* __restrict__ out,
               const BiasRef bias, int M, int N, int K, int bn, uint32_t idesc_base, int* status,
               const __grid_constant__ OutSpec outs, const __grid_constant__ OutMaps omaps, const __grid_constant__ FwdMaps fmaps) {
    using C = Cfg<MH, MXF4>;
    constexpr int STAGES = C::STAGES;
    constexpr bool MULTI = EPI == EPI_GATHER;
    constexpr bool TMA_EPI = EPI == EPI_TMA || EPI == EPI_GATHER_TMA;
    constexpr int EPI_WARPS = TMA_EPI ? EPI_TMA_WARPS : 4;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;                    // 1024-aligned operand ring
    uint8_t* ring_ptr = smem_raw + (ring - raw);
    // ring | staging slots of the asynchronous epilogue | boxes of the forwarding warp (EPI_GATHER_TMA) | barriers
    constexpr uint32_t SLOTS = TMA_EPI ? EPI_TMA_WARPS * EPI_SLOT_BYTES : 0;
    constexpr uint32_t STAGING = SLOTS + (EPI == EPI_GATHER_TMA ? FWD_BUFS * FWD_BUF_BYTES : 0);
    const uint32_t bars = ring + STAGES * C::STAGE_BYTES + STAGING;  // full[S], empty[S], accum_full, tmem_empty[2], drain, tmem slot
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ring_ptr + STAGES * C::STAGE_BYTES + STAGING + 8 * (2 * STAGES + 4));
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (2 * STAGES);
    auto tmem_empty_bar = [&](int h) { return bars + 8u * (2 * STAGES + 1 + h); };   // one per accumulator
    const uint32_t drain_bar = bars + 8u * (2 * STAGES + 3);                         // used only when the MMA warp unwinds
    auto stored_bar = [&](int h) { return bars + STORED_BAR_OFF + 8u * h; };
    auto ack_bar = [&](int h) { return bars + ACK_BAR_OFF + 8u * h; };
    auto fwd_bar = [&](int b) { return bars + FWD_BAR_OFF + 8u * b; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = (K + C::K_PER_STAGE - 1) / C::K_PER_STAGE;       // stages per tile
    const int KT128 = (K + BK - 1) / BK;                            // scale chunks per row tile
    const int MT = (M + C::BM - 1) / C::BM, NT = (N + bn - 1) / bn;
    const int num_tiles = MT * NT;
    // the right operand's copy counts the bytes it reads: dense 6-bit (formats 3, 4) and 4-bit (5) codes are narrower
    const uint32_t b_fmt = (idesc_base >> 10) & 7u;
    const uint32_t b_bits = b_fmt <= 1u ? 8u : (b_fmt == 5u ? 4u : 6u);
    // (packed nibbles of the 4-bit x 4-bit kernel fill the 128 bytes per row: 256 codes)
    const uint32_t tx_bytes = (uint32_t)C::TX_FIXED + (MXF4 ? (uint32_t)(bn * BK) : (uint32_t)(bn * BK) * b_bits / 8u);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        mbar_init(tmem_empty_bar(0), EPI_WARPS);                     // one arrival per epilogue warp
        mbar_init(tmem_empty_bar(1), EPI_WARPS);
        mbar_init(drain_bar, 1);
        if constexpr (MULTI) {
            for (int h = 0; h < 2; ++h) {
                mbar_init(stored_bar(h), 4);                         // epilogue warps: "this accumulator's rows are in local memory"
                mbar_init(ack_bar(h), FWD_WARPS);                    // copy-out warps: "seen it"
            }
        }
        if constexpr (EPI == EPI_GATHER_TMA) {
            for (int h = 0; h < 2; ++h) {
                mbar_init(stored_bar(h), EPI_WARPS);                 // epilogue warps: "my stores of this half tile have been written"
                mbar_init(ack_bar(h), 1);                            // the forwarding thread: "seen it"
            }
            for (int b = 0; b < FWD_BUFS_MAX; ++b) mbar_init(fwd_bar(b), 1);
        }
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
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            int mt, nt;
            tile_coords(tile, MT, NT, mt, nt);
            // A scale tiles are 256 rows (2 chunks); a 128-row CTA tile uses one of the two chunks
            const uint8_t* sfa_tile = (MH == 2) ? sfa + (size_t)mt * KT128 * 1024 : sfa + (size_t)(mt >> 1) * KT128 * 1024 + (mt & 1) * 512;
            const uint8_t* sfb_tile = sfb + (size_t)nt * KT128 * 1024;
            for (int kt = 0; kt < KT && ok; ++kt, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES) ok = mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, status, ST_PRODUCER_TIMEOUT);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t st = ring + s * C::STAGE_BYTES;
                    mbar_expect_tx(full_bar(s), tx_bytes);
                    tma_load_2d(st, &map_a, kt * C::K_PER_STAGE, mt * C::BM, full_bar(s));
                    tma_load_2d(st + C::A_BYTES, &map_b, kt * C::K_PER_STAGE, nt * bn, full_bar(s));
#pragma unroll
                    for (int c = 0; c < C::SF_STEPS; ++c) {
                        const size_t chunk = (size_t)(kt * C::SF_STEPS + c) * 1024;
                        bulk_load(st + C::A_BYTES + B_BYTES + c * SF_REGION, sfa_tile + chunk, MH * 512, full_bar(s));
                        bulk_load(st + C::A_BYTES + B_BYTES + c * SF_REGION + 1024, sfb_tile + chunk, 1024, full_bar(s));
                    }
                }
                __syncwarp();
            }
        }
        // Every copy this warp started must have landed before the CTA gives its shared memory back.  In a
        // run that went well the MMA warp has consumed them all and these waits return at once; after a
        // wait that ran out they (bounded, too) cover the copies nobody consumed.
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
                const uint32_t sf = st + C::A_BYTES + B_BYTES;
                const uint64_t b_desc = smem_desc(st + C::A_BYTES, 16, 1024, LAYOUT_SW128);
#pragma unroll
                for (int h = 0; h < MH; ++h) {
                    // the first MMA into an accumulator overwrites it: the epilogue must have drained that
                    // accumulator of the previous tile (accumulator 1 is still being read while 0 refills)
                    if (kt == 0 && tcount > 0 && ok) ok = mbar_wait(tmem_empty_bar(h), (tcount - 1) & 1, status, ST_MMA_TIMEOUT);
                    tc_fence_after();
                    if (ok && lane == 0) {
                        constexpr int SA = MXF4 ? SFA4_COL : SFA_COL, SB = MXF4 ? SFB4_COL : SFB_COL;
                        if (h == 0) {
#pragma unroll
                            for (int c = 0; c < C::SF_STEPS; ++c) {             // 8 columns per operand and 128-element K step
#pragma unroll
                                for (int hh = 0; hh < MH; ++hh)
                                    tmem_cp_32x128b(tmem_base + SA + 8 * c + 4 * hh, smem_desc(sf + c * SF_REGION + 512 * hh, 0, 128, LAYOUT_NONE));
                                tmem_cp_32x128b(tmem_base + SB + 8 * c, smem_desc(sf + c * SF_REGION + 1024, 0, 128, LAYOUT_NONE));
                                tmem_cp_32x128b(tmem_base + SB + 8 * c + 4, smem_desc(sf + c * SF_REGION + 1536, 0, 128, LAYOUT_NONE));
                            }
                        }
                        const uint64_t a_desc = smem_desc(st + h * 16384, 16, 1024, LAYOUT_SW128);
#pragma unroll
                        for (uint32_t k = 0; k < BK / 32; ++k) {
                            // +32 bytes along K inside the 128-byte swizzle span = +2 in the address field
                            if constexpr (MXF4) {
                                // 64 elements per instruction: scale bytes (0, 1) or (2, 3) of the column set of K step k / 2
                                const uint32_t id = (k & 1u) * 2u;
                                const uint32_t idesc = idesc_base | (id << 29) | (id << 4);
                                mma_mxf4(tmem_base + h * BN_MAX, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + SA + 8 * (k >> 1) + 4 * h,
                                         tmem_base + SB + 8 * (k >> 1), (kt > 0 || k > 0) ? 1u : 0u);
                            } else {
                                // scale-factor byte k of each 32-bit TMEM column
                                const uint32_t idesc = idesc_base | (k << 29) | (k << 4);
                                mma_mxf8f6f4(tmem_base + h * BN_MAX, a_desc + 2 * k, b_desc + 2 * k, idesc, tmem_base + SA + 4 * h,
                                             tmem_base + SB, (kt > 0 || k > 0) ? 1u : 0u);
                            }
                        }
                        if (h == MH - 1) mma_commit(empty_bar(s));     // frees the stage once these MMAs have read it
                    }
                    __syncwarp();
                }
            }
#ifndef MXQ_TEST_DROP_ACCUM_COMMIT
            if (lane == 0) mma_commit(accum_bar);         // accumulators of this tile complete (or unwinding)
#endif
            __syncwarp();
        }
#ifdef MXQ_TEST_DROP_ACCUM_COMMIT
        ok = false;                                       // test-only build: nothing above tracked the MMAs' completion
#endif
        if (!ok) {
            // unwinding after a wait that ran out: the MMAs already issued must finish before tensor memory is freed
            if (lane == 0) mma_commit(drain_bar);
            __syncwarp();
            mbar_wait(drain_bar, 0, nullptr, 0);
        }
    } else if (TMA_EPI && warp < 2 + EPI_WARPS) {
        // ---------------- epilogue: TMEM -> registers -> shared staging -> TMA store ----------------
        if constexpr (TMA_EPI) {
            const int e = warp - 2, q = warp & 3;          // two warps per TMEM lane quadrant; each takes every other chunk
            const int grp = e >> 2;
            const int n_chunks = (bn + 31) >> 5;
            const bool tail16 = (bn & 16) != 0;
            uint8_t* slots = ring_ptr + STAGES * C::STAGE_BYTES + e * EPI_SLOT_BYTES;
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
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + h * BN_MAX;
                    // the group that took the even chunks of accumulator 0 takes the odd ones of accumulator 1
                    drain_accumulator_tma<OUT_DT>(taddr, n_chunks, tail16, (grp ^ h) & 1, 2, bias, nt * bn, mt * C::BM + h * 128 + q * 32, M, N,
                                                  slots, turn, omaps, tmem_empty_bar(h), lane);
                    if constexpr (EPI == EPI_GATHER_TMA) {
                        // tell the forwarding thread that this warp's part of half tile h has been written to local
                        // memory; it must have picked up the same half of the previous tile first (one tile of slack)
                        if (lane == 0) bulk_wait_all();
                        if (tcount > 0) ok = mbar_wait(ack_bar(h), (tcount - 1) & 1, status, ST_EPILOGUE_TIMEOUT);
                        __syncwarp();
                        if (lane == 0) mbar_arrive(stored_bar(h));
                    }
                }
            }
            if (lane == 0) bulk_wait_all();                // the stores issued by this warp have been written
        }
    } else if (EPI == EPI_GATHER_TMA) {
        // ---------------- gather-fused kernel, forwarding by the copy engine: local output -> peers ----------------
        if constexpr (EPI == EPI_GATHER_TMA) {
            if (lane == 0) {
                const uint32_t own = ring + STAGES * C::STAGE_BYTES + SLOTS;
                // box b: the first FWD_BUFS have memory of their own, the others sit behind the bn rows of a stage's B tile
                auto buf = [&](uint32_t b) {
                    return b < (uint32_t)FWD_BUFS ? own + b * FWD_BUF_BYTES : ring + (b - FWD_BUFS) * C::STAGE_BYTES + C::A_BYTES + (uint32_t)(bn * BK);
                };
                const uint32_t NB = (uint32_t)fmaps.n_bufs;
                const int ahead = NB >= 3u ? (int)NB - 2 : 1;           // loads requested beyond the box being sent
                const int FR = fmaps.box_rows;
                bool ok = true;
                uint32_t tcount = 0, loaded = 0, sent = 0;          // boxes whose load has been started / whose stores have been issued
                for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
                    int mt, nt;
                    tile_coords(tile, MT, NT, mt, nt);
                    for (int h = 0; h < MH && ok; ++h) {
                        ok = mbar_wait(stored_bar(h), tcount & 1, status, ST_FORWARD_TIMEOUT);
                        if (!ok) break;
                        mbar_arrive(ack_bar(h));
                        asm volatile("fence.proxy.async.global;" ::: "memory");      // the half tile was written through the async proxy by other threads
                        const int row0 = mt * C::BM + h * 128;
                        const int rows = min(128, M - row0);
                        if (rows <= 0) continue;
                        const int boxes = (rows + FR - 1) / FR;
                        int issued = 0;                              // boxes of this half tile whose load has been requested
                        for (int i = 0; i < boxes && ok; ++i) {
                            while (issued < boxes && issued <= i + ahead) {
                                const uint32_t b = loaded % NB;
                                // The stores that read this box NB boxes ago must have finished reading it.  Groups retire in
                                // order and at most `ahead` + 1 boxes separate this load from the last store issued, so
                                // "all but the newest group" (all groups, with two boxes) covers it.
                                if (loaded >= NB) { if (NB >= 3u) bulk_wait_read<1>(); else bulk_wait_read<0>(); }
                                mbar_expect_tx(fwd_bar(b), (uint32_t)fmaps.box_bytes);
                                tma_load_2d(buf(b), &fmaps.src, nt * bn, row0 + issued * FR, fwd_bar(b));
                                ++loaded;
                                ++issued;
                            }
                            const uint32_t b = sent % NB;
                            ok = mbar_wait(fwd_bar(b), (sent / NB) & 1, status, ST_FORWARD_TIMEOUT);
                            if (!ok) break;
                            for (int d = 0; d < fmaps.n; ++d)
                                if (d != fmaps.self) tma_store_2d(&fmaps.dst[d], nt * bn, row0 + i * FR, buf(b));
                            bulk_commit();
                            ++sent;
                        }
                    }
                }
                // after a wait that ran out: a load may still be in flight into this CTA's shared memory
                for (; sent < loaded; ++sent) mbar_wait(fwd_bar(sent % NB), (sent / NB) & 1, status, ST_FORWARD_TIMEOUT);
                bulk_wait_all();                               // every box has been written to every peer
            }
            __syncwarp();
        }
    } else if (!TMA_EPI && warp < 6) {
        // ---------------- epilogue: TMEM -> registers -> global ----------------
        const int q = warp & 3;                            // TMEM lane quadrant this warp may access
        const int full_chunks = bn >> 5;                   // 32-column chunks, then possibly one of 16 columns
        const bool tail16 = (bn & 16) != 0;
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
                const int row = mt * C::BM + h * 128 + q * 32 + lane;
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + h * BN_MAX;
                void* dst = MULTI ? outs.ptr[outs.self] : out;
                const int64_t ld = MULTI ? outs.ld : (int64_t)N, shift = MULTI ? outs.col0 : 0;
#pragma unroll 1
                for (int c = 0; c < full_chunks; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c == full_chunks - 1 && !tail16) {
                        // last read of this accumulator: hand it back to the MMA warp
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tmem_empty_bar(h));
                    }
                    store_chunk<OUT_DT, 32>(dst, bias, r, row, nt * bn + c * 32, M, N, ld, shift);
                }
                if (tail16) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x16(taddr + full_chunks * 32, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(tmem_empty_bar(h));
                    store_chunk<OUT_DT, 16>(dst, bias, r, row, nt * bn + full_chunks * 32, M, N, ld, shift);
                }
                if constexpr (MULTI) {
                    // tell the copy-out warps that this warp's rows of accumulator h are in local memory; they
                    // must have picked up the same accumulator of the previous tile first (one tile of slack)
                    if (tcount > 0) ok = mbar_wait(ack_bar(h), (tcount - 1) & 1, status, ST_EPILOGUE_TIMEOUT);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(stored_bar(h));
                }
            }
        }
    } else {
        // ---------------- gather-fused kernel only: copy-out warps, local output -> peers ----------------
        if constexpr (MULTI) {
            const int fw = warp - 6;
            bool ok = true;
            uint32_t tcount = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
                int mt, nt;
                tile_coords(tile, MT, NT, mt, nt);
                for (int h = 0; h < MH && ok; ++h) {                  // 128 rows at a time, as the epilogue finishes them
                    ok = mbar_wait(stored_bar(h), tcount & 1, status, ST_FORWARD_TIMEOUT);
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(ack_bar(h));
                    const int row0 = mt * C::BM + h * 128;
                    if (row0 < M) forward_tile<OUT_DT>(outs, fw, lane, row0, min(128, M - row0), nt * bn, min(bn, N - nt * bn));
                }
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

// ------------------------------------------------------------------------------------------------
// operand packing: reference codes + scales -> hardware codes + scale chunks
// ------------------------------------------------------------------------------------------------
struct PackTables {
    uint8_t plain[256];     // reference code -> hardware code of the same value
    uint8_t halved[256];    // reference code -> hardware code of value / 2 (round half to even)
    uint32_t bad[8];        // bit c set: reference code c has no hardware encoding (block is re-biased)
};

__global__ void __launch_bounds__(256) mx_pack_kernel(const uint8_t* __restrict__ scales, const uint8_t* elements,
                                                     uint8_t* hw_codes, uint8_t* __restrict__ hw_sf,
                                                     int64_t rows, int64_t K, int tile_rows, PackTables t) {
    __shared__ uint8_t s_plain[256], s_halved[256];
    s_plain[threadIdx.x] = t.plain[threadIdx.x];
    s_halved[threadIdx.x] = t.halved[threadIdx.x];
    __syncthreads();
    const int64_t kb_per_row = K / 32;
    const int64_t KT = (K + 127) / 128;
    const int64_t n_tiles = (rows + tile_rows - 1) / tile_rows;
    // one (tile, chunk-local row, K block) per thread, padding included: every byte of hw_sf is written
    const int64_t total = n_tiles * 256 * KT * 4;
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int64_t kb = i % (KT * 4);
    const int64_t lr = (i / (KT * 4)) % 256;          // tile-local row 0..255 (rows >= tile_rows are padding)
    const int64_t tile = i / (KT * 4 * 256);
    const int64_t r = tile * tile_rows + lr;
    const int64_t in_chunk = lr % 128;
    uint8_t* sf_dst = hw_sf + ((tile * KT + kb / 4) * 2 + lr / 128) * 512 + (in_chunk % 32) * 16 + (in_chunk / 32) * 4 + (kb % 4);
    if (lr >= tile_rows || r >= rows || kb >= kb_per_row) { *sf_dst = 127; return; }   // padding: scale 1.0 (codes there are TMA zero fill)
    const int64_t blk = r * kb_per_row + kb;
    if (hw_codes == nullptr) {                        // scale chunks only: the codes keep their own (sub-byte) format
        *sf_dst = scales != nullptr ? scales[blk] : (uint8_t)127;
        return;
    }
    // `elements` and `hw_codes` may be the same buffer: the whole block is read before it is written
    const uint4* src = reinterpret_cast<const uint4*>(elements + blk * 32);
    uint4 c[2] = {src[0], src[1]};
    const uint8_t* cb = reinterpret_cast<const uint8_t*>(c);
    bool any_bad = false;
#pragma unroll
    for (int j = 0; j < 32; ++j) any_bad |= (t.bad[cb[j] >> 5] >> (cb[j] & 31)) & 1u;
    const uint8_t* lut = any_bad ? s_halved : s_plain;
    uint4 o[2];
    uint8_t* ob = reinterpret_cast<uint8_t*>(o);
#pragma unroll
    for (int j = 0; j < 32; ++j) ob[j] = lut[cb[j]];
    uint4* dst = reinterpret_cast<uint4*>(hw_codes + blk * 32);
    dst[0] = o[0];
    dst[1] = o[1];
    const uint32_t s = scales != nullptr ? scales[blk] : 127u;           // no scales: every block is 2^0
    *sf_dst = (uint8_t)((any_bad && s < 255u) ? s + 1u : s);
}

// exact value -> OCP E4M3 / E5M2 byte (round half to even when the value is not representable)
static uint8_t hw_encode(double v, int hw_fmt) {
    const int eb = hw_fmt == 0 ? 4 : 5, fb = hw_fmt == 0 ? 3 : 2, bias = hw_fmt == 0 ? 7 : 15;
    const uint8_t sign = std::signbit(v) ? 0x80 : 0;
    double a = std::fabs(v);
    if (a == 0.0) return sign;
    int e;
    std::frexp(a, &e);
    e -= 1;                                                    // a = m * 2^e, m in [1,2)
    int E = e + bias;
    double scaled;                                             // value in units of the last mantissa bit
    if (E <= 0) { scaled = std::ldexp(a, bias - 1 + fb); E = 0; }          // subnormal: units of 2^(1-bias-fb)
    else scaled = std::ldexp(a, fb - e) - (1 << fb);                        // fraction field
    double fl = std::floor(scaled), rem = scaled - fl;
    int f = (int)fl;
    if (rem > 0.5 || (rem == 0.5 && (f & 1))) ++f;
    if (f == (1 << fb)) { f = 0; ++E; }
    (void)eb;
    return (uint8_t)(sign | (E << fb) | f);
}

static bool build_pack_tables(int eb, int fb, PackTables* t, int* hw_fmt) {
    if (!((eb == 4 && fb == 3) || (eb == 5 && fb == 2) || (eb == 2 && fb == 3) || (eb == 3 && fb == 2) || (eb == 2 && fb == 1))) return false;
    *hw_fmt = (eb == 5) ? 1 : 0;
    const double hw_max = *hw_fmt == 0 ? 448.0 : 57344.0;
    FmtRT f{eb, fb, 1, 0};
    for (int i = 0; i < 8; ++i) t->bad[i] = 0;
    for (int c = 0; c < 256; ++c) {
        const int bits = eb + fb + 1;
        // bits above the sign bit of the reference format are ignored by its decoder
        const uint32_t code = (uint32_t)c & ((1u << bits) - 1u);
        const double v = (double)bits_f32(decode_f32(code, f));
        const bool bad = std::fabs(v) > hw_max;
        if (bad) t->bad[c >> 5] |= 1u << (c & 31);
        t->plain[c] = bad ? 0 : hw_encode(v, *hw_fmt);
        t->halved[c] = hw_encode(v * 0.5, *hw_fmt);
    }
    return true;
}

// hardware operand formats (the instruction descriptor's encoding): one byte per code for the 8-bit formats; the
// 6- and 4-bit formats are dense bit streams in memory that TMA spreads to 16 codes per 16 bytes of shared memory
constexpr int HW_E4M3 = 0, HW_E5M2 = 1, HW_E2M3 = 3, HW_E3M2 = 4, HW_E2M1 = 5;
static int hw_code_bits(int hw_format) {
    switch (hw_format) {
        case HW_E4M3: case HW_E5M2: return 8;
        case HW_E2M3: case HW_E3M2: return 6;
        case HW_E2M1: return 4;
        default: return 0;
    }
}

// nibbles: the 4-bit x 4-bit kernel keeps two codes per byte in shared memory too (256 codes per 128-byte row)
static bool make_operand_map(CUtensorMap* map, const void* codes, int64_t rows, int64_t K, int box_rows, int hw_format = HW_E4M3,
                             bool nibbles = false) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const int bits = hw_code_bits(hw_format);
    const CUtensorMapDataType dt = nibbles ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN8B : bits == 8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : bits == 6 ? CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};                  // in codes, whatever their width
    const cuuint64_t strides[1] = {(cuuint64_t)(K * bits / 8)};
    const cuuint32_t box[2] = {(cuuint32_t)(nibbles ? 2 * BK : BK), (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(codes), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// outs == nullptr: plain epilogue into `out`; otherwise the gather-fused epilogue into outs->ptr[]
template <int OUT_DT, int MH, int EPI, bool MXF4 = false>
static int launch_gemm(const uint8_t* a_codes, const uint8_t* b_codes, const uint8_t* sfa, const uint8_t* sfb, void* out,
                       const BiasRef& bias, int M, int N, int K, int bn, uint32_t idesc, int* status, cudaStream_t st, const OutSpec* outs,
                       const OutMaps& omaps, const FwdMaps& fmaps) {
    using C = Cfg<MH, MXF4>;
    constexpr int SMEM = kernel_smem<EPI, MH, MXF4>();
    static_assert(SMEM <= 232448, "more shared memory than a CTA can have");
    static bool attr_done[MAX_DEVICES] = {false};
    const cudaError_t attr_err = raise_smem_limit(mx_gemm_kernel<OUT_DT, MH, EPI, MXF4>, SMEM, attr_done);
    if (attr_err != cudaSuccess) { set_last_cuda_error(attr_err); return MXQ_ELAUNCH; }
    CUtensorMap ma, mb;
    if constexpr (MXF4) {
        if (!make_operand_map(&ma, a_codes, M, K, C::BM, HW_E2M1, true) || !make_operand_map(&mb, b_codes, N, K, bn, HW_E2M1, true)) return MXQ_ELAUNCH;
    } else {
        if (!make_operand_map(&ma, a_codes, M, K, C::BM) || !make_operand_map(&mb, b_codes, N, K, bn, (int)((idesc >> 10) & 7u))) return MXQ_ELAUNCH;
    }
    const int tiles = ((M + C::BM - 1) / C::BM) * ((N + bn - 1) / bn);
    const int grid = tiles < sm_count() ? tiles : sm_count();          // persistent: one CTA per SM
    mx_gemm_kernel<OUT_DT, MH, EPI, MXF4><<<grid, kernel_threads<EPI>(), SMEM, st>>>(ma, mb, sfa, sfb, out, bias, M, N, K, bn, idesc, status,
                                                                               EPI == EPI_GATHER ? *outs : OutSpec{}, omaps, fmaps);
    return check_launch();
}

// Both operands as packed E2M1 nibbles: tcgen05.mma.kind::mxf4 (twice the arithmetic per instruction).  Only with an
// output the asynchronous epilogue can describe.
template <int OUT_DT>
static int launch_gemm_mxf4(const uint8_t* a_codes, const uint8_t* b_codes, const uint8_t* sfa, const uint8_t* sfb, void* out,
                            const BiasRef& bias, int M, int N, int K, int bn, int* status, cudaStream_t st) {
    OutMaps omaps{};
    FwdMaps fmaps{};
    if (!make_out_maps(&omaps, out, M, N, N, OUT_DT)) return MXQ_ESIZE;
    // formats: E2M1 is 1 in this kind's encoding; K-major operands, N >> 3, E8M0 scales, M >> 4; 64 elements of K per instruction
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24);
    if (M <= 128) return launch_gemm<OUT_DT, 1, EPI_TMA, true>(a_codes, b_codes, sfa, sfb, out, bias, M, N, K, bn, idesc, status, st, nullptr, omaps, fmaps);
    return launch_gemm<OUT_DT, 2, EPI_TMA, true>(a_codes, b_codes, sfa, sfb, out, bias, M, N, K, bn, idesc, status, st, nullptr, omaps, fmaps);
}

// Maps of the gather-fused kernel that forwards with the copy engine: the local epilogue's maps and one box map per
// destination, all over columns [col0, col0 + N) of the [M, ld] matrices.  False when a matrix cannot be described.
static bool make_gather_maps(const OutSpec& outs, int M, int N, int bn, int dt, OutMaps* omaps, FwdMaps* fmaps) {
    const int esz = dt == MXQ_F32 ? 4 : 2;
    int box_rows = 32;                                   // largest power of two whose box fits a forwarding buffer
    while (box_rows > 1 && box_rows * bn * esz > FWD_BUF_BYTES) box_rows >>= 1;
    if (box_rows * bn * esz > FWD_BUF_BYTES) return false;
    auto region = [&](int d) { return static_cast<void*>(static_cast<uint8_t*>(outs.ptr[d]) + outs.col0 * esz); };
    if (!make_out_maps(omaps, region(outs.self), M, N, outs.ld, dt)) return false;
    if (!make_rows_map(&fmaps->src, region(outs.self), M, N, outs.ld, dt, bn, box_rows)) return false;
    for (int d = 0; d < outs.n; ++d)
        if (d != outs.self && !make_rows_map(&fmaps->dst[d], region(d), M, N, outs.ld, dt, bn, box_rows)) return false;
    fmaps->n = outs.n; fmaps->self = outs.self; fmaps->box_rows = box_rows; fmaps->box_bytes = box_rows * bn * esz;
    // a tile narrower than the widest leaves (BN_MAX - bn) * BK bytes of every stage's B region unused: one more box each
    const int stages = M <= 128 ? Cfg<1>::STAGES : Cfg<2>::STAGES;
    const bool tails = (BN_MAX - bn) * BK >= fmaps->box_bytes;
    fmaps->n_bufs = FWD_BUFS + (tails ? (stages < FWD_BUFS_MAX - FWD_BUFS ? stages : FWD_BUFS_MAX - FWD_BUFS) : 0);
    return true;
}

template <int OUT_DT>
static int launch_gemm_dt(const uint8_t* a_codes, const uint8_t* b_codes, const uint8_t* sfa, const uint8_t* sfb, void* out,
                          const BiasRef& bias, int M, int N, int K, int bn, uint32_t idesc, int* status, cudaStream_t st,
                          const OutSpec* outs = nullptr) {
    OutMaps omaps{};
    FwdMaps fmaps{};
    if (outs != nullptr) {
        // the copy engine forwards whole row segments of a tile; outputs it cannot describe take the copy-out warps
        if (make_gather_maps(*outs, M, N, bn, OUT_DT, &omaps, &fmaps)) {
            if (M <= 128) return launch_gemm<OUT_DT, 1, EPI_GATHER_TMA>(a_codes, b_codes, sfa, sfb, nullptr, bias, M, N, K, bn, idesc, status, st, outs, omaps, fmaps);
            return launch_gemm<OUT_DT, 2, EPI_GATHER_TMA>(a_codes, b_codes, sfa, sfb, nullptr, bias, M, N, K, bn, idesc, status, st, outs, omaps, fmaps);
        }
        if (M <= 128) return launch_gemm<OUT_DT, 1, EPI_GATHER>(a_codes, b_codes, sfa, sfb, nullptr, bias, M, N, K, bn, idesc, status, st, outs, omaps, fmaps);
        return launch_gemm<OUT_DT, 2, EPI_GATHER>(a_codes, b_codes, sfa, sfb, nullptr, bias, M, N, K, bn, idesc, status, st, outs, omaps, fmaps);
    }
    // the asynchronous epilogue needs an output TMA can describe (16-byte aligned base and row pitch)
    if (make_out_maps(&omaps, out, M, N, N, OUT_DT)) {
        if (M <= 128) return launch_gemm<OUT_DT, 1, EPI_TMA>(a_codes, b_codes, sfa, sfb, out, bias, M, N, K, bn, idesc, status, st, nullptr, omaps, fmaps);
        return launch_gemm<OUT_DT, 2, EPI_TMA>(a_codes, b_codes, sfa, sfb, out, bias, M, N, K, bn, idesc, status, st, nullptr, omaps, fmaps);
    }
    if (M <= 128) return launch_gemm<OUT_DT, 1, EPI_REGS>(a_codes, b_codes, sfa, sfb, out, bias, M, N, K, bn, idesc, status, st, nullptr, omaps, fmaps);
    return launch_gemm<OUT_DT, 2, EPI_REGS>(a_codes, b_codes, sfa, sfb, out, bias, M, N, K, bn, idesc, status, st, nullptr, omaps, fmaps);
}

// instruction descriptor: A/B formats, K-major operands, N >> 3, E8M0 scales, M >> 4
static uint32_t mx_idesc(int a_hw_format, int b_hw_format, int bn) {
    return ((uint32_t)a_hw_format << 7) | ((uint32_t)b_hw_format << 10) | ((uint32_t)(bn >> 3) << 17) | (1u << 23) |
           ((uint32_t)(128 >> 4) << 24);
}

// the right operand's tile width: 0 selects the default, otherwise a multiple of 16 in [16, BN_MAX]
static int resolve_b_tile(int b_tile_rows) {
    if (b_tile_rows == 0) return BN_MAX;
    return (b_tile_rows >= 16 && b_tile_rows <= BN_MAX && b_tile_rows % 16 == 0) ? b_tile_rows : -1;
}

}  // namespace gemm
}  // namespace mxq

using namespace mxq;

// rows per scale-factor tile: 256 for the left operand; for the right one the CTA tile width it will be multiplied with
static int sf_tile_rows(int operand, int tile_rows) { return operand == MXQ_OPERAND_A ? gemm::A_TILE_ROWS : gemm::resolve_b_tile(tile_rows); }

// the left operand is one byte per code; the right one may also be a dense 6- or 4-bit stream (whole 128-code K steps,
// 32-byte aligned rows: what the packed tensor-map types ask for)
static bool operand_formats_ok(int a_hw_format, int b_hw_format, const uint8_t* b_codes, int64_t K) {
    if (a_hw_format == gemm::HW_E2M1)           // packed nibbles on the left: only against packed nibbles on the right (mxq_mx_gemm)
        return false;
    if (a_hw_format != gemm::HW_E4M3 && a_hw_format != gemm::HW_E5M2) return false;
    const int bits = gemm::hw_code_bits(b_hw_format);
    if (bits == 0) return false;
    if (bits != 8 && (K % 128 != 0 || reinterpret_cast<uintptr_t>(b_codes) % 32 != 0)) return false;
    return true;
}

extern "C" int mxq_mx_best_tile_rows(int64_t N) {
    // fewest padded columns first, the wider tile on a tie; widths below 160 only cost arithmetic intensity
    if (N <= 0) return gemm::BN_MAX;
    int best = gemm::BN_MAX;
    int64_t best_padded = ((N + best - 1) / best) * best;
    for (int t = gemm::BN_MAX - 16; t >= 160; t -= 16) {
        const int64_t padded = ((N + t - 1) / t) * t;
        if (padded < best_padded) { best = t; best_padded = padded; }
    }
    return best;
}

extern "C" int64_t mxq_mx_sf_bytes(int64_t rows, int64_t K, int operand, int tile_rows) {
    if (rows < 0 || K < 0 || (operand & ~1)) return MXQ_EINVAL;
    const int64_t t = sf_tile_rows(operand, tile_rows);
    if (t <= 0) return MXQ_EINVAL;
    return ((rows + t - 1) / t) * ((K + 127) / 128) * 1024;
}

extern "C" int mxq_mx_pack_operand(const uint8_t* scales, const uint8_t* elements, int64_t rows, int64_t K, int eb, int fb,
                                   int operand, int tile_rows, uint8_t* hw_codes, uint8_t* hw_sf, int* hw_format, void* stream) {
    if (rows <= 0 || K <= 0 || K % 32 != 0 || (operand & ~1) || !elements || !hw_codes || !hw_sf || !hw_format) return MXQ_EINVAL;
    if ((reinterpret_cast<uintptr_t>(elements) | reinterpret_cast<uintptr_t>(hw_codes)) % 16 != 0) return MXQ_EINVAL;
    gemm::PackTables t;
    if (!gemm::build_pack_tables(eb, fb, &t, hw_format)) return MXQ_EINVAL;
    const int tile = sf_tile_rows(operand, tile_rows);
    if (tile <= 0) return MXQ_EINVAL;
    const int64_t total = ((rows + tile - 1) / tile) * 256 * (((K + 127) / 128) * 4);
    gemm::mx_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(scales, elements, hw_codes, hw_sf, rows, K, tile, t);
    return check_launch();
}

extern "C" int mxq_mx_pack_operand_native(const uint8_t* scales, const uint8_t* elements, int64_t rows, int64_t K, int eb, int fb,
                                          int operand, int tile_rows, uint8_t* hw_codes, uint8_t* hw_sf, int* hw_format, void* stream) {
    if (rows <= 0 || K <= 0 || (operand & ~1) || !elements || !hw_codes || !hw_sf || !hw_format) return MXQ_EINVAL;
    if (operand == MXQ_OPERAND_A && !(eb == 2 && fb == 1)) return MXQ_ESIZE;      // a left operand only as nibbles for the 4-bit x 4-bit GEMM
    int fmt;
    if (eb == 2 && fb == 3) fmt = gemm::HW_E2M3;
    else if (eb == 3 && fb == 2) fmt = gemm::HW_E3M2;
    else if (eb == 2 && fb == 1) fmt = gemm::HW_E2M1;
    else return MXQ_ESIZE;
    if (K % 128 != 0 || reinterpret_cast<uintptr_t>(hw_codes) % 32 != 0 || reinterpret_cast<uintptr_t>(elements) % 16 != 0) return MXQ_ESIZE;
    const int tile = sf_tile_rows(operand, tile_rows);
    if (tile <= 0) return MXQ_EINVAL;
    // the reference's code bytes are the hardware's codes (sign, exponent, fraction in the low bits, the same subnormals,
    // no Inf / NaN): only the scale bytes move, and the codes are squeezed to their width
    const int64_t total = ((rows + tile - 1) / tile) * 256 * ((K / 128) * 4);
    gemm::mx_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(scales, elements, nullptr, hw_sf, rows, K, tile,
                                                                                          gemm::PackTables{});
    int rc = check_launch();
    if (rc != MXQ_OK) return rc;
    rc = mxq_pack_codes(elements, hw_codes, rows * K, gemm::hw_code_bits(fmt), stream);
    if (rc == MXQ_OK) *hw_format = fmt;
    return rc;
}

static int mx_gemm_impl(const uint8_t* a_codes, const uint8_t* a_sf, int a_hw_format, const uint8_t* b_codes, const uint8_t* b_sf,
                        int b_hw_format, int b_tile_rows, void* out, int out_dtype, const tc::BiasRef& bias, int64_t M, int64_t N, int64_t K,
                        int* status, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return MXQ_EINVAL;
    if (!a_codes || !a_sf || !b_codes || !b_sf || !out) return MXQ_EINVAL;
    if (a_hw_format == gemm::HW_E2M1 && b_hw_format == gemm::HW_E2M1) {
        // 4-bit x 4-bit: both operands dense nibbles, whole stages of 256 codes
        const int bn4 = gemm::resolve_b_tile(b_tile_rows);
        if (bn4 <= 0) return MXQ_EINVAL;
        if (K % 256 != 0) return MXQ_ESIZE;
        if ((reinterpret_cast<uintptr_t>(a_codes) | reinterpret_cast<uintptr_t>(b_codes)) % 32 != 0 ||
            (reinterpret_cast<uintptr_t>(a_sf) | reinterpret_cast<uintptr_t>(b_sf) | reinterpret_cast<uintptr_t>(out)) % 16 != 0) return MXQ_EINVAL;
        cudaStream_t st4 = (cudaStream_t)stream;
        if (out_dtype == MXQ_F32) return gemm::launch_gemm_mxf4<MXQ_F32>(a_codes, b_codes, a_sf, b_sf, out, bias, (int)M, (int)N, (int)K, bn4, status, st4);
        if (out_dtype == MXQ_BF16) return gemm::launch_gemm_mxf4<MXQ_BF16>(a_codes, b_codes, a_sf, b_sf, out, bias, (int)M, (int)N, (int)K, bn4, status, st4);
        if (out_dtype == MXQ_F16) return gemm::launch_gemm_mxf4<MXQ_F16>(a_codes, b_codes, a_sf, b_sf, out, bias, (int)M, (int)N, (int)K, bn4, status, st4);
        return MXQ_EINVAL;
    }
    if (!operand_formats_ok(a_hw_format, b_hw_format, b_codes, K)) return MXQ_EINVAL;
    const int bn = gemm::resolve_b_tile(b_tile_rows);
    if (bn <= 0) return MXQ_EINVAL;
    if ((reinterpret_cast<uintptr_t>(a_codes) | reinterpret_cast<uintptr_t>(b_codes) | reinterpret_cast<uintptr_t>(a_sf) |
         reinterpret_cast<uintptr_t>(b_sf) | reinterpret_cast<uintptr_t>(out)) % 16 != 0) return MXQ_EINVAL;
    const uint32_t idesc = gemm::mx_idesc(a_hw_format, b_hw_format, bn);
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == MXQ_F32) return gemm::launch_gemm_dt<MXQ_F32>(a_codes, b_codes, a_sf, b_sf, out, bias, (int)M, (int)N, (int)K, bn, idesc, status, st);
    if (out_dtype == MXQ_BF16) return gemm::launch_gemm_dt<MXQ_BF16>(a_codes, b_codes, a_sf, b_sf, out, bias, (int)M, (int)N, (int)K, bn, idesc, status, st);
    if (out_dtype == MXQ_F16) return gemm::launch_gemm_dt<MXQ_F16>(a_codes, b_codes, a_sf, b_sf, out, bias, (int)M, (int)N, (int)K, bn, idesc, status, st);
    return MXQ_EINVAL;
}

extern "C" int mxq_mx_gemm(const uint8_t* a_codes, const uint8_t* a_sf, int a_hw_format, const uint8_t* b_codes,
                           const uint8_t* b_sf, int b_hw_format, int b_tile_rows, void* out, int out_dtype, const void* bias,
                           int64_t M, int64_t N, int64_t K, int* status, void* stream) {
    return mx_gemm_impl(a_codes, a_sf, a_hw_format, b_codes, b_sf, b_hw_format, b_tile_rows, out, out_dtype, tc::BiasRef(bias), M, N, K, status, stream);
}

extern "C" int mxq_mx_gemm_qbias(const uint8_t* a_codes, const uint8_t* a_sf, int a_hw_format, const uint8_t* b_codes,
                                 const uint8_t* b_sf, int b_hw_format, int b_tile_rows, void* out, int out_dtype,
                                 const uint8_t* bias_scales, const uint8_t* bias_elements, int bias_exp_bits, int bias_frac_bits,
                                 int64_t M, int64_t N, int64_t K, int* status, void* stream) {
    if (!bias_scales || !bias_elements || N % 32 != 0) return MXQ_EINVAL;
    if (bias_exp_bits < 1 || bias_frac_bits < 1 || bias_exp_bits + bias_frac_bits > 7) return MXQ_EINVAL;
    return mx_gemm_impl(a_codes, a_sf, a_hw_format, b_codes, b_sf, b_hw_format, b_tile_rows, out, out_dtype,
                        tc::BiasRef(bias_elements, bias_scales, bias_exp_bits, bias_frac_bits), M, N, K, status, stream);
}

extern "C" int mxq_mx_gemm_gather(const uint8_t* a_codes, const uint8_t* a_sf, int a_hw_format, const uint8_t* b_codes,
                                  const uint8_t* b_sf, int b_hw_format, int b_tile_rows, void* const* outs, int n_outs, int self_index,
                                  int64_t ld_out, int64_t col_offset, int out_dtype, const void* bias, int64_t M, int64_t N, int64_t K,
                                  int* status, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return MXQ_EINVAL;
    if (!a_codes || !a_sf || !b_codes || !b_sf || !outs || n_outs < 1 || n_outs > gemm::MAX_DEST || self_index < 0 || self_index >= n_outs) return MXQ_EINVAL;
    if (!operand_formats_ok(a_hw_format, b_hw_format, b_codes, K)) return MXQ_EINVAL;
    const int bn = gemm::resolve_b_tile(b_tile_rows);
    if (bn <= 0) return MXQ_EINVAL;
    if (col_offset < 0 || ld_out < col_offset + N) return MXQ_EINVAL;
    if (out_dtype != MXQ_F32 && out_dtype != MXQ_BF16 && out_dtype != MXQ_F16) return MXQ_EINVAL;
    // whole 16-byte units only: the shard width, its offset and the leading dimension in units of 16 bytes
    const int64_t epu = out_dtype == MXQ_F32 ? 4 : 8;
    if (N % epu != 0 || ld_out % epu != 0 || col_offset % epu != 0) return MXQ_ESIZE;
    uintptr_t align = reinterpret_cast<uintptr_t>(a_codes) | reinterpret_cast<uintptr_t>(b_codes) | reinterpret_cast<uintptr_t>(a_sf) |
                      reinterpret_cast<uintptr_t>(b_sf);
    gemm::OutSpec spec{};
    for (int d = 0; d < n_outs; ++d) {
        if (!outs[d]) return MXQ_EINVAL;
        spec.ptr[d] = outs[d];
        align |= reinterpret_cast<uintptr_t>(outs[d]);
    }
    if (align % 16 != 0) return MXQ_EINVAL;
    spec.n = n_outs; spec.self = self_index; spec.ld = ld_out; spec.col0 = col_offset;
    const uint32_t idesc = gemm::mx_idesc(a_hw_format, b_hw_format, bn);
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == MXQ_F32) return gemm::launch_gemm_dt<MXQ_F32>(a_codes, b_codes, a_sf, b_sf, nullptr, bias, (int)M, (int)N, (int)K, bn, idesc, status, st, &spec);
    if (out_dtype == MXQ_BF16) return gemm::launch_gemm_dt<MXQ_BF16>(a_codes, b_codes, a_sf, b_sf, nullptr, bias, (int)M, (int)N, (int)K, bn, idesc, status, st, &spec);
    return gemm::launch_gemm_dt<MXQ_F16>(a_codes, b_codes, a_sf, b_sf, nullptr, bias, (int)M, (int)N, (int)K, bn, idesc, status, st, &spec);
}

// ------------------------------------------------------------------------------------------------
// fused-backend linear: quantise the activation, pack it, run the GEMM -- scratch supplied by the caller
// ------------------------------------------------------------------------------------------------
static int linear_with_scratch(const void* x, int x_dtype, int64_t M, int64_t K, int x_eb, int x_fb, const uint8_t* w_codes,
                               const uint8_t* w_sf, int w_hw_format, int w_tile_rows, int64_t N, void* out, int out_dtype, const void* bias,
                               uint8_t* scratch, int* status, void* stream) {
    // scratch: [M*K] element codes (re-encoded in place) | [M*K/32] reference scales | packed scale chunks
    uint8_t* codes = scratch;
    uint8_t* ref_scales = codes + M * K;
    uint8_t* sf = ref_scales + ((M * K / 32 + 255) / 256) * 256;
    int x_fmt = 0;
    // MXFP8 activations: one pass straight into the operand layout; other formats take extract + pack.  An MXFP4
    // activation is packed as nibbles (one pass too) only against a weight packed as nibbles: the 4-bit x 4-bit GEMM.
    const bool x_e2m1 = x_eb == 2 && x_fb == 1;
    const bool nibble_pair = x_e2m1 && w_hw_format == gemm::HW_E2M1 && K % 256 == 0;
    int rc = (x_e2m1 && !nibble_pair) ? MXQ_ESIZE
                                      : quantize_pack_left_operand(x, x_dtype, M, K, x_eb, x_fb, codes, sf, mxq_mx_sf_bytes(M, K, MXQ_OPERAND_A, 0),
                                                                   &x_fmt, (cudaStream_t)stream);
    if (rc == MXQ_OK) return mxq_mx_gemm(codes, sf, x_fmt, w_codes, w_sf, w_hw_format, w_tile_rows, out, out_dtype, bias, M, N, K, status, stream);
    if (rc != MXQ_ESIZE) return rc;
    rc = mxq_mxfp_extract(x, x_dtype, ref_scales, codes, M * K, 32, x_eb, x_fb, 1, MXQ_RN, stream);
    if (rc != MXQ_OK) return rc;
    int x_hw_format = 0;
    rc = mxq_mx_pack_operand(ref_scales, codes, M, K, x_eb, x_fb, MXQ_OPERAND_A, 0, codes, sf, &x_hw_format, stream);
    if (rc != MXQ_OK) return rc;
    return mxq_mx_gemm(codes, sf, x_hw_format, w_codes, w_sf, w_hw_format, w_tile_rows, out, out_dtype, bias, M, N, K, status, stream);
}

extern "C" int64_t mxq_mx_linear_scratch_bytes(int64_t M, int64_t K) {
    if (M <= 0 || K <= 0 || K % 32 != 0) return MXQ_EINVAL;
    return M * K + ((M * K / 32 + 255) / 256) * 256 + mxq_mx_sf_bytes(M, K, MXQ_OPERAND_A, 0);
}

extern "C" int mxq_mx_linear(const void* x, int x_dtype, int64_t M, int64_t K, int x_exp_bits, int x_frac_bits,
                             const uint8_t* w_codes, const uint8_t* w_sf, int w_hw_format, int w_tile_rows, int64_t N, void* out,
                             int out_dtype, const void* bias, void* scratch, int64_t scratch_bytes, int* status, void* stream) {
    if (!x || !w_codes || !w_sf || !out || !scratch || M <= 0 || N <= 0 || K <= 0 || K % 32 != 0) return MXQ_EINVAL;
    if (reinterpret_cast<uintptr_t>(scratch) % 256 != 0) return MXQ_EINVAL;
    if (scratch_bytes < mxq_mx_linear_scratch_bytes(M, K)) return MXQ_ESIZE;
    return linear_with_scratch(x, x_dtype, M, K, x_exp_bits, x_frac_bits, w_codes, w_sf, w_hw_format, w_tile_rows, N, out, out_dtype, bias,
                               static_cast<uint8_t*>(scratch), status, stream);
}

// ------------------------------------------------------------------------------------------------
// the same linear for callers that must not allocate: scratch is a fixed array inside the library
// ------------------------------------------------------------------------------------------------
// Some hosts of this code cannot call cudaMalloc at the point where they run a layer: a real-time
// inference loop that has handed all device memory to its own arena, a plugin loaded into a process
// whose allocator is off limits, a thread that runs while another thread captures a CUDA graph.
// For them the scratch of mxq_mx_linear lives here, in device memory reserved when the library is
// loaded (MXQ_STATIC_SCRATCH_BYTES on every GPU that loads it, until the process exits).
#define MXQ_STATIC_SCRATCH_BYTES (8ll << 20)
static __device__ __align__(256) uint8_t g_static_scratch[MXQ_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address: the address
// is looked up once per device, with that device current, and cached.
static uint8_t* static_scratch_ptr() {
    static std::mutex mu;
    static uint8_t* cache[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) { set_last_cuda_error(e); return nullptr; }
        cache[dev] = static_cast<uint8_t*>(p);
    }
    return cache[dev];
}

extern "C" int64_t mxq_mx_linear_static_capacity(void) { return MXQ_STATIC_SCRATCH_BYTES; }

extern "C" int mxq_mx_linear_static(const void* x, int x_dtype, int64_t M, int64_t K, int x_exp_bits, int x_frac_bits,
                                    const uint8_t* w_codes, const uint8_t* w_sf, int w_hw_format, int w_tile_rows, int64_t N,
                                    void* out, int out_dtype, const void* bias, int* status, void* stream) {
    if (!x || !w_codes || !w_sf || !out || M <= 0 || N <= 0 || K <= 0 || K % 32 != 0) return MXQ_EINVAL;
    if (mxq_mx_linear_scratch_bytes(M, K) > MXQ_STATIC_SCRATCH_BYTES) return MXQ_ESIZE;   // activation too large for the fixed scratch
    uint8_t* scratch = static_scratch_ptr();
    if (scratch == nullptr) return MXQ_ELAUNCH;
    // every byte of the scratch that the GEMM reads is written by the two kernels before it, so
    // nothing has to be cleared between calls
    return linear_with_scratch(x, x_dtype, M, K, x_exp_bits, x_frac_bits, w_codes, w_sf, w_hw_format, w_tile_rows, N, out, out_dtype, bias,
                               scratch, status, stream);
}

extern "C" int mxq_mx_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int exp_bits, int frac_bits,
                                    uint8_t* hw_codes, uint8_t* hw_sf, int* hw_format, void* stream) {
    if (!x || !hw_codes || !hw_sf || !hw_format || M <= 0 || K <= 0 || K % 32 != 0) return MXQ_EINVAL;
    return quantize_pack_left_operand(x, x_dtype, M, K, exp_bits, frac_bits, hw_codes, hw_sf, mxq_mx_sf_bytes(M, K, MXQ_OPERAND_A, 0),
                                      hw_format, (cudaStream_t)stream);
}

extern "C" int mxq_minifloat_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int exp_bits, int frac_bits,
                                           int round_mode, uint8_t* hw_codes, uint8_t* hw_sf, int* hw_format, void* stream) {
    if (!x || !hw_codes || !hw_sf || !hw_format || M <= 0 || K <= 0 || K % 32 != 0) return MXQ_EINVAL;
    if (round_mode != MXQ_RN) return MXQ_ESIZE;
    return minifloat_quantize_pack_left_operand(x, x_dtype, M, K, exp_bits, frac_bits, hw_codes, hw_sf,
                                                mxq_mx_sf_bytes(M, K, MXQ_OPERAND_A, 0), hw_format, (cudaStream_t)stream);
}
