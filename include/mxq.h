/*
 * libmxq — C ABI of the B200 (sm_100a) MXFP / minifloat fake-quantisation library.
 *
 * mase-triton is pure Python: it has no FFI of its own.  The functions below are
 * the seam its Python host code would bind in place of its Triton kernel hosts
 * (module mase_triton.{minifloat,mxfp}.kernels); each declaration cites the
 * reference function it replaces.  Every pointer is a DEVICE pointer on the
 * current CUDA device; `stream` is a cudaStream_t passed as void*.  The library
 * never allocates or frees device memory and never synchronises: the caller
 * owns every buffer and keeps it alive until the stream work has run.
 *
 * All functions return MXQ_OK (0) or a negative MXQ_E* code; none throws or traps.
 */
#ifndef MXQ_H_
#define MXQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element dtypes of floating-point tensors */
#define MXQ_F32 0
#define MXQ_BF16 1
#define MXQ_F16 2

/* rounding modes of MinifloatMeta.round_mode / MXFPMeta.round_mode */
#define MXQ_RN 0 /* "rn": half to even */
#define MXQ_RU 1 /* "ru": away from zero on the magnitude */
#define MXQ_RD 2 /* "rd": truncate the 15-bit mantissa */
#define MXQ_RZ 3 /* "rz": truncate the 23-bit mantissa */

#define MXQ_OK 0
#define MXQ_EINVAL -1   /* bad argument (null pointer, bad dtype, bad format, n % block_size != 0) */
#define MXQ_ELAUNCH -2  /* the CUDA launch failed; see mxq_last_cuda_error() */
#define MXQ_ESIZE -3    /* problem size outside what the entry point supports */

/* Library version (major * 1000 + minor). */
int mxq_version(void);
/* Text for an MXQ_* status. */
const char* mxq_status_string(int status);
/* cudaGetErrorString of the last failed launch made through this library on this thread. */
const char* mxq_last_cuda_error(void);

/*
 * Minifloat extract: floating tensor -> one uint16 code per element.
 * Replaces minifloat.kernels.extract_minifloat_component
 * (src/mase_triton/minifloat/kernels/cast.py:148-170); results follow the
 * reference's PyTorch path (src/mase_triton/minifloat/fake.py:7-78) bit for bit.
 * bf16/fp16 inputs are widened exactly inside the kernel (the reference casts to
 * fp32 first, minifloat/functional/cast.py:27).
 */
int mxq_minifloat_extract(const void* x, int x_dtype, uint16_t* codes, int64_t n,
                          int exp_bits, int frac_bits, int is_finite, int round_mode, void* stream);

/*
 * Minifloat compose: uint16 codes -> floating tensor of out_dtype.
 * Replaces minifloat.kernels.compose_minifloat_component
 * (src/mase_triton/minifloat/kernels/cast.py:263-288); follows fake.py:81-125.
 */
int mxq_minifloat_compose(const uint16_t* codes, void* out, int out_dtype, int64_t n,
                          int exp_bits, int frac_bits, int is_finite, void* stream);

/*
 * Fused minifloat quantize_dequantize (extract + compose without the uint16
 * intermediate). Replaces the two launches behind
 * minifloat.functional.quantize_dequantize (src/mase_triton/minifloat/functional/cast.py:72-90).
 */
int mxq_minifloat_qdq(const void* x, int x_dtype, void* out, int out_dtype, int64_t n,
                      int exp_bits, int frac_bits, int is_finite, int round_mode, void* stream);

/*
 * MXFP extract: flat floating tensor of n elements (n % block_size == 0) ->
 * scales[n / block_size] (E8M0 bytes) and elements[n] (one code per byte).
 * Replaces mxfp.kernels.extract_mxfp_components including its _find_block_max
 * pre-pass (src/mase_triton/mxfp/kernels/cast.py:15-21,126-160); follows
 * src/mase_triton/mxfp/fake.py:11-59.
 */
int mxq_mxfp_extract(const void* x, int x_dtype, uint8_t* scales, uint8_t* elements, int64_t n,
                     int block_size, int exp_bits, int frac_bits, int is_finite, int round_mode,
                     void* stream);

/*
 * MXFP compose: (scales, elements) -> flat floating tensor of out_dtype.
 * Replaces mxfp.kernels.compose_mxfp_tensor (src/mase_triton/mxfp/kernels/cast.py:237-272);
 * follows src/mase_triton/mxfp/fake.py:62-79.
 */
int mxq_mxfp_compose(const uint8_t* scales, const uint8_t* elements, void* out, int out_dtype,
                     int64_t n, int block_size, int exp_bits, int frac_bits, int is_finite,
                     void* stream);

/*
 * Fused MXFP quantize_dequantize (one pass, no scales/elements written).
 * Replaces the extract + compose pair behind mxfp.functional.quantize_dequantize
 * (src/mase_triton/mxfp/functional/cast.py:103-129) for a flat tensor.
 */
int mxq_mxfp_qdq(const void* x, int x_dtype, void* out, int out_dtype, int64_t n,
                 int block_size, int exp_bits, int frac_bits, int is_finite, int round_mode,
                 void* stream);

/*
 * ---- MXFP with blocks along a dimension that is not the contiguous one ----
 * The tensor is [outer, D, inner] (row-major, contiguous) and the blocks run along D.  The three
 * functions give the bytes the reference produces by first moving D last with a permute + copy
 * (flatten_for_quantize / permute_for_dequantize, src/mase_triton/mxfp/helpers.py:4-47, called from
 * src/mase_triton/mxfp/functional/cast.py:36-38,97-99) and then running the flat functions above:
 *   elements[(o * inner + i) * D + j], scales[(o * inner + i) * (D / block_size) + j / block_size]
 * while x / out keep the original layout, so no permuted copy is made.
 * They return MXQ_ESIZE for what they do not cover (block_size != 32, D % 32 != 0, a format or
 * rounding mode outside the round-to-nearest presets, out_dtype != x_dtype for the fused form,
 * unaligned buffers); the caller then takes the permute + flat route.
 */
int mxq_mxfp_extract_strided(const void* x, int x_dtype, uint8_t* scales, uint8_t* elements, int64_t outer,
                             int64_t D, int64_t inner, int block_size, int exp_bits, int frac_bits,
                             int is_finite, int round_mode, void* stream);
int mxq_mxfp_compose_strided(const uint8_t* scales, const uint8_t* elements, void* out, int out_dtype,
                             int64_t outer, int64_t D, int64_t inner, int block_size, int exp_bits,
                             int frac_bits, int is_finite, void* stream);
int mxq_mxfp_qdq_strided(const void* x, int x_dtype, void* out, int out_dtype, int64_t outer, int64_t D,
                         int64_t inner, int block_size, int exp_bits, int frac_bits, int is_finite,
                         int round_mode, void* stream);

/*
 * ---- MX GEMM (tcgen05 block-scaled tensor-core path) ----
 * Together these replace the "dequantise, then cuBLAS" sequence of mxfp_linear_XqWq / mxfp_matmul
 * (src/mase_triton/mxfp/functional/linear.py:36-64, matmul.py:10-35); the reference's own "fused"
 * backend is a stub that raises NotImplementedError (linear.py:62-63).
 */

/* operand roles of the GEMM: the scale-factor array is tiled to the CTA tile of its side */
#define MXQ_OPERAND_A 0 /* left operand  [M, K]: 256-row scale tiles */
#define MXQ_OPERAND_B 1 /* right operand [N, K]: scale tiles of `tile_rows` rows = the CTA tile width */

/*
 * The right operand is packed for one CTA tile width (`tile_rows`: 0 = the default 224, else a
 * multiple of 16 in [16, 224]) and the same value is handed to the GEMM as `b_tile_rows`.  224 gives
 * the highest arithmetic intensity; a narrower tile pays when N is not close to a multiple of 224
 * (N = 1024: five tiles of 208 instead of five of 224) or when whole 128-byte lines per row segment
 * matter (192 for the gather-fused kernel).  mxq_mx_best_tile_rows(N) returns the width with the
 * least padded work.  The left operand ignores `tile_rows` (pass 0).
 */
int mxq_mx_best_tile_rows(int64_t N);

/* Bytes of the hardware scale-factor array of an operand with `rows` rows and K columns. */
int64_t mxq_mx_sf_bytes(int64_t rows, int64_t K, int operand, int tile_rows);

/*
 * Re-encode an MXFP operand (reference scales [rows*K/32] and elements [rows*K], 32-element blocks
 * along K, as produced by mxq_mxfp_extract) for the tensor cores:
 *   hw_codes [rows*K]  : one OCP E4M3 byte per element (E5M2 when the element format is E5M2)
 *   hw_sf              : E8M0 scales in 512-byte chunks per (128 rows, 128 K), mxq_mx_sf_bytes() long,
 *                        tiled for `operand` (MXQ_OPERAND_A or MXQ_OPERAND_B)
 *   *hw_format (host)  : 0 = E4M3, 1 = E5M2
 * `scales` may be NULL: every block then has scale 2^0, which is how per-tensor minifloat codes
 * (low byte of the uint16 codes of mxq_minifloat_extract, formats of at most 8 bits) are fed to the
 * same GEMM for minifloat_linear (src/mase_triton/minifloat/functional/linear.py:108-171).
 * FP6/FP4 element values are exactly representable in E4M3. A block holding a value the hardware
 * format cannot encode (reference E4M3 480, reference E5M2 top binade) is stored with its scale
 * raised by one and its elements halved.
 */
int mxq_mx_pack_operand(const uint8_t* scales, const uint8_t* elements, int64_t rows, int64_t K,
                        int exp_bits, int frac_bits, int operand, int tile_rows, uint8_t* hw_codes,
                        uint8_t* hw_sf, int* hw_format, void* stream);

/*
 * An operand in the tensor cores' own 6- and 4-bit formats, for MXFP6 / MXFP4 tensors (element formats E2M3,
 * E3M2, E2M1; the reference's code bytes are already the hardware's codes):
 *   hw_codes           : rows * K codes as a dense little-endian bit stream of 6 (4) bits per code,
 *                        rows * K * 6 / 8 (rows * K / 2) bytes, 32-byte aligned - three quarters (half) of the
 *                        bytes the GEMM reads per element with mxq_mx_pack_operand
 *   hw_sf              : as mxq_mx_pack_operand(..., operand, tile_rows, ...)
 *   *hw_format (host)  : 3 = E2M3, 4 = E3M2, 5 = E2M1; pass it to the GEMM entry points as a/b_hw_format
 * MXQ_OPERAND_B, any of the three formats: against an 8-bit left operand the copy engine spreads every 16 codes
 * to 16 bytes of shared memory; the products are the same as with the one-byte-per-code form.
 * MXQ_OPERAND_A, E2M1 only: for the 4-bit x 4-bit GEMM (mxq_mx_gemm with a_hw_format = b_hw_format = 5), in
 * which both operands stay packed two codes per byte in shared memory and every tensor-core instruction covers 64
 * elements of K (tcgen05.mma.kind::mxf4): twice the arithmetic rate of the 8-bit kinds; K % 256 == 0 there.
 * K must be a multiple of 128 (else MXQ_ESIZE: use mxq_mx_pack_operand); MXQ_ESIZE also for the 8-bit element
 * formats.  `scales` may be NULL (unit scales).  No counterpart in the reference.
 */
int mxq_mx_pack_operand_native(const uint8_t* scales, const uint8_t* elements, int64_t rows, int64_t K,
                               int exp_bits, int frac_bits, int operand, int tile_rows, uint8_t* hw_codes,
                               uint8_t* hw_sf, int* hw_format, void* stream);

/*
 * One-pass alternative to mxq_mxfp_extract + mxq_mx_pack_operand for the LEFT operand: quantise
 * x [M,K] to MXFP8 (E4M3 or E5M2 elements, 32-element blocks along K, round to nearest) directly
 * into hardware codes and MXQ_OPERAND_A scale chunks. Same bytes as the two-step route.
 * E2M1 elements (MXFP4) are written as packed nibbles, M * K / 2 bytes, *hw_format = 5: the left operand
 * of the 4-bit x 4-bit GEMM, the bytes of mxq_mxfp_extract + mxq_mx_pack_operand_native(MXQ_OPERAND_A).
 * Returns MXQ_ESIZE for other element formats or unaligned buffers (use the two-step route).
 */
int mxq_mx_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int exp_bits, int frac_bits,
                         uint8_t* hw_codes, uint8_t* hw_sf, int* hw_format, void* stream);

/*
 * The same one-pass route for a per-tensor minifloat activation (minifloat_linear with layer type
 * XqWq*, src/mase_triton/minifloat/functional/linear.py:36-64): x [M,K] is quantised to FP8 E4M3 or
 * E5M2 (is_finite, round to nearest) and written as hardware codes with unit scale chunks.
 * MXQ_ESIZE for other formats, rounding modes or unaligned buffers (then: mxq_minifloat_extract,
 * narrow the codes to bytes, mxq_mx_pack_operand with scales = NULL).
 */
int mxq_minifloat_quantize_pack(const void* x, int x_dtype, int64_t M, int64_t K, int exp_bits, int frac_bits,
                                int round_mode, uint8_t* hw_codes, uint8_t* hw_sf, int* hw_format, void* stream);

/*
 * out[M,N] = A[M,K] * B[N,K]^T (+ bias[N]) on operands packed as MXQ_OPERAND_A / MXQ_OPERAND_B,
 * fp32 accumulation in tensor memory.  `b_tile_rows` is the value B was packed with.
 * a_hw_format: 0 / 1; b_hw_format: 0 / 1, or 3 / 4 / 5 for codes packed by mxq_mx_pack_operand_native;
 * a_hw_format = b_hw_format = 5 (both packed by mxq_mx_pack_operand_native): the 4-bit x 4-bit kernel
 * (K % 256 == 0 and an output whose base and row pitch are multiples of 16 bytes, else MXQ_ESIZE).
 * out_dtype / bias dtype: MXQ_F32, MXQ_BF16 or MXQ_F16 (bias may be NULL). K % 32 == 0.
 * `status` (an int32 the GPU can write: device memory, or pinned host memory mapped into the device so
 * that the host can poll it without synchronising; may be NULL; must be zero on entry) receives a
 * non-zero code if a bounded wait inside the kernel ran out: 1 operand copies, 2 MMA issue,
 * 3 epilogue, 4 copy-out to peers.  The kernel then unwinds (waits, bounded, for its own copies and
 * MMAs in flight, frees its tensor memory) and returns; the output is undefined.
 */
int mxq_mx_gemm(const uint8_t* a_codes, const uint8_t* a_sf, int a_hw_format, const uint8_t* b_codes,
                const uint8_t* b_sf, int b_hw_format, int b_tile_rows, void* out, int out_dtype,
                const void* bias, int64_t M, int64_t N, int64_t K, int* status, void* stream);

/*
 * mxq_mx_gemm with an MXFP-quantised bias (layer types *Bq, src/mase_triton/mxfp/functional/linear.py:52-57):
 * bias_elements [N] code bytes and bias_scales [N / 32] E8M0 bytes, as mxq_mxfp_extract writes them for the bias
 * vector (32-element blocks, is_finite element format with exp_bits + frac_bits <= 7).  The epilogue decodes the
 * code of every output column - the value and the rounding to out_dtype of mxq_mxfp_compose - and adds it:
 * no separate dequantisation launch, no dense bias in memory.  N % 32 == 0.
 */
int mxq_mx_gemm_qbias(const uint8_t* a_codes, const uint8_t* a_sf, int a_hw_format, const uint8_t* b_codes,
                      const uint8_t* b_sf, int b_hw_format, int b_tile_rows, void* out, int out_dtype,
                      const uint8_t* bias_scales, const uint8_t* bias_elements, int bias_exp_bits,
                      int bias_frac_bits, int64_t M, int64_t N, int64_t K, int* status, void* stream);

/*
 * ---- Dense storage of element codes ----
 * The reference keeps one MXFP element code per byte (`elements`, src/mase_triton/mxfp/fake.py:57-59;
 * the Parameter `w_elements` of MXFPLinearPTQ, src/mase_triton/mxfp/layers.py:66-80) although a code
 * has 1 + exp_bits + frac_bits significant bits.  mxq_pack_codes writes n codes of `bits` bits (4, 6
 * or 8) as a little-endian bit stream of mxq_packed_bytes(n, bits) = n * bits / 8 bytes (code i in
 * bits [i * bits, (i + 1) * bits)); mxq_unpack_codes restores one code per byte.  n must be a
 * multiple of 16 (else MXQ_ESIZE), both buffers 16-byte aligned.  No counterpart in the reference.
 */
int64_t mxq_packed_bytes(int64_t n, int bits);
int mxq_pack_codes(const uint8_t* codes, uint8_t* packed, int64_t n, int bits, void* stream);
int mxq_unpack_codes(const uint8_t* packed, uint8_t* codes, int64_t n, int bits, void* stream);

/*
 * ---- Tensor-core GEMMs for the layer types whose operands are not both block-quantised ----
 * out[M,N] = x[M,K] * W[N,K]^T (+ bias[N]); x, out and bias are bf16 or fp16 (`dtype`: MXQ_BF16 /
 * MXQ_F16; MXQ_F32 returns MXQ_ESIZE), fp32 accumulation in tensor memory (tcgen05.mma.kind::f16,
 * 256 x 256 tiles - 256 x 128 or 256 x 64 for dense operands when that occupies more SMs -, x by TMA).  `status` as for mxq_mx_gemm (code 5: a dequantiser wait ran out).
 * They replace "compose the weight to a dense tensor, then torch.nn.functional.linear" in
 * mxfp_linear_XWq / _XqW / _XW (src/mase_triton/mxfp/functional/linear.py:10-33,67-116),
 * minifloat_linear_XWq / _XqW / _XW (src/mase_triton/minifloat/functional/linear.py:10-105) and the
 * matmul forms (mxfp/functional/matmul.py:10-35, minifloat/functional/matmul.py:10-35); an activation
 * that the layer type quantises is fake-quantised first by mxq_mxfp_qdq / mxq_minifloat_qdq.
 */

/* W is a dense [N, K] matrix of the same dtype as x (brought in by TMA). K % 8 == 0. */
int mxq_dense_linear(const void* x, const void* w, int dtype, void* out, const void* bias, int64_t M,
                     int64_t N, int64_t K, int* status, void* stream);

/*
 * W stays quantised in memory, in the reference's own layout: w_elements [N*K] code bytes and
 * w_scales [N*K/32] E8M0 bytes of 32-element blocks along K (what mxq_mxfp_extract writes for a
 * [N, K] weight; the Parameters of MXFPLinearPTQ, src/mase_triton/mxfp/layers.py:66-80).  Eight
 * warps of each CTA expand the codes to `dtype` inside the operand loader, with the rounding of
 * compose_mxfp_tensor(..., output_dtype=dtype) (src/mase_triton/mxfp/fake.py:62-79); the dense weight
 * is never written to memory.  Element format: is_finite, exp_bits + frac_bits <= 7.  K % 32 == 0.
 */
int mxq_mxfp_weight_linear(const void* x, int dtype, const uint8_t* w_scales, const uint8_t* w_elements,
                           int exp_bits, int frac_bits, void* out, const void* bias, int64_t M,
                           int64_t N, int64_t K, int* status, void* stream);

/*
 * The same with a per-tensor minifloat weight: w_codes [N*K] uint16 codes as written by
 * mxq_minifloat_extract (Parameter `w_element` of MinifloatLinearPTQ), decoded like
 * compose_minifloat_component(..., output_dtype=dtype) (src/mase_triton/minifloat/fake.py:81-125).
 * exp_bits <= 8 (else MXQ_ESIZE).  K % 8 == 0.
 */
int mxq_minifloat_weight_linear(const void* x, int dtype, const uint16_t* w_codes, int exp_bits,
                                int frac_bits, int is_finite, void* out, const void* bias, int64_t M,
                                int64_t N, int64_t K, int* status, void* stream);

/*
 * mxq_mx_gemm that also performs the all-gather of a column-parallel linear (no counterpart in the
 * reference, which has no distributed code).  The [M, N] result of this rank's weight shard goes
 * to columns [col_offset, col_offset + N) of EVERY row-major [>= M, ld_out] matrix in
 * outs[0 .. n_outs) (host array of device pointers, at most 8): outs[self_index] is this GPU's own
 * output, the others are the peers' outputs mapped into this process (CUDA IPC / virtual-memory
 * mappings).  The epilogue warps write the local output; one more warp of the same CTAs reads each
 * finished half tile back (from L2) into small shared-memory boxes with TMA loads and sends every box
 * to each peer with a TMA store (whole row segments of the tile; no multicast), while the tensor cores
 * work on the next tile.  Outputs TMA cannot describe take four copy-out warps that store 16 bytes
 * per lane instead.  Nothing in the kernel waits on another GPU.  Ordering against the readers on the
 * other ranks is the caller's business (a collective or event after this call on the same stream).
 * N, ld_out and col_offset must be multiples of 8 elements (4 for MXQ_F32), else MXQ_ESIZE.
 */
int mxq_mx_gemm_gather(const uint8_t* a_codes, const uint8_t* a_sf, int a_hw_format, const uint8_t* b_codes,
                       const uint8_t* b_sf, int b_hw_format, int b_tile_rows, void* const* outs, int n_outs, int self_index,
                       int64_t ld_out, int64_t col_offset, int out_dtype, const void* bias, int64_t M,
                       int64_t N, int64_t K, int* status, void* stream);

/*
 * mxfp_linear with quantised activation and weight in one call (layer types XqWqB / XqWqBq,
 * src/mase_triton/mxfp/functional/linear.py:36-64): x [M,K] is quantised to the MXFP format
 * (x_exp_bits, x_frac_bits; 32-element blocks along K, round to nearest, is_finite), packed as
 * MXQ_OPERAND_A and multiplied with a weight already packed as MXQ_OPERAND_B.
 * `scratch` (device, 256-byte aligned, at least mxq_mx_linear_scratch_bytes(M, K) bytes) holds the
 * quantised activation between the three kernels; its contents are undefined afterwards.
 */
int64_t mxq_mx_linear_scratch_bytes(int64_t M, int64_t K);
int mxq_mx_linear(const void* x, int x_dtype, int64_t M, int64_t K, int x_exp_bits, int x_frac_bits,
                  const uint8_t* w_codes, const uint8_t* w_sf, int w_hw_format, int w_tile_rows, int64_t N,
                  void* out, int out_dtype, const void* bias, void* scratch, int64_t scratch_bytes,
                  int* status, void* stream);

/*
 * mxq_mx_linear for callers that cannot allocate device memory (no counterpart in the reference,
 * which always allocates through PyTorch).  Same arguments and same result as mxq_mx_linear, but
 * the scratch is a fixed array of mxq_mx_linear_static_capacity() bytes (8 MiB) that every GPU
 * loading this library reserves until the process exits.  Meant for hosts such as a real-time
 * serving loop that gave all device memory to its own arena, a plugin inside a process whose
 * allocator must not be touched, or work issued while another thread captures a CUDA graph.
 *   - Returns MXQ_ESIZE when mxq_mx_linear_scratch_bytes(M, K) exceeds the capacity
 *     (for instance M*K above roughly 7.5 Mi elements).
 *   - The first call on each device looks up the array's device address (no allocation); make that
 *     first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps the previous call's contents (nothing
 *     needs clearing: each call overwrites all it reads).  Two calls whose kernels can overlap on
 *     the GPU - different streams without an ordering between them - race on it; serialise them.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 */
int64_t mxq_mx_linear_static_capacity(void);
int mxq_mx_linear_static(const void* x, int x_dtype, int64_t M, int64_t K, int x_exp_bits, int x_frac_bits,
                         const uint8_t* w_codes, const uint8_t* w_sf, int w_hw_format, int w_tile_rows,
                         int64_t N, void* out, int out_dtype, const void* bias, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MXQ_H_ */
