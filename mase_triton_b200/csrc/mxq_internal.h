// Host-side helpers shared by the translation units of libmxq.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mxq {
// Records the error of a failed launch for mxq_last_cuda_error(); returns MXQ_OK or MXQ_ELAUNCH.
int check_launch();
void set_last_cuda_error(cudaError_t e);
// One-pass quantise + pack of a left GEMM operand (mxq_elementwise.cu); MXQ_ESIZE = not covered.
int quantize_pack_left_operand(const void* x, int x_dtype, int64_t M, int64_t K, int eb, int fb, uint8_t* hw_codes,
                               uint8_t* hw_sf, int64_t sf_bytes, int* hw_format, cudaStream_t st);
// The same for per-tensor minifloat FP8 codes with unit block scales (mxq_elementwise.cu).
int minifloat_quantize_pack_left_operand(const void* x, int x_dtype, int64_t M, int64_t K, int eb, int fb, uint8_t* hw_codes,
                                         uint8_t* hw_sf, int64_t sf_bytes, int* hw_format, cudaStream_t st);
}  // namespace mxq
