// Host-side helpers shared by the translation units of libmxq.
#pragma once
#include <cuda_runtime.h>

namespace mxq {
// Records the error of a failed launch for mxq_last_cuda_error(); returns MXQ_OK or MXQ_ELAUNCH.
int check_launch();
void set_last_cuda_error(cudaError_t e);
}  // namespace mxq
