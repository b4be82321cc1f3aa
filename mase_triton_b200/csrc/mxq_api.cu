// Version, status strings and per-thread launch-error record of libmxq.
#include <cuda_runtime.h>

#include "../../include/mxq.h"
#include "mxq_internal.h"

namespace mxq {
static thread_local cudaError_t g_last_error = cudaSuccess;

void set_last_cuda_error(cudaError_t e) { g_last_error = e; }

int check_launch() {
    const cudaError_t e = cudaPeekAtLastError();
    if (e == cudaSuccess) return MXQ_OK;
    g_last_error = e;
    return MXQ_ELAUNCH;
}
}  // namespace mxq

extern "C" int mxq_version(void) { return 1100; }

extern "C" const char* mxq_status_string(int status) {
    switch (status) {
        case MXQ_OK: return "ok";
        case MXQ_EINVAL: return "invalid argument";
        case MXQ_ELAUNCH: return "CUDA launch failed";
        case MXQ_ESIZE: return "size not supported by this entry point";
        default: return "unknown status";
    }
}

extern "C" const char* mxq_last_cuda_error(void) { return cudaGetErrorString(mxq::g_last_error); }
