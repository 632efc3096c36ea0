// Host-side helpers shared by the translation units of libcdssm_b200.so.
#pragma once
#include "../../include/cdssm_b200.h"
#include "cdssm_math.cuh"

namespace cdssm {

// CUDA error of the last failed call on this host thread (read by cdssm_b200_last_cuda_error).
int& last_cuda_error_ref();

inline int check_cuda(cudaError_t e) {
    if (e == cudaSuccess) return CDSSM_OK;
    last_cuda_error_ref() = (int)e;
    return CDSSM_ERR_CUDA;
}
inline int check_launch() { return check_cuda(cudaGetLastError()); }

}  // namespace cdssm
