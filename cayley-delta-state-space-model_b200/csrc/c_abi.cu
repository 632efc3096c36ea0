// Entry points of the C ABI that are not tied to one kernel file.
#include "cdssm_common.cuh"

namespace cdssm {
int& last_cuda_error_ref() {
    static thread_local int e = 0;
    return e;
}
}  // namespace cdssm

extern "C" int cdssm_b200_version(void) { return 100; }
extern "C" int cdssm_b200_last_cuda_error(void) { return cdssm::last_cuda_error_ref(); }
