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

// Performance-debugging hook (not part of the public header): device buffer of 16*5*16 int64 that
// receives clock64 stamps of one thread block of the tensor-core scans (the single-chain kernel uses the
// first 8*5*16 entries), or NULL to switch tracing off.
namespace cdssm { void scan_tc_set_trace(long long* p); void scan_tc4_set_trace(long long* p); }
extern "C" __attribute__((visibility("default"))) void cdssm_b200_debug_set_trace(void* p) {
    cdssm::scan_tc_set_trace(static_cast<long long*>(p));
    cdssm::scan_tc4_set_trace(static_cast<long long*>(p));
}
