// Entry points of the C ABI that are not tied to one kernel file.
#include "cdssm_common.cuh"
#include "sm100_ptx.cuh"
#include <atomic>

namespace cdssm {
int& last_cuda_error_ref() {
    static thread_local int e = 0;
    return e;
}
}  // namespace cdssm

namespace cdssm {
static std::atomic<unsigned long long> g_wait_limit_ns{0};
unsigned long long wait_limit_ns() {
    const unsigned long long v = g_wait_limit_ns.load(std::memory_order_relaxed);
    return v ? v : 400ull * 1000 * 1000;
}

__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        abort_flag = 0;
        sm100::fence_barrier_init();
    }
    __syncthreads();
    // nothing ever arrives on the barrier: the wait has to give up after limit_ns and say so
    const bool ok = sm100::mbar_wait_suspend(&bar, 0, &abort_flag, limit_ns);
    __syncthreads();
    if (threadIdx.x == 0) *status = ok ? 2 : 1;
}
}  // namespace cdssm

extern "C" uint64_t cdssm_b200_set_wait_limit_ns(uint64_t limit_ns) {
    return cdssm::g_wait_limit_ns.exchange(limit_ns);
}
extern "C" int cdssm_b200_selftest_bounded_wait(int* status_dev, uint64_t limit_ns, void* stream) {
    if (!status_dev || limit_ns == 0 || limit_ns > 2000ull * 1000 * 1000) return CDSSM_ERR_BAD_ARG;
    cdssm::bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status_dev, limit_ns);
    return cdssm::check_launch();
}

extern "C" int cdssm_b200_version(void) { return 201; }
extern "C" int cdssm_b200_last_cuda_error(void) { return cdssm::last_cuda_error_ref(); }
