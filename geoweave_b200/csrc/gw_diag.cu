// Diagnostics that are not part of the data path.
//
// gw_debug_bounded_wait_selftest shows the way every kernel of this library leaves a wait that can never be
// satisfied: one warp of a tiny kernel waits on an mbarrier nobody arrives at, with the limit given by the
// caller (milliseconds instead of the ~2 s of the real pipelines); when the limit passes, the warp records
// GW_ERR_TIMEOUT in the caller's status word and the kernel returns normally.  No trap, no fault, no endless
// loop: the context stays usable and the next call works.
#include "gw_common.cuh"

namespace gw {
namespace {

__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, int* status, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const unsigned long long t0 = global_timer_ns();
    const bool ok = mbar_wait_limit(&bar, 0u, limit_ns);  // phase 0 never completes: no thread arrives
    if (threadIdx.x == 0) {
      if (waited_ns != nullptr) *waited_ns = global_timer_ns() - t0;
      if (!ok) report_status(status, GW_ERR_TIMEOUT);
    }
  }
}

}  // namespace
}  // namespace gw

extern "C" int gw_debug_bounded_wait_selftest(unsigned int limit_us, int* status_dev, unsigned long long* waited_ns_dev,
                                              gw_stream_t stream) {
  if (status_dev == nullptr || limit_us == 0 || limit_us > 100000u) return GW_ERR_INVALID_ARG;  // at most 0.1 s
  gw::bounded_wait_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long>(limit_us) * 1000ull, status_dev, waited_ns_dev);
  GW_LAUNCH_CHECK();
  return GW_OK;
}
