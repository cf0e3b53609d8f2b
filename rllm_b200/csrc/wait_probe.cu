// The bounded wait of the tcgen05 kernels (sm100::mbar_wait), alone, so that its giving-up can be
// seen: one CTA of one warp initialises an mbarrier that nobody ever arrives at, waits on it for
// at most `limit_cycles` clock cycles, records the failure in the device error word the other
// kernels use, and returns. No cluster, no tensor memory, no copy in flight: nothing is left
// behind, and the GPU goes on as before. The host then sees the error at its next check, which is
// the path a production kernel's time-out takes.
#include "common.cuh"
#include "sm100.cuh"

using namespace rllm;

namespace {

__global__ void wait_probe_kernel(int* err, long long limit_cycles, int arrive_first) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&bar, 1);
    abort_flag = 0;
    sm100::fence_barrier_init();
    if (arrive_first) sm100::mbar_arrive(&bar);            // the wait below then succeeds at once
    if (!sm100::mbar_wait(&bar, 0, &abort_flag, limit_cycles)) sm100::record_failure(err, 9, 1);
  }
}

}  // namespace

// err: the device error word; limit_cycles: how long the wait may last (clamped to 1..10^7, some
// milliseconds at most); arrive_first != 0: the barrier is completed before the wait (no failure).
RLLM_API int rllm_wait_probe(int* err, long long limit_cycles, int arrive_first, void* stream) {
  if (!err) return ERR_BAD_SIZE;
  if (limit_cycles < 1) limit_cycles = 1;
  if (limit_cycles > 10000000LL) limit_cycles = 10000000LL;
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(err, limit_cycles, arrive_first);
  return launch_status();
}
