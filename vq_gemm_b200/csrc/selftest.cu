// Self-test of the failure path every pipelined kernel of this library relies on: a wait on an mbarrier
// that is bounded in time, records a code in the device status word when the limit passes, and lets the
// kernel return normally so that the context stays usable.  The kernel below waits on a barrier that nobody
// ever signals, with a caller-given (short) limit; nothing faults, traps or spins without bound.
#include "tc_ptx.cuh"

namespace vqg {
namespace {

__global__ void selftest_wait_kernel(int* status, long long limit_cycles, int* done) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    tc::mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // phase 0 never completes: there is no arrival
  const bool ok = tc::mbar_wait_limit(bar, 0, status, DS_SELFTEST_TIMEOUT, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && done) *done = ok ? 1 : 2;   // 2: the wait gave up, as it must
}

}  // namespace

int launch_selftest_wait(long long limit_cycles, cudaStream_t s) {
  if (limit_cycles < 1000 || limit_cycles > 2000000000LL) return VQG_ERR_BAD_ARG;   // at most about a second
  selftest_wait_kernel<<<1, 64, 0, s>>>(device_status_ptr(), limit_cycles, nullptr);
  count_launch();
  return cuda_status(cudaGetLastError());
}

}  // namespace vqg
