// Barrier across the GPUs of a sharded product: one epoch flag per (waiting rank, arriving rank) in
// peer-mapped memory, plain system-scope stores and loads over NVLink (no multicast, no TMA), and a wait that
// is bounded in time: when a rank does not arrive within the limit the kernel records a code in the device
// status word and returns, so that the context stays usable and the host learns of it from
// vqg_device_status().  The reference has nothing of the kind (single GPU, strategy_1/src.cu:343).
//
// Protocol: rank a announces its arrival at barrier number `epoch` by storing `epoch` into slot a of every
// other rank's flag array (release at system scope: everything this rank wrote before -- the kernels ahead
// of the barrier on the stream have completed -- is visible to whoever reads the flag), then waits until every
// slot of its own array has reached `epoch` (acquire loads).  Epochs only grow, so a rank that is already one
// barrier ahead never holds up one that is still waiting, and flags never need resetting.
#include "common.cuh"

namespace vqg {
namespace {

struct FlagPtrs {
  unsigned* f[8];
};

__global__ void rank_barrier_kernel(const FlagPtrs flags, int rank, int nranks, unsigned epoch, long long limit_cycles,
                                    int* status) {
  // launched with programmatic stream serialisation: this block may already sit on an SM while the product ahead
  // of it on the stream is still running; everything that kernel stored is complete and visible after this wait
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int r = threadIdx.x;
  if (r >= nranks || r == rank) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.f[r] + rank), "r"(epoch) : "memory");
  const unsigned* mine = flags.f[rank] + r;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int>(v - epoch) >= 0) return;
    if ((++spins & 15u) == 0 && clock64() - t0 > limit_cycles) {
      atomicCAS(status, 0, static_cast<int>(DS_RANK_BARRIER_TIMEOUT));
      return;
    }
  }
}

}  // namespace

int launch_rank_barrier(unsigned* const* flags, int rank, int nranks, unsigned epoch, long long limit_cycles, cudaStream_t s) {
  FlagPtrs fp{};
  for (int r = 0; r < nranks; ++r) fp.f[r] = flags[r];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, rank_barrier_kernel, fp, rank, nranks, epoch, limit_cycles, device_status_ptr());
  count_launch();
  return cuda_status(e == cudaSuccess ? cudaGetLastError() : e);
}

}  // namespace vqg
