// The give-up path of the bounded waits, reachable without a fault.
//
// The tensor-core and TMA kernels of this package wait on mbarriers with a limit (tcgen05.cuh:
// mbar_wait); when the limit runs out a block records code 2 in the device's status word, leaves
// in order, and the host raises at its next read of the word. In a healthy run no wait ever runs
// out, so that path would go untested. This file holds one tiny kernel that waits, with a limit
// its caller chooses (a millisecond or so), on a barrier that nothing will ever arrive at. The
// wait returns by itself, the kernel records the same code the real kernels record and returns
// normally: nothing traps, faults or hangs, and the context stays usable.
#include "tcgen05.cuh"

namespace {

__global__ void wait_probe_kernel(int* status, long long limit_cycles, int* gave_up_after_spins) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    pkv::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool arrived = pkv::mbar_wait(&bar, 0, &abort_flag, limit_cycles);
    if (!arrived && abort_flag) atomicExch(status, 2);
    if (gave_up_after_spins) *gave_up_after_spins = arrived ? 0 : 1;
  }
}

}  // namespace

// Runs one bounded wait that cannot succeed, with a limit of `limit_cycles` SM clock cycles (at
// most 2e8, a tenth of a second), and records status code 2 in `status` when it has given up.
// `gave_up` (a device int, may be null) is set to 1 when the wait returned without an arrival.
PKV_EXPORT int pkv_wait_probe(int* status, long long limit_cycles, int* gave_up, void* stream) {
  if (!status || limit_cycles <= 0 || limit_cycles > 200000000LL) return PKV_ERR_SIZE;
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, limit_cycles, gave_up);
  return pkv::launch_status();
}
