// Flags for the copy-engine transport between pipeline stages (see p2p_signal.h).
#include "p2p_signal.h"

#include "sm100_ptx.cuh"
#include "dp_signal.cuh"

namespace elfb {

namespace {

__global__ void p2p_signal_kernel(int* flag, int value) {
  // everything this stream did before (the copy into the peer's ring slot) is complete and
  // visible when the kernel starts; the release store orders the flag after it system-wide
  __threadfence_system();
  st_release_sys(flag, value);
}

__global__ void __launch_bounds__(32) p2p_wait_kernel(const int* flag, int value, unsigned long long timeout_ns, int* status, int where) {
  if (threadIdx.x != 0) return;
  if (ld_acquire_sys(flag) >= value) return;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(flag) < value) {
    if (globaltimer_ns() - t0 > timeout_ns) {
      if (status != nullptr && atomicCAS(status, kOk, kErrPeerTimeout) == kOk) {
        status[1] = where;
        status[2] = value;
        status[3] = ld_acquire_sys(flag);
      }
      return;
    }
    __nanosleep(500);
  }
}

}  // namespace

cudaError_t p2p_signal(int* flag, int value, cudaStream_t s) {
  p2p_signal_kernel<<<1, 1, 0, s>>>(flag, value);
  return cudaGetLastError();
}

cudaError_t p2p_wait(const int* flag, int value, unsigned long long timeout_ns, int* status, int where, cudaStream_t s) {
  p2p_wait_kernel<<<1, 32, 0, s>>>(flag, value, timeout_ns, status, where);
  return cudaGetLastError();
}

}  // namespace elfb
