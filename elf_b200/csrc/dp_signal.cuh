// Device-side helpers of the peer-memory gradient exchange: system-scope flag access and the
// "last CTA of the launch raises the flags" election.
#pragma once

#include "dp_reduce.h"

namespace elfb {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Call with all threads of every CTA of the launch, after the CTA's last store to peer
// memory.  The CTA whose increment completes the count publishes `flag_value` on every
// peer; nobody waits for anybody.
__device__ __forceinline__ void signal_peers_when_last(unsigned int* done_counter, int* const* peer_flags, int n_peers, int flag_value) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;  // ready for the next launch on this stream
      __threadfence_system();
      for (int p = 0; p < n_peers; ++p) st_release_sys(peer_flags[p], flag_value);
    }
  }
}

}  // namespace elfb
