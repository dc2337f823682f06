// Peer-memory gradient exchange kernels (see dp_reduce.h for the protocol).
#include "dp_reduce.h"

#include <cuda_bf16.h>

#include "sm100_ptx.cuh"
#include "dp_signal.cuh"

namespace elfb {

namespace {

__global__ void __launch_bounds__(256) push_ranges_kernel(const uint4* __restrict__ grad, const long long* __restrict__ ranges, int n_ranges,
                                                          void* const* __restrict__ peer_slots, int* const* __restrict__ peer_flags, int n_peers,
                                                          int flag_value, unsigned int* done_counter) {
  // ranges are in elements of 2 bytes and 8-element aligned (flat buffers pad every tensor)
  for (int r = 0; r < n_ranges; ++r) {
    const long long b8 = ranges[2 * r] / 8, e8 = (ranges[2 * r + 1] + 7) / 8;
    for (long long i = b8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < e8; i += (long long)gridDim.x * blockDim.x) {
      const uint4 v = grad[i];
      for (int p = 0; p < n_peers; ++p) reinterpret_cast<uint4*>(peer_slots[p])[i] = v;
    }
  }
  signal_peers_when_last(done_counter, peer_flags, n_peers, flag_value);
}

__global__ void __launch_bounds__(256) finalize_reduce_kernel(uint4* __restrict__ grad, const uint4* __restrict__ inbox, long long n8,
                                                              long long slot_stride8, int n_peers, const int* __restrict__ my_flags, int n_flags,
                                                              const int* __restrict__ wait_idx, int n_wait, int flag_value, float scale,
                                                              unsigned long long timeout_ns, int* __restrict__ status) {
  // every CTA checks the flags itself: no CTA ever waits for another CTA
  // Flags carry the epoch of the step that wrote them and only ever grow, so "landed" is
  // flag >= epoch (a fast peer may already have announced the next step).
  for (int k = threadIdx.x; k < n_peers * n_wait; k += blockDim.x) {
    const int* flag = my_flags + (k / n_wait) * n_flags + wait_idx[k % n_wait];
    if (ld_acquire_sys(flag) >= flag_value) continue;
    const unsigned long long t0 = globaltimer_ns();
    while (ld_acquire_sys(flag) < flag_value) {
      if (globaltimer_ns() - t0 > timeout_ns) {
        if (status != nullptr && atomicCAS(status, kOk, kErrPeerTimeout) == kOk) {
          status[1] = k;
          status[2] = flag_value;
          status[3] = ld_acquire_sys(flag);
        }
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  // A wait that ran out (here or in an earlier kernel of the step) means the inbox may hold
  // stale or half-written data: leave the local gradient untouched.  The optimizer kernel
  // reads the same status word and skips its update, and the host raises at the next step.
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != kOk) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 g = grad[i];
    float acc[8];
    {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 t = __bfloat1622float2(h[k]);
        acc[2 * k] = t.x;
        acc[2 * k + 1] = t.y;
      }
    }
    for (int p = 0; p < n_peers; ++p) {
      const uint4 v = __ldcg(inbox + p * slot_stride8 + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 t = __bfloat1622float2(h[k]);
        acc[2 * k] += t.x;
        acc[2 * k + 1] += t.y;
      }
    }
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&g);
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[2 * k] * scale, acc[2 * k + 1] * scale);
    grad[i] = g;
  }
}

}  // namespace

cudaError_t push_ranges(const void* grad, const long long* ranges_dev, int n_ranges, void* const* peer_slots_dev, int* const* peer_flags_dev,
                        int n_peers, int flag_value, unsigned int* done_counter, cudaStream_t s) {
  push_ranges_kernel<<<296, 256, 0, s>>>((const uint4*)grad, ranges_dev, n_ranges, peer_slots_dev, peer_flags_dev, n_peers, flag_value, done_counter);
  return cudaGetLastError();
}

cudaError_t finalize_reduce(void* grad, const void* inbox, long long n, long long slot_stride, int n_peers, const int* my_flags, int n_flags,
                            const int* wait_idx, int n_wait, int flag_value, float scale, unsigned long long timeout_ns, int* status,
                            cudaStream_t s) {
  if (n % 8 || slot_stride % 8) return cudaErrorInvalidValue;
  finalize_reduce_kernel<<<592, 256, 0, s>>>((uint4*)grad, (const uint4*)inbox, n / 8, slot_stride / 8, n_peers, my_flags, n_flags, wait_idx,
                                             n_wait, flag_value, scale, timeout_ns, status);
  return cudaGetLastError();
}

}  // namespace elfb
