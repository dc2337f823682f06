// Data-parallel gradient exchange over NVLink peer memory (no NCCL on this path).
//
// Every replica owns, per pipeline stage, one contiguous bf16 gradient buffer and, in
// symmetric memory that its peers have mapped, one *inbox* of (R-1) slots of the same size
// plus a small array of 32-bit flags.  A replica PUSHES its finished gradients into its
// slot of every peer's inbox - from the epilogue of the weight-gradient GEMM for the
// matrices (gemm kernels with a PushTarget), and with `push_ranges` for everything else -
// then raises a flag on each peer.  `finalize_reduce` waits (bounded) for the peers' flags
// and computes grad = scale * (local + sum of inbox slots) from local memory only.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace elfb {

constexpr int kMaxPeers = 7;

// Where the epilogue of a weight-gradient GEMM also stores its output tile.
struct PushTarget {
  int n_peers = 0;
  void* peer_out[kMaxPeers] = {};    // address of D[0,0] inside my slot of peer p's inbox
  int* peer_flag[kMaxPeers] = {};    // flag word on peer p that announces "this matrix has landed"
  int flag_value = 0;                // value to write (the step's epoch)
  unsigned int* done_counter = nullptr;  // local counter used to elect the last CTA of the launch
};

// Copy `n_ranges` element ranges [begin, end) of my gradient buffer into my slot on every
// peer, then raise `flag_value` on each peer's flag word.
cudaError_t push_ranges(const void* grad, const long long* ranges_dev, int n_ranges, void* const* peer_slots_dev, int* const* peer_flags_dev,
                        int n_peers, int flag_value, unsigned int* done_counter, cudaStream_t s);

// Wait until the flags listed in wait_idx[0 .. n_wait) of every peer slot have reached
// `flag_value` (flags only grow; each wait is bounded by `timeout_ns`; on a timeout `status`
// gets kErrPeerTimeout and the gradient is left as it was), then
// grad[i] = scale * (grad[i] + sum_p inbox[p][i]) for i in [0, n).
//   my_flags: n_peers * n_flags words in my own symmetric memory, peer-major.
cudaError_t finalize_reduce(void* grad, const void* inbox, long long n, long long slot_stride, int n_peers, const int* my_flags,
                            int n_flags, const int* wait_idx, int n_wait, int flag_value, float scale, unsigned long long timeout_ns,
                            int* status, cudaStream_t s);

}  // namespace elfb
