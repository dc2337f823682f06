// Stream-ordered flags for the copy-engine transport between pipeline stages.
//
// A producer copies a tensor into a ring slot in the consumer's memory with the copy engines
// (cudaMemcpyAsync over NVLink, no SM involved) and then raises a sequence number on the
// consumer: `p2p_signal`, a one-thread kernel doing a system-scope release store, queued on
// the same stream right after the copy.  The consumer queues `p2p_wait` on its compute stream
// before it reads the slot: one thread polls its own memory until the sequence number has
// been reached.  The wait is bounded: after `timeout_ns` it records kErrPeerTimeout in the
// status word (detail: `where`, the value waited for, the value seen) and returns, so the
// stream never hangs on a peer that is gone.  The same pair, in the other direction, tells
// the producer that a slot may be overwritten.  Sequence numbers only grow.
#pragma once
#include <cuda_runtime.h>

namespace elfb {

// *flag = value (release, system scope) once all prior work of stream `s` has completed.
cudaError_t p2p_signal(int* flag, int value, cudaStream_t s);

// Block stream `s` until *flag >= value, for at most `timeout_ns`.
cudaError_t p2p_wait(const int* flag, int value, unsigned long long timeout_ns, int* status, int where, cudaStream_t s);

}  // namespace elfb
