// Host entry point of the tcgen05 GEMM family (gemm_sm100.cu).
#pragma once
#include <cuda_runtime.h>

#include "dp_reduce.h"

namespace elfb {

struct GemmArgs {
  const void* a = nullptr;     // A operand: [M][K] (K-major) or [K][M] (MN-major), 16-bit
  const void* b = nullptr;     // B operand: [N][K] (K-major) or [K][N] (MN-major), 16-bit
  void* d = nullptr;           // D [M][N], 16-bit (operand format) or fp32
  const void* bias = nullptr;  // optional [N], same type as D
  int M = 0, N = 0, K = 0;
  long long lda = 0, ldb = 0, ldd = 0;  // leading dimensions in elements
  int fmt = 1;                 // 1 = bf16, 0 = fp16
  bool a_mn_major = false, b_mn_major = false;
  bool out_f32 = false;
  bool accumulate = false;     // D += alpha * A.B instead of D = alpha * A.B
  float alpha = 1.0f;
  int* status = nullptr;       // optional device int[4] error record
  int variant = 0;             // 0 = single-CTA kernel, 1 = CTA-pair kernel (cta_group::2)
  bool split_tail = true;      // cut the tiles of the last, partial wave into column strips
  PushTarget push;             // optional: also store D into peer GPUs' inboxes and flag them (16-bit D only)
};

// Returns nullptr on success, otherwise a static description of the failure.
const char* gemm_tcgen05(const GemmArgs& args, int num_sms, cudaStream_t stream);

// Same contract, CTA-pair kernel (gemm_sm100_2cta.cu).
const char* gemm_tcgen05_pair(const GemmArgs& args, int num_sms, cudaStream_t stream);

// Whether this library was compiled with -DELF_BOUNDS_CHECK (tiled TMA copies validate their
// coordinates, record a violation in the status word and skip the copy instead of trapping).
bool bounds_check_build();
// Check build only: runs two copies with forbidden coordinates through the checked wrappers; the
// status word must read {5, 4, 3, 0} afterwards and nothing may have been issued.
cudaError_t bounds_check_selftest(int* status, cudaStream_t stream);

}  // namespace elfb
