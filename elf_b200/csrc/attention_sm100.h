// Causal grouped-query flash attention for sm_100a (attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>

namespace elfb {

struct AttnArgs {
  const void* qkv = nullptr;  // bf16 [B*S][(Hq + 2 Hkv) * 128]: Q heads, then K heads, then V heads
  void* out = nullptr;        // bf16 [B*S][Hq * 128]
  float* lse = nullptr;       // fp32 [B][Hq][S], natural-log sum of exp of the scaled scores
  int batch = 0, seq = 0, n_heads = 0, n_kv_heads = 0;
  float scale = 0.0f;         // softmax scale (1/sqrt(128) when 0)
  int* status = nullptr;
};

// head_dim is fixed at 128; seq must be a multiple of 128.  Returns nullptr or an error text.
const char* attention_forward(const AttnArgs& a, cudaStream_t stream);

struct AttnBwdArgs {
  const void* qkv = nullptr;   // bf16 [B*S][(Hq + 2 Hkv) * 128], as in the forward
  const void* out = nullptr;   // bf16 [B*S][Hq * 128]: the forward's output
  const void* dout = nullptr;  // bf16 [B*S][Hq * 128]: gradient of the output
  const float* lse = nullptr;  // fp32 [B][Hq][S]: the forward's log-sum-exp
  void* dqkv = nullptr;        // bf16 [B*S][(Hq + 2 Hkv) * 128]: gradient of qkv (every element is written)
  float* dq_acc = nullptr;     // fp32 [B*S][Hq * 128] scratch: all zero on entry, all zero again on return
  float* lse2 = nullptr;       // fp32 [B][Hq][S] scratch
  float* delta = nullptr;      // fp32 [B][Hq][S] scratch
  int batch = 0, seq = 0, n_heads = 0, n_kv_heads = 0;
  float scale = 0.0f;
  int* status = nullptr;
};

// Backward of attention_forward (attention_bwd_sm100.cu): three launches on `stream`.
const char* attention_backward(const AttnBwdArgs& a, cudaStream_t stream);

}  // namespace elfb
