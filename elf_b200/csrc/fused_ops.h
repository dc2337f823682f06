// Launchers of the bandwidth-bound sm_100a kernels (fused_ops.cu).  All pointers are device
// pointers; 16-bit activations are bf16 unless `fp16` is set; every launcher returns the
// CUDA error of its launch.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace elfb {

// y = (x [+ residual]) * rsqrt(mean(.^2) + eps) * w ; optionally writes h = x + residual.
cudaError_t rmsnorm_forward(const void* x, const void* residual, const void* w, void* y, void* h, float* rstd, int rows,
                            int dim, float eps, cudaStream_t s);
// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)) [+ dres_in]; dw_partial[group][dim] = sum over a group of rows of dy*x*rstd.
// `dw_partial` is scratch of rmsnorm_backward_blocks(rows) * dim floats; `dw` ([dim]) receives (+=) the column sums:
// fp32, written or accumulated, or bf16 (`dw_bf16`, a gradient buffer, accumulate only; the sum is formed in fp32).
// `scratch_rows` says how many rows of `dim` floats `dw_partial` holds: rmsnorm_backward_blocks(rows) selects the
// single-pass persistent kernel, rmsnorm_backward_min_blocks() is the least that works (two-pass kernels).
int rmsnorm_backward_blocks(int rows);
int rmsnorm_backward_min_blocks();
cudaError_t rmsnorm_backward(const void* dy, const void* x, const void* w, const float* rstd, const void* dres_in, void* dx,
                             float* dw_partial, int scratch_rows, void* dw, bool dw_bf16, bool accumulate_dw, int rows, int dim,
                             cudaStream_t s);
// out[b, s, 0:hq] = dq, out[b, s, hq:hq+hkv] = dk, out[b, s, hq+hkv:] = dv for bf16 tensors given as [batch, seq, heads, head_dim]
// views with element strides {batch, seq, head} (head_dim contiguous; all strides multiples of 8): packs an attention backward's
// three gradients into the fused-QKV layout in one pass.  With `cos_t` / `sin_t` (fp32 [>= seq, head_dim / 2] tables) the
// backward of RoPE is applied to the query and key heads on the way (position = index along `seq`).
cudaError_t pack_qkv_grad(const void* dq, const void* dk, const void* dv, void* out, int batch, int seq, int hq, int hkv, int head_dim,
                          const long long* q_strides, const long long* k_strides, const long long* v_strides, const float* cos_t,
                          const float* sin_t, cudaStream_t s);
// out[i] += res[i] over n bf16 elements (n % 8 == 0): the residual add after a projection, in place.
cudaError_t residual_add(void* out, const void* res, long long n, cudaStream_t s);

// In-place rotary embedding on the first `n_rot_heads` heads of a [rows][n_heads*head_dim] bf16 matrix;
// position = row % seq_len; cos/sin tables are fp32 [seq_len][head_dim/2]; sign = +1 forward, -1 backward.
cudaError_t rope_inplace(void* x, const float* cos_t, const float* sin_t, int rows, int row_stride, int n_rot_heads,
                         int head_dim, int seq_len, float sign, cudaStream_t s);

// out[rows][F] = silu(gu[:, :F]) * gu[:, F:]
cudaError_t swiglu_forward(const void* gu, void* out, int rows, int f, cudaStream_t s);
// dgu[:, :F] = dout * up * dsilu(gate), dgu[:, F:] = dout * silu(gate)
cudaError_t swiglu_backward(const void* dout, const void* gu, void* dgu, int rows, int f, cudaStream_t s);

// Row-wise cross entropy over bf16 logits [rows][vocab] (row pitch `ld`): loss[row] = lse - logit[target], lse[row] saved.
cudaError_t cross_entropy_forward(const void* logits, const int64_t* targets, float* loss, float* lse, int rows, int vocab,
                                  long long ld, int64_t ignore_index, cudaStream_t s);
// dlogits = (exp(logit - lse) - onehot) * gscale[0] * scale, written over `logits` (in place) or into `dlogits`.
cudaError_t cross_entropy_backward(const void* logits, void* dlogits, const int64_t* targets, const float* lse,
                                   const float* gscale, float scale, int rows, int vocab, long long ld, int64_t ignore_index,
                                   cudaStream_t s);

// out[row] = table[ids[row]]
// Cross entropy with the vocabulary processed in column chunks.  `logits` = columns [col0, col0 + width) of all rows
// (row pitch `ld` elements).  stats: fold the chunk into run_max / run_sum (sum of exp(x - run_max)) / tgt_logit per row
// (`first` initialises them).  grad: logits <- (exp(logits - lse) - [col == target]) * scale * gscale, in place.
cudaError_t cross_entropy_chunk_stats(const void* logits, const int64_t* targets, float* run_max, float* run_sum, float* tgt_logit, int rows,
                                      int width, long long ld, long long col0, bool first, cudaStream_t s);
cudaError_t cross_entropy_chunk_grad(void* logits, const int64_t* targets, const float* lse, const float* gscale, float scale, int rows, int width,
                                     long long ld, long long col0, long long vocab, int64_t ignore_index, cudaStream_t s);
// out[row] = table[ids[row]].  An id outside [0, vocab) gives a zero row (no access) and, when `status`
// (int[4], may be null) still reads 0, records {4, 1 forward / 2 backward, row, id} there.
cudaError_t embedding_forward(const void* table, const int64_t* ids, void* out, int rows, int dim, long long vocab, int* status,
                              cudaStream_t s);
// dtable[ids[row]] += dout[row]   (fp32 or bf16 table gradient; atomics; ids outside [0, vocab) skipped and recorded)
// grad[sorted_ids[k]] += dout[perm[k]] for every k, deterministically: equal ids are adjacent in
// `sorted_ids` (ascending, stable), one CTA sums a run in order and adds it to the gradient row
// (bf16 or fp32) in place.  Ids outside [0, vocab) are skipped.
cudaError_t embedding_backward_sorted(const void* dout, const int64_t* sorted_ids, const int64_t* perm, void* grad, bool grad_f32, int rows,
                                      int dim, long long vocab, cudaStream_t s);
cudaError_t embedding_backward(const void* dout, const int64_t* ids, void* dtable, bool dtable_f32, int rows, int dim, long long vocab,
                               int* status, cudaStream_t s);

// Fused AdamW over flat buffers: bf16 params, fp32 master/m/v, grads bf16 or fp32.
//   g' = g * grad_scale; m = b1 m + (1-b1) g'; v = b2 v + (1-b2) g'^2
//   master = master * (1 - lr*wd) - lr * (m / bc1) / (sqrt(v / bc2) + eps); p = bf16(master)
// `status` (may be null): the per-device error record of this package's kernels; when its
// first word is non-zero the update is skipped, so parameters never move on gradients that a
// timed-out kernel left incomplete.
cudaError_t adamw_step(void* p_bf16, const void* grad, bool grad_f32, float* master, float* m, float* v, long long n,
                       float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                       float grad_scale, const int* status, cudaStream_t s);

// y = a * x (16-bit, in place allowed) — used for gradient scaling of flat buffers.
cudaError_t scale_bf16(void* x, long long n, float a, cudaStream_t s);

}  // namespace elfb
