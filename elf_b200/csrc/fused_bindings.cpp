// torch glue for fused_ops.cu: shape checks, output allocation, stream selection.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "fused_ops.h"

namespace {

cudaStream_t cur() { return at::cuda::getCurrentCUDAStream(); }

void check(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, "elf_b200 ", what, ": ", cudaGetErrorString(e)); }

void need_bf16(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), name, " must be a contiguous CUDA bf16 tensor");
}

// returns (y, rstd, h) where h = x + residual (or x itself when residual is None)
std::tuple<at::Tensor, at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps,
                                                            const c10::optional<at::Tensor>& residual) {
  need_bf16(x, "x");
  need_bf16(w, "weight");
  c10::cuda::CUDAGuard g(x.device());
  const int dim = (int)x.size(-1);
  const int rows = (int)(x.numel() / dim);
  TORCH_CHECK(w.numel() == dim, "weight must have ", dim, " elements");
  auto y = at::empty_like(x);
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  at::Tensor h = x;
  const void* res = nullptr;
  if (residual.has_value() && residual->defined()) {
    need_bf16(*residual, "residual");
    TORCH_CHECK(residual->sizes() == x.sizes(), "residual must match x");
    h = at::empty_like(x);
    res = residual->data_ptr();
  }
  check(elfb::rmsnorm_forward(x.data_ptr(), res, w.data_ptr(), y.data_ptr(), res ? h.data_ptr() : nullptr,
                              rstd.data_ptr<float>(), rows, dim, (float)eps, cur()),
        "rmsnorm_forward");
  return {y, rstd, h};
}

// returns dx; dw (fp32 [dim]) is written or accumulated in place.  `scratch` may be passed to avoid an allocation.
at::Tensor rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd, at::Tensor& dw,
                       bool accumulate_dw, const c10::optional<at::Tensor>& dres, const c10::optional<at::Tensor>& scratch) {
  need_bf16(dy, "dy");
  need_bf16(x, "x");
  need_bf16(w, "weight");
  c10::cuda::CUDAGuard g(x.device());
  const int dim = (int)x.size(-1);
  const int rows = (int)(x.numel() / dim);
  const bool dw_bf16 = dw.scalar_type() == at::kBFloat16;
  TORCH_CHECK((dw.scalar_type() == at::kFloat || dw_bf16) && dw.is_cuda() && dw.numel() == dim && dw.is_contiguous(), "dw must be a contiguous fp32 or bf16 [dim] CUDA tensor");
  TORCH_CHECK(!dw_bf16 || accumulate_dw, "a bf16 dw is a gradient buffer: it can only be accumulated into");
  const int nb = elfb::rmsnorm_backward_blocks(rows);
  at::Tensor part = (scratch.has_value() && scratch->defined()) ? *scratch : at::empty({(int64_t)nb * dim}, x.options().dtype(at::kFloat));
  TORCH_CHECK(part.scalar_type() == at::kFloat && part.is_contiguous() && part.numel() >= (int64_t)elfb::rmsnorm_backward_min_blocks() * dim, "scratch too small");
  const int scratch_rows = (int)(part.numel() / dim);
  auto dx = at::empty_like(x);
  const void* dr = nullptr;
  if (dres.has_value() && dres->defined()) {
    need_bf16(*dres, "dres");
    dr = dres->data_ptr();
  }
  check(elfb::rmsnorm_backward(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dr, dx.data_ptr(),
                               part.data_ptr<float>(), scratch_rows, dw.data_ptr(), dw_bf16, accumulate_dw, rows, dim, cur()),
        "rmsnorm_backward");
  return dx;
}

// dq [B,S,hq,D], dk / dv [B,S,hkv,D] (any batch / seq / head strides, D contiguous) -> packed [B,S,hq+2hkv,D]
at::Tensor pack_qkv_grad(const at::Tensor& dq, const at::Tensor& dk, const at::Tensor& dv, const c10::optional<at::Tensor>& cos_t,
                         const c10::optional<at::Tensor>& sin_t) {
  for (const at::Tensor* t : {&dq, &dk, &dv})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16 && t->dim() == 4 && t->stride(3) == 1, "dq, dk, dv must be 4-D bf16 CUDA tensors with a contiguous last dimension");
  TORCH_CHECK(dk.sizes() == dv.sizes() && dq.size(0) == dk.size(0) && dq.size(1) == dk.size(1) && dq.size(3) == dk.size(3), "shape mismatch");
  c10::cuda::CUDAGuard g(dq.device());
  const int64_t B = dq.size(0), S = dq.size(1), hq = dq.size(2), hkv = dk.size(2), D = dq.size(3);
  auto out = at::empty({B, S, hq + 2 * hkv, D}, dq.options());
  const long long qs[3] = {dq.stride(0), dq.stride(1), dq.stride(2)}, ks[3] = {dk.stride(0), dk.stride(1), dk.stride(2)},
                  vs[3] = {dv.stride(0), dv.stride(1), dv.stride(2)};
  for (const at::Tensor* t : {&dq, &dk, &dv}) TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "gradients must be 16-byte aligned");
  const float *cp = nullptr, *sp = nullptr;
  if (cos_t.has_value() && cos_t->defined()) {
    TORCH_CHECK(sin_t.has_value() && sin_t->defined(), "cos and sin tables come together");
    for (const at::Tensor* t : {&*cos_t, &*sin_t})
      TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->dim() == 2 && t->size(0) >= S && t->size(1) == D / 2,
                  "cos/sin tables must be contiguous fp32 [>= seq, head_dim / 2]");
    cp = cos_t->data_ptr<float>();
    sp = sin_t->data_ptr<float>();
  }
  check(elfb::pack_qkv_grad(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), out.data_ptr(), (int)B, (int)S, (int)hq, (int)hkv, (int)D, qs, ks, vs, cp, sp,
                            cur()),
        "pack_qkv_grad");
  return out;
}

// out += res in place; returns out
at::Tensor residual_add(at::Tensor& out, const at::Tensor& res) {
  need_bf16(out, "out");
  need_bf16(res, "res");
  TORCH_CHECK(out.numel() == res.numel() && out.numel() % 8 == 0, "residual_add needs equally sized tensors with a multiple of 8 elements");
  c10::cuda::CUDAGuard g(out.device());
  check(elfb::residual_add(out.data_ptr(), res.data_ptr(), out.numel(), cur()), "residual_add");
  return out;
}

void rope_(at::Tensor& x, const at::Tensor& cos_t, const at::Tensor& sin_t, int64_t n_rot_heads, int64_t head_dim,
           int64_t seq_len, bool backward) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "x must be a 2-D bf16 CUDA matrix");
  TORCH_CHECK(cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat && cos_t.is_contiguous() && sin_t.is_contiguous(),
              "cos/sin tables must be contiguous fp32");
  TORCH_CHECK(cos_t.size(0) >= seq_len && cos_t.size(1) == head_dim / 2, "cos/sin tables must be [>=seq_len, head_dim/2]");
  TORCH_CHECK(n_rot_heads * head_dim <= x.size(1), "more rotary heads than columns");
  c10::cuda::CUDAGuard g(x.device());
  check(elfb::rope_inplace(x.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), (int)x.size(0), (int)x.stride(0),
                           (int)n_rot_heads, (int)head_dim, (int)seq_len, backward ? -1.f : 1.f, cur()),
        "rope");
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
  need_bf16(gu, "gate_up");
  c10::cuda::CUDAGuard g(gu.device());
  const int f = (int)gu.size(-1) / 2;
  const int rows = (int)(gu.numel() / (2 * f));
  auto sizes = gu.sizes().vec();
  sizes.back() = f;
  auto out = at::empty(sizes, gu.options());
  check(elfb::swiglu_forward(gu.data_ptr(), out.data_ptr(), rows, f, cur()), "swiglu_forward");
  return out;
}
at::Tensor swiglu_bwd(const at::Tensor& dout, const at::Tensor& gu) {
  need_bf16(dout, "dout");
  need_bf16(gu, "gate_up");
  c10::cuda::CUDAGuard g(gu.device());
  const int f = (int)gu.size(-1) / 2;
  const int rows = (int)(gu.numel() / (2 * f));
  auto dgu = at::empty_like(gu);
  check(elfb::swiglu_backward(dout.data_ptr(), gu.data_ptr(), dgu.data_ptr(), rows, f, cur()), "swiglu_backward");
  return dgu;
}

// returns (loss per row fp32, lse per row fp32)
std::tuple<at::Tensor, at::Tensor> ce_fwd(const at::Tensor& logits, const at::Tensor& targets, int64_t ignore_index) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1, "logits must be a 2-D bf16 CUDA matrix");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0), "targets must be int64 [rows]");
  c10::cuda::CUDAGuard g(logits.device());
  auto loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  auto lse = at::empty_like(loss);
  check(elfb::cross_entropy_forward(logits.data_ptr(), targets.data_ptr<int64_t>(), loss.data_ptr<float>(), lse.data_ptr<float>(),
                                    (int)logits.size(0), (int)logits.size(1), logits.stride(0), ignore_index, cur()),
        "cross_entropy_forward");
  return {loss, lse};
}
// writes dlogits over `out` (pass logits itself for the in-place form)
void ce_bwd(const at::Tensor& logits, at::Tensor& out, const at::Tensor& targets, const at::Tensor& lse,
            const c10::optional<at::Tensor>& gscale, double scale, int64_t ignore_index) {
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.sizes() == logits.sizes() && out.stride(0) == logits.stride(0), "out must match logits");
  c10::cuda::CUDAGuard g(logits.device());
  const float* gs = nullptr;
  if (gscale.has_value() && gscale->defined()) {
    TORCH_CHECK(gscale->scalar_type() == at::kFloat && gscale->numel() == 1, "gscale must be one fp32 value");
    gs = gscale->data_ptr<float>();
  }
  check(elfb::cross_entropy_backward(logits.data_ptr(), out.data_ptr(), targets.data_ptr<int64_t>(), lse.data_ptr<float>(), gs,
                                     (float)scale, (int)logits.size(0), (int)logits.size(1), logits.stride(0), ignore_index, cur()),
        "cross_entropy_backward");
}

void ce_chunk_stats(const at::Tensor& logits, const at::Tensor& targets, at::Tensor& run_max, at::Tensor& run_sum, at::Tensor& tgt_logit, int64_t col0,
                    bool first) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1, "logits must be a 2-D bf16 CUDA matrix");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0), "one int64 target per row");
  for (const at::Tensor* t : {&run_max, &run_sum, &tgt_logit})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == logits.size(0), "row statistics must be fp32 [rows]");
  c10::cuda::CUDAGuard g(logits.device());
  check(elfb::cross_entropy_chunk_stats(logits.data_ptr(), targets.data_ptr<int64_t>(), run_max.data_ptr<float>(), run_sum.data_ptr<float>(),
                                        tgt_logit.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), logits.stride(0), col0, first, cur()),
        "cross_entropy_chunk_stats");
}

void ce_chunk_grad(at::Tensor& logits, const at::Tensor& targets, const at::Tensor& lse, const c10::optional<at::Tensor>& gscale, double scale,
                   int64_t col0, int64_t vocab, int64_t ignore_index) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1, "logits must be a 2-D bf16 CUDA matrix");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0), "one int64 target per row");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == logits.size(0), "lse must be fp32 [rows]");
  const float* gs = nullptr;
  if (gscale.has_value() && gscale->defined()) {
    TORCH_CHECK(gscale->scalar_type() == at::kFloat && gscale->numel() == 1 && gscale->is_cuda(), "gscale must be one fp32 value on the device");
    gs = gscale->data_ptr<float>();
  }
  c10::cuda::CUDAGuard g(logits.device());
  check(elfb::cross_entropy_chunk_grad(logits.data_ptr(), targets.data_ptr<int64_t>(), lse.data_ptr<float>(), gs, (float)scale, (int)logits.size(0),
                                       (int)logits.size(1), logits.stride(0), col0, vocab, ignore_index, cur()),
        "cross_entropy_chunk_grad");
}

int* status_ptr(const c10::optional<at::Tensor>& status, const at::Tensor& like) {
  if (!status.has_value()) return nullptr;
  TORCH_CHECK(status->is_cuda() && status->scalar_type() == at::kInt && status->numel() >= 4 && status->get_device() == like.get_device(),
              "status must be an int32[4] tensor on the same device");
  return status->data_ptr<int>();
}

at::Tensor embedding_fwd(const at::Tensor& table, const at::Tensor& ids, const c10::optional<at::Tensor>& status) {
  need_bf16(table, "table");
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && ids.is_cuda(), "ids must be contiguous int64 CUDA");
  c10::cuda::CUDAGuard g(table.device());
  auto sizes = ids.sizes().vec();
  sizes.push_back(table.size(1));
  auto out = at::empty(sizes, table.options());
  check(elfb::embedding_forward(table.data_ptr(), ids.data_ptr<int64_t>(), out.data_ptr(), (int)ids.numel(), (int)table.size(1),
                                (long long)table.size(0), status_ptr(status, table), cur()),
        "embedding_forward");
  return out;
}
void embedding_bwd(const at::Tensor& dout, const at::Tensor& ids, at::Tensor& dtable, const c10::optional<at::Tensor>& status) {
  need_bf16(dout, "dout");
  TORCH_CHECK(dtable.is_contiguous() && (dtable.scalar_type() == at::kFloat || dtable.scalar_type() == at::kBFloat16), "dtable must be fp32 or bf16");
  c10::cuda::CUDAGuard g(dout.device());
  check(elfb::embedding_backward(dout.data_ptr(), ids.data_ptr<int64_t>(), dtable.data_ptr(), dtable.scalar_type() == at::kFloat,
                                 (int)ids.numel(), (int)dtable.size(1), (long long)dtable.size(0), status_ptr(status, dout), cur()),
        "embedding_backward");
}

void embedding_bwd_sorted(const at::Tensor& dout, const at::Tensor& sorted_ids, const at::Tensor& perm, at::Tensor& grad) {
  need_bf16(dout, "dout");
  TORCH_CHECK(dout.is_contiguous(), "dout must be contiguous");
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && grad.dim() == 2 && (grad.scalar_type() == at::kFloat || grad.scalar_type() == at::kBFloat16),
              "grad must be a contiguous [vocab, dim] fp32 or bf16 CUDA tensor");
  for (const at::Tensor* t : {&sorted_ids, &perm})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong && t->is_contiguous() && t->dim() == 1, "sorted_ids / perm must be 1-D contiguous int64 CUDA");
  TORCH_CHECK(sorted_ids.numel() == perm.numel() && dout.numel() == perm.numel() * grad.size(1), "shape mismatch between dout, ids and grad");
  c10::cuda::CUDAGuard g(dout.device());
  check(elfb::embedding_backward_sorted(dout.data_ptr(), sorted_ids.data_ptr<int64_t>(), perm.data_ptr<int64_t>(), grad.data_ptr(),
                                        grad.scalar_type() == at::kFloat, (int)perm.numel(), (int)grad.size(1), (long long)grad.size(0), cur()),
        "embedding_backward_sorted");
}

void adamw(at::Tensor& p, const at::Tensor& grad, at::Tensor& master, at::Tensor& m, at::Tensor& v, double lr, double b1, double b2,
           double eps, double wd, int64_t step, double grad_scale, const c10::optional<at::Tensor>& status) {
  need_bf16(p, "param");
  const int* status_ptr = nullptr;
  if (status.has_value()) {
    TORCH_CHECK(status->is_cuda() && status->scalar_type() == at::kInt && status->numel() >= 1, "status must be a CUDA int32 tensor");
    status_ptr = status->data_ptr<int>();
  }
  TORCH_CHECK(grad.is_contiguous() && grad.numel() == p.numel(), "grad must be contiguous and match param");
  TORCH_CHECK(grad.scalar_type() == at::kFloat || grad.scalar_type() == at::kBFloat16, "grad must be fp32 or bf16");
  for (const at::Tensor* t : {&master, &m, &v})
    TORCH_CHECK(t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == p.numel(), "optimizer state must be contiguous fp32");
  c10::cuda::CUDAGuard g(p.device());
  const double bc1 = 1.0 - std::pow(b1, (double)step), bc2 = 1.0 - std::pow(b2, (double)step);
  check(elfb::adamw_step(p.data_ptr(), grad.data_ptr(), grad.scalar_type() == at::kFloat, master.data_ptr<float>(), m.data_ptr<float>(),
                         v.data_ptr<float>(), p.numel(), (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, (float)bc1, (float)bc2,
                         (float)grad_scale, status_ptr, cur()),
        "adamw_step");
}

void scale_(at::Tensor& x, double a) {
  need_bf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  check(elfb::scale_bf16(x.data_ptr(), x.numel(), (float)a, cur()), "scale");
}

}  // namespace

void register_fused_ops(pybind11::module_& m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("weight"), py::arg("eps"), py::arg("residual") = c10::nullopt);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("weight"), py::arg("rstd"), py::arg("dw"),
        py::arg("accumulate_dw") = false, py::arg("dres") = c10::nullopt, py::arg("scratch") = c10::nullopt);
  m.def("rmsnorm_bwd_blocks", &elfb::rmsnorm_backward_blocks);
  m.def("rope_", &rope_, py::arg("x"), py::arg("cos"), py::arg("sin"), py::arg("n_rot_heads"), py::arg("head_dim"),
        py::arg("seq_len"), py::arg("backward") = false);
  m.def("pack_qkv_grad", &pack_qkv_grad, "pack dq, dk, dv ([B,S,H,D] views) into the fused-QKV gradient layout, optionally applying RoPE's backward",
        py::arg("dq"), py::arg("dk"), py::arg("dv"), py::arg("cos") = c10::nullopt, py::arg("sin") = c10::nullopt);
  m.def("residual_add", &residual_add, "out += res (bf16, in place); returns out");
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("ce_fwd", &ce_fwd, py::arg("logits"), py::arg("targets"), py::arg("ignore_index") = -100);
  m.def("ce_bwd", &ce_bwd, py::arg("logits"), py::arg("out"), py::arg("targets"), py::arg("lse"), py::arg("gscale") = c10::nullopt,
        py::arg("scale") = 1.0, py::arg("ignore_index") = -100);
  m.def("ce_chunk_stats", &ce_chunk_stats, py::arg("logits"), py::arg("targets"), py::arg("run_max"), py::arg("run_sum"), py::arg("tgt_logit"),
        py::arg("col0"), py::arg("first"));
  m.def("ce_chunk_grad", &ce_chunk_grad, py::arg("logits"), py::arg("targets"), py::arg("lse"), py::arg("gscale") = c10::nullopt, py::arg("scale") = 1.0,
        py::arg("col0") = 0, py::arg("vocab") = 0, py::arg("ignore_index") = -100);
  m.def("embedding_fwd", &embedding_fwd, "table[ids]; an id outside the table gives a zero row and is recorded in status", py::arg("table"), py::arg("ids"),
        py::arg("status") = c10::nullopt);
  m.def("embedding_bwd", &embedding_bwd, py::arg("dout"), py::arg("ids"), py::arg("dtable"), py::arg("status") = c10::nullopt);
  m.def("embedding_bwd_sorted", &embedding_bwd_sorted);
  m.def("adamw", &adamw, py::arg("param"), py::arg("grad"), py::arg("master"), py::arg("m"), py::arg("v"), py::arg("lr"),
        py::arg("beta1"), py::arg("beta2"), py::arg("eps"), py::arg("weight_decay"), py::arg("step"), py::arg("grad_scale") = 1.0, py::arg("status") = c10::nullopt);
  m.def("scale_", &scale_);
}
