// torch glue for attention_sm100.cu.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "attention_sm100.h"

namespace {

// qkv: bf16 [B, S, Hq + 2 Hkv, 128] contiguous; out: bf16 [B, S, Hq, 128]; lse: fp32 [B, Hq, S]
void attention_fwd(const at::Tensor& qkv, at::Tensor& out, at::Tensor& lse, int64_t n_heads, int64_t n_kv_heads, double scale,
                   const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.is_contiguous() && qkv.dim() == 4, "qkv must be contiguous CUDA bf16 [B,S,H,128]");
  TORCH_CHECK(qkv.size(3) == 128 && qkv.size(2) == n_heads + 2 * n_kv_heads, "qkv must hold Hq + 2 Hkv heads of 128");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.numel() == qkv.size(0) * qkv.size(1) * n_heads * 128,
              "out must be contiguous CUDA bf16 [B,S,Hq,128]");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == qkv.size(0) * n_heads * qkv.size(1),
              "lse must be contiguous CUDA fp32 [B,Hq,S]");
  c10::cuda::CUDAGuard g(qkv.device());
  elfb::AttnArgs a;
  a.qkv = qkv.data_ptr();
  a.out = out.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.batch = (int)qkv.size(0);
  a.seq = (int)qkv.size(1);
  a.n_heads = (int)n_heads;
  a.n_kv_heads = (int)n_kv_heads;
  a.scale = (float)scale;
  a.status = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
  const char* err = elfb::attention_forward(a, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, "elf_b200 attention: ", err ? err : "");
}

// Backward of attention_fwd.  dq_acc: fp32 [B, S, Hq, 128], all zero on entry and on return; lse2 / delta: fp32 [B, Hq, S] scratch.
void attention_bwd(const at::Tensor& qkv, const at::Tensor& out, const at::Tensor& dout, const at::Tensor& lse, at::Tensor& dqkv, at::Tensor& dq_acc,
                   at::Tensor& lse2, at::Tensor& delta, int64_t n_heads, int64_t n_kv_heads, double scale, const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.is_contiguous() && qkv.dim() == 4, "qkv must be contiguous CUDA bf16 [B,S,H,128]");
  TORCH_CHECK(qkv.size(3) == 128 && qkv.size(2) == n_heads + 2 * n_kv_heads, "qkv must hold Hq + 2 Hkv heads of 128");
  const int64_t B = qkv.size(0), S = qkv.size(1);
  const int64_t n_out = B * S * n_heads * 128, n_stat = B * n_heads * S;
  for (const at::Tensor* t : {&out, &dout})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kBFloat16 && t->is_contiguous() && t->numel() == n_out, "out / dout must be contiguous CUDA bf16 [B,S,Hq,128]");
  TORCH_CHECK(dqkv.is_cuda() && dqkv.scalar_type() == at::kBFloat16 && dqkv.is_contiguous() && dqkv.numel() == qkv.numel(), "dqkv must match qkv");
  TORCH_CHECK(dq_acc.is_cuda() && dq_acc.scalar_type() == at::kFloat && dq_acc.is_contiguous() && dq_acc.numel() == n_out, "dq_acc must be contiguous CUDA fp32 [B,S,Hq,128]");
  for (const at::Tensor* t : {&lse, (const at::Tensor*)&lse2, (const at::Tensor*)&delta})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == n_stat, "lse / lse2 / delta must be contiguous CUDA fp32 [B,Hq,S]");
  c10::cuda::CUDAGuard g(qkv.device());
  elfb::AttnBwdArgs a;
  a.qkv = qkv.data_ptr();
  a.out = out.data_ptr();
  a.dout = dout.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.dqkv = dqkv.data_ptr();
  a.dq_acc = dq_acc.data_ptr<float>();
  a.lse2 = lse2.data_ptr<float>();
  a.delta = delta.data_ptr<float>();
  a.batch = (int)B;
  a.seq = (int)S;
  a.n_heads = (int)n_heads;
  a.n_kv_heads = (int)n_kv_heads;
  a.scale = (float)scale;
  a.status = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
  const char* err = elfb::attention_backward(a, at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, "elf_b200 attention backward: ", err ? err : "");
}

}  // namespace

void register_attention(pybind11::module_& m) {
  m.def("attention_fwd", &attention_fwd, "causal GQA flash attention forward (tcgen05), head_dim 128", py::arg("qkv"), py::arg("out"), py::arg("lse"),
        py::arg("n_heads"), py::arg("n_kv_heads"), py::arg("scale") = 0.0, py::arg("status") = c10::nullopt);
  m.def("attention_bwd", &attention_bwd, "backward of attention_fwd (tcgen05): dK, dV, dQ into the packed gradient", py::arg("qkv"), py::arg("out"), py::arg("dout"),
        py::arg("lse"), py::arg("dqkv"), py::arg("dq_acc"), py::arg("lse2"), py::arg("delta"), py::arg("n_heads"), py::arg("n_kv_heads"), py::arg("scale") = 0.0,
        py::arg("status") = c10::nullopt);
}
