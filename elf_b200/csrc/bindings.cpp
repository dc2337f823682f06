// Python bindings (torch extension) for the sm_100a kernels and the native host runtime.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "gemm_sm100.h"

namespace {

int fmt_of(const at::Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return 1;
  if (t.scalar_type() == at::kHalf) return 0;
  TORCH_CHECK(false, "elf_b200 GEMM operands must be bf16 or fp16, got ", t.scalar_type());
}

int sm_count() {
  static int n = 0;
  if (n == 0) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

// d (+)= alpha * op(a) . op(b) (+ bias).  Logical shapes: d [M,N]; a is [M,K] (a_mn_major=false,
// K contiguous) or [K,M] (a_mn_major=true, M contiguous); b is [N,K] or [K,N] likewise.
void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& d, const c10::optional<at::Tensor>& bias, bool a_mn_major,
          bool b_mn_major, bool accumulate, double alpha, const c10::optional<at::Tensor>& status, int64_t variant, bool split_tail,
          const std::vector<int64_t>& push_out, const std::vector<int64_t>& push_flags, int64_t push_flag_value,
          const c10::optional<at::Tensor>& push_counter) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && d.is_cuda(), "elf_b200 GEMM needs CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && d.dim() == 2, "elf_b200 GEMM takes 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && d.stride(1) == 1, "innermost dimension must be contiguous");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "A and B must have the same dtype");
  c10::cuda::CUDAGuard guard(d.device());
  elfb::GemmArgs g;
  g.fmt = fmt_of(a);
  g.M = (int)d.size(0);
  g.N = (int)d.size(1);
  g.K = (int)(a_mn_major ? a.size(0) : a.size(1));
  TORCH_CHECK((a_mn_major ? a.size(1) : a.size(0)) == g.M, "A does not match D's rows");
  TORCH_CHECK((b_mn_major ? b.size(1) : b.size(0)) == g.N, "B does not match D's columns");
  TORCH_CHECK((b_mn_major ? b.size(0) : b.size(1)) == g.K, "A and B disagree on the reduction length");
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.d = d.data_ptr();
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  g.ldd = d.stride(0);
  g.a_mn_major = a_mn_major;
  g.b_mn_major = b_mn_major;
  g.out_f32 = d.scalar_type() == at::kFloat;
  TORCH_CHECK(g.out_f32 || d.scalar_type() == a.scalar_type(), "D must be fp32 or the operand dtype");
  g.accumulate = accumulate;
  g.alpha = (float)alpha;
  g.variant = (int)variant;
  g.split_tail = split_tail;
  if (!push_out.empty()) {
    // peer_out[p]: address of this matrix inside my slot of peer p's inbox; peer_flag[p]: its flag word there
    TORCH_CHECK(push_out.size() == push_flags.size() && push_out.size() <= (size_t)elfb::kMaxPeers, "bad push target");
    TORCH_CHECK(!g.out_f32, "peer push needs a 16-bit output");
    TORCH_CHECK(push_counter.has_value() && push_counter->is_cuda() && push_counter->scalar_type() == at::kInt, "push needs an int32 CUDA counter");
    g.push.n_peers = (int)push_out.size();
    for (size_t p = 0; p < push_out.size(); ++p) {
      g.push.peer_out[p] = reinterpret_cast<void*>(push_out[p]);
      g.push.peer_flag[p] = reinterpret_cast<int*>(push_flags[p]);
    }
    g.push.flag_value = (int)push_flag_value;
    g.push.done_counter = reinterpret_cast<unsigned int*>(push_counter->data_ptr<int>());
  }
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == d.scalar_type() && bias->numel() == g.N && bias->is_contiguous(), "bias must be a contiguous [N] tensor of D's dtype");
    TORCH_CHECK(g.N % 8 == 0, "bias epilogue needs N % 8 == 0");
    g.bias = bias->data_ptr();
  }
  if (status.has_value() && status->defined()) g.status = status->data_ptr<int>();
  const char* err = elfb::gemm_tcgen05(g, sm_count(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(err == nullptr, "elf_b200 GEMM: ", err);
}

}  // namespace

void register_fused_ops(pybind11::module_& m);
void register_host_runtime(pybind11::module_& m);
void register_symm_runtime(pybind11::module_& m);
void register_dp_reduce(pybind11::module_& m);
void register_attention(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, "tcgen05 GEMM: d (+)= alpha * a.b (+ bias)", py::arg("a"), py::arg("b"), py::arg("d"),
        py::arg("bias") = c10::nullopt, py::arg("a_mn_major") = false, py::arg("b_mn_major") = false,
        py::arg("accumulate") = false, py::arg("alpha") = 1.0, py::arg("status") = c10::nullopt, py::arg("variant") = 0,
        py::arg("split_tail") = true, py::arg("push_out") = std::vector<int64_t>(), py::arg("push_flags") = std::vector<int64_t>(),
        py::arg("push_flag_value") = 0, py::arg("push_counter") = c10::nullopt);
  m.def("bounds_check_build", &elfb::bounds_check_build, "whether this library validates TMA coordinates on the device (-DELF_BOUNDS_CHECK)");
  m.def("bounds_check_selftest", [](at::Tensor& status) {
    TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 4, "status must be an int32[4] CUDA tensor");
    c10::cuda::CUDAGuard guard(status.device());
    const cudaError_t e = elfb::bounds_check_selftest(status.data_ptr<int>(), at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(e == cudaSuccess, "bounds_check_selftest: ", cudaGetErrorString(e));
  }, "check build only: two copies with forbidden coordinates go through the checked wrappers (recorded, not issued)");
#ifdef ELFB_WITH_DP_REDUCE
  register_dp_reduce(m);
#endif
#ifdef ELFB_WITH_ATTENTION
  register_attention(m);
#endif
  register_fused_ops(m);
  register_host_runtime(m);
  register_symm_runtime(m);
}
