// torch glue for dp_reduce.cu.  Peer addresses arrive as integers (they come from the
// symmetric-memory rendezvous and are not torch tensors of this process).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "dp_reduce.h"
#include "p2p_signal.h"

namespace {

void check(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, "elf_b200 ", what, ": ", cudaGetErrorString(e)); }

// ranges: int64 CUDA tensor [n_ranges, 2]; peer_slots / peer_flags: int64 CUDA tensors [n_peers] holding device addresses
void push_ranges(const at::Tensor& grad, const at::Tensor& ranges, const at::Tensor& peer_slots, const at::Tensor& peer_flags, int64_t flag_value,
                 at::Tensor& counter) {
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && grad.element_size() == 2, "grad must be a contiguous 16-bit CUDA tensor");
  TORCH_CHECK(ranges.is_cuda() && ranges.scalar_type() == at::kLong && ranges.is_contiguous() && ranges.dim() == 2 && ranges.size(1) == 2, "ranges must be int64 [n,2] on the device");
  TORCH_CHECK(peer_slots.is_cuda() && peer_slots.scalar_type() == at::kLong && peer_flags.is_cuda() && peer_flags.scalar_type() == at::kLong &&
                  peer_slots.numel() == peer_flags.numel(), "peer tables must be int64 CUDA tensors of equal length");
  TORCH_CHECK(counter.is_cuda() && counter.scalar_type() == at::kInt, "counter must be an int32 CUDA tensor");
  c10::cuda::CUDAGuard g(grad.device());
  check(elfb::push_ranges(grad.data_ptr(), ranges.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(ranges.data_ptr<int64_t>()) : nullptr,
                          (int)ranges.size(0), reinterpret_cast<void* const*>(peer_slots.data_ptr<int64_t>()),
                          reinterpret_cast<int* const*>(peer_flags.data_ptr<int64_t>()), (int)peer_slots.numel(), (int)flag_value,
                          reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), at::cuda::getCurrentCUDAStream()),
        "push_ranges");
}

void finalize_reduce(at::Tensor& grad, const at::Tensor& inbox, int64_t n_peers, const at::Tensor& my_flags, int64_t n_flags,
                     const at::Tensor& wait_idx, int64_t flag_value, double scale, double timeout_ms, const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && grad.scalar_type() == at::kBFloat16, "grad must be contiguous CUDA bf16");
  TORCH_CHECK(inbox.is_cuda() && inbox.is_contiguous() && inbox.scalar_type() == at::kBFloat16 && inbox.numel() >= n_peers * grad.numel(), "inbox too small");
  TORCH_CHECK(my_flags.is_cuda() && my_flags.scalar_type() == at::kInt && my_flags.numel() >= n_peers * n_flags, "flag array too small");
  TORCH_CHECK(wait_idx.is_cuda() && wait_idx.scalar_type() == at::kInt && wait_idx.is_contiguous(), "wait_idx must be an int32 CUDA tensor");
  c10::cuda::CUDAGuard g(grad.device());
  int* st = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
  check(elfb::finalize_reduce(grad.data_ptr(), inbox.data_ptr(), grad.numel(), grad.numel(), (int)n_peers, my_flags.data_ptr<int>(), (int)n_flags,
                              wait_idx.data_ptr<int>(), (int)wait_idx.numel(), (int)flag_value, (float)scale,
                              (unsigned long long)(timeout_ms * 1e6), st, at::cuda::getCurrentCUDAStream()),
        "finalize_reduce");
}

// flag addresses arrive as integers: they may point into a peer's symmetric memory
void p2p_signal(int64_t flag_addr, int64_t value) {
  TORCH_CHECK(flag_addr != 0 && flag_addr % 4 == 0, "bad flag address");
  check(elfb::p2p_signal(reinterpret_cast<int*>(flag_addr), (int)value, at::cuda::getCurrentCUDAStream()), "p2p_signal");
}

void p2p_wait(const at::Tensor& flags, int64_t index, int64_t value, double timeout_ms, const c10::optional<at::Tensor>& status, int64_t where) {
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.is_contiguous() && index >= 0 && index < flags.numel(), "flags must be an int32 CUDA tensor holding `index`");
  c10::cuda::CUDAGuard g(flags.device());
  int* st = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
  check(elfb::p2p_wait(flags.data_ptr<int>() + index, (int)value, (unsigned long long)(timeout_ms * 1e6), st, (int)where, at::cuda::getCurrentCUDAStream()),
        "p2p_wait");
}

}  // namespace

void register_dp_reduce(pybind11::module_& m) {
  m.def("push_ranges", &push_ranges, "copy ranges of my gradient buffer into my slot on every peer and flag them");
  m.def("finalize_reduce", &finalize_reduce, "wait for the peers' flags, then grad = scale * (grad + sum of inbox slots)");
  m.def("p2p_signal", &p2p_signal, "after the current stream's prior work: store `value` (release, system scope) to the flag at `flag_addr`");
  m.def("p2p_wait", &p2p_wait, "block the current stream until flags[index] >= value (bounded by timeout_ms; records a peer timeout in `status`)",
        py::arg("flags"), py::arg("index"), py::arg("value"), py::arg("timeout_ms"), py::arg("status") = c10::nullopt, py::arg("where") = 0);
}
