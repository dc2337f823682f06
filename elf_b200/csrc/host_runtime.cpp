// Native host-side runtime pieces.
//
// PinnedArena: sub-allocator over large pinned host blocks used by activation offload.
// First fit over an address-ordered free list with coalescing on release, so a step that
// offloads and restores the same tensors every iteration settles on a fixed set of
// addresses and never calls cudaHostAlloc again.  (Behavioural counterpart of the
// reference's Python PinnedHostTensorPool, elf/execution/offload.py:14-163.)
#include <torch/extension.h>

#include <algorithm>
#include <deque>
#include <limits>
#include <vector>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <mutex>
#include <stdexcept>
#include <vector>

namespace {

class PinnedArena {
 public:
  explicit PinnedArena(size_t min_block_bytes) : min_block_(min_block_bytes ? min_block_bytes : (size_t(64) << 20)) {}
  ~PinnedArena() {
    for (auto& b : blocks_) {
      if (pinned_) cudaFreeHost(b.first); else free(b.first);
    }
  }

  void reserve(size_t bytes) {
    std::lock_guard<std::mutex> g(mu_);
    if (largest_free() < bytes) grow(bytes);
  }

  // returns an address aligned to 256 bytes
  uintptr_t allocate(size_t bytes) {
    std::lock_guard<std::mutex> g(mu_);
    bytes = round_up(bytes ? bytes : 1);
    for (int attempt = 0; attempt < 2; ++attempt) {
      for (auto it = free_.begin(); it != free_.end(); ++it) {
        if (it->second >= bytes) {
          const uintptr_t addr = it->first;
          const size_t rest = it->second - bytes;
          free_.erase(it);
          if (rest) free_[addr + bytes] = rest;
          live_[addr] = bytes;
          in_use_ += bytes;
          if (in_use_ > peak_) peak_ = in_use_;
          return addr;
        }
      }
      grow(bytes);
    }
    throw std::runtime_error("PinnedArena: allocation failed");
  }

  void release(uintptr_t addr) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = live_.find(addr);
    if (it == live_.end()) throw std::runtime_error("PinnedArena: release of an address that is not live");
    size_t bytes = it->second;
    live_.erase(it);
    in_use_ -= bytes;
    auto next = free_.lower_bound(addr);
    if (next != free_.end() && addr + bytes == next->first && same_block(addr, next->first)) {
      bytes += next->second;
      next = free_.erase(next);
    }
    if (next != free_.begin()) {
      auto prev = std::prev(next);
      if (prev->first + prev->second == addr && same_block(prev->first, addr)) {
        prev->second += bytes;
        return;
      }
    }
    free_[addr] = bytes;
  }

  size_t capacity() const { return capacity_; }
  size_t in_use() const { return in_use_; }
  size_t peak() const { return peak_; }
  size_t n_blocks() const { return blocks_.size(); }
  bool pinned() const { return pinned_; }

 private:
  static size_t round_up(size_t b) { return (b + 255) & ~size_t(255); }

  size_t largest_free() const {
    size_t m = 0;
    for (auto& f : free_) m = f.second > m ? f.second : m;
    return m;
  }

  bool same_block(uintptr_t a, uintptr_t b) const {
    for (auto& blk : blocks_) {
      const uintptr_t lo = reinterpret_cast<uintptr_t>(blk.first), hi = lo + blk.second;
      if (a >= lo && a < hi) return b >= lo && b < hi;
    }
    return false;
  }

  void grow(size_t at_least) {
    size_t bytes = min_block_;
    while (bytes < at_least) bytes <<= 1;  // next power of two at or above the request
    void* p = nullptr;
    if (pinned_) {
      if (cudaHostAlloc(&p, bytes, cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        if (!blocks_.empty()) throw std::runtime_error("PinnedArena: cudaHostAlloc failed");
        pinned_ = false;  // no CUDA runtime (CPU-only tests): plain host memory
      }
    }
    if (!pinned_) {
      if (posix_memalign(&p, 4096, bytes) != 0) throw std::bad_alloc();
    }
    blocks_.emplace_back(p, bytes);
    capacity_ += bytes;
    free_[reinterpret_cast<uintptr_t>(p)] = bytes;
  }

  size_t min_block_;
  bool pinned_ = true;
  std::mutex mu_;
  std::vector<std::pair<void*, size_t>> blocks_;
  std::map<uintptr_t, size_t> free_;  // address-ordered
  std::map<uintptr_t, size_t> live_;
  size_t capacity_ = 0, in_use_ = 0, peak_ = 0;
};

}  // namespace

// uint8 CPU tensor over arena memory; the arena, not the tensor, owns the bytes.
static at::Tensor host_tensor(uintptr_t addr, int64_t nbytes) {
  return at::from_blob(reinterpret_cast<void*>(addr), {nbytes}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
}

// Minimum-volume contiguous k-way cut of a topologically ordered graph (the solver behind the
// in-tree "metis" / "dagP" partitioners).  prefix[i] = load of nodes [0, i); cost[i] = bytes that
// cross a cut placed before node i; allowed[i] says whether a cut may be placed there; every part's
// load stays within `cap`.  Dynamic programme over (parts closed, position) with a sliding-window
// minimum over the admissible starts of the current part: O(n_parts * n).  Returns the n_parts - 1
// cut positions, or an empty vector when the bound admits no solution.
std::vector<int64_t> min_volume_cuts(const std::vector<double>& prefix, const std::vector<double>& cost, const std::vector<bool>& allowed, int64_t n_parts,
                                     double cap) {
  const int64_t n = (int64_t)prefix.size() - 1;
  const double inf = std::numeric_limits<double>::infinity();
  if (n <= 0 || n_parts <= 0 || (int64_t)cost.size() < n + 1 || (int64_t)allowed.size() < n + 1) return {};
  std::vector<std::vector<double>> best(n_parts + 1, std::vector<double>(n + 1, inf));
  std::vector<std::vector<int64_t>> back(n_parts + 1, std::vector<int64_t>(n + 1, -1));
  best[0][0] = 0.0;
  for (int64_t k = 1; k <= n_parts; ++k) {
    std::deque<int64_t> window;  // candidate starts j with increasing best[k-1][j]
    int64_t j_next = 0;
    const bool last = k == n_parts;
    for (int64_t i = 1; i <= n; ++i) {
      for (; j_next < i; ++j_next) {
        if (best[k - 1][j_next] < inf) {
          while (!window.empty() && best[k - 1][window.back()] >= best[k - 1][j_next]) window.pop_back();
          window.push_back(j_next);
        }
      }
      while (!window.empty() && prefix[i] - prefix[window.front()] > cap) window.pop_front();
      if (window.empty()) continue;
      if (last ? i != n : !allowed[i]) continue;
      const int64_t j = window.front();
      best[k][i] = best[k - 1][j] + (last ? 0.0 : cost[i]);
      back[k][i] = j;
    }
  }
  if (best[n_parts][n] == inf) return {};
  std::vector<int64_t> cuts;
  int64_t i = n;
  for (int64_t k = n_parts; k >= 1; --k) {
    i = back[k][i];
    cuts.push_back(i);
  }
  std::sort(cuts.begin(), cuts.end());
  cuts.erase(cuts.begin());  // the leading 0
  return cuts;
}

void register_host_runtime(pybind11::module_& m) {
  m.def("min_volume_cuts", &min_volume_cuts, "minimum-volume contiguous k-way cut (dynamic programme)", py::arg("prefix"), py::arg("cost"), py::arg("allowed"),
        py::arg("n_parts"), py::arg("cap"));
  m.def("host_tensor", &host_tensor, "view arena memory as a uint8 CPU tensor");
  py::class_<PinnedArena>(m, "PinnedArena")
      .def(py::init<size_t>(), py::arg("min_block_bytes") = size_t(64) << 20)
      .def("reserve", &PinnedArena::reserve)
      .def("allocate", &PinnedArena::allocate)
      .def("release", &PinnedArena::release)
      .def_property_readonly("capacity", &PinnedArena::capacity)
      .def_property_readonly("in_use", &PinnedArena::in_use)
      .def_property_readonly("peak", &PinnedArena::peak)
      .def_property_readonly("n_blocks", &PinnedArena::n_blocks)
      .def_property_readonly("pinned", &PinnedArena::pinned);
}
