// Symmetric memory on CUDA virtual-memory management, without a library in between: one physical
// allocation per rank, exported as a POSIX file descriptor, imported and mapped by the other ranks
// of the node, so that every rank holds a device address for every rank's buffer (plain peer
// loads / stores over NVLink; no multicast object is created).
//
// The reference has no counterpart: its data-parallel traffic goes through an NCCL communicator
// (elf/execution/block.py:506-527).  Here the gradient exchange and the stage-to-stage rings
// write straight into peers' memory, which needs exactly this: allocate, exchange handles, map.
// The default provider of such buffers is torch.distributed._symmetric_memory; this runtime is
// the alternative selected with ELF_B200_SYMM=vmm (elf_b200/parallel/symm.py), for hosts whose
// torch build has no symmetric memory and for callers that want to own the mapping's lifetime.
//
// The driver API is reached through cudaGetDriverEntryPoint, so the extension has no link-time
// dependency on libcuda and still loads on machines without a GPU.  The file descriptors travel
// between the processes in Python (UNIX-domain sockets, SCM_RIGHTS).
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <torch/extension.h>
#include <unistd.h>

#include <cstdint>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

template <class F>
F driver_entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
  TORCH_CHECK(p != nullptr, "CUDA driver entry point ", name, " is not available");
  return reinterpret_cast<F>(p);
}

struct Driver {
  decltype(&cuMemGetAllocationGranularity) granularity = driver_entry<decltype(&cuMemGetAllocationGranularity)>("cuMemGetAllocationGranularity");
  decltype(&cuMemCreate) create = driver_entry<decltype(&cuMemCreate)>("cuMemCreate");
  decltype(&cuMemRelease) release = driver_entry<decltype(&cuMemRelease)>("cuMemRelease");
  decltype(&cuMemAddressReserve) reserve = driver_entry<decltype(&cuMemAddressReserve)>("cuMemAddressReserve");
  decltype(&cuMemAddressFree) address_free = driver_entry<decltype(&cuMemAddressFree)>("cuMemAddressFree");
  decltype(&cuMemMap) map = driver_entry<decltype(&cuMemMap)>("cuMemMap");
  decltype(&cuMemUnmap) unmap = driver_entry<decltype(&cuMemUnmap)>("cuMemUnmap");
  decltype(&cuMemSetAccess) set_access = driver_entry<decltype(&cuMemSetAccess)>("cuMemSetAccess");
  decltype(&cuMemExportToShareableHandle) export_handle = driver_entry<decltype(&cuMemExportToShareableHandle)>("cuMemExportToShareableHandle");
  decltype(&cuMemImportFromShareableHandle) import_handle = driver_entry<decltype(&cuMemImportFromShareableHandle)>("cuMemImportFromShareableHandle");
};

const Driver& driver() {
  static const Driver d;
  return d;
}

void check(CUresult r, const char* what) { TORCH_CHECK(r == CUDA_SUCCESS, "symmetric memory: ", what, " failed (CUresult ", (int)r, ")"); }

struct Mapping {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr ptr = 0;
  size_t bytes = 0;
};

// One rank's end of a symmetric buffer: its own allocation plus the mappings of its peers'.
class VmmArena {
 public:
  VmmArena(size_t bytes, int device) : device_(device) {
    TORCH_CHECK(bytes > 0, "symmetric memory: empty allocation");
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
    TORCH_CHECK(cudaFree(nullptr) == cudaSuccess, "symmetric memory: no CUDA context on device ", device);
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    check(driver().granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    own_.bytes = (bytes + gran - 1) / gran * gran;
    granularity_ = gran;
    check(driver().create(&own_.handle, own_.bytes, &prop, 0), "cuMemCreate");
    map_here(own_);
    TORCH_CHECK(cudaMemset(reinterpret_cast<void*>(own_.ptr), 0, own_.bytes) == cudaSuccess, "symmetric memory: clearing the allocation failed");
    TORCH_CHECK(cudaDeviceSynchronize() == cudaSuccess, "symmetric memory: synchronisation failed");
  }
  VmmArena(const VmmArena&) = delete;
  VmmArena& operator=(const VmmArena&) = delete;
  ~VmmArena() {
    for (Mapping& m : peers_) unmap(m);
    unmap(own_);
  }

  size_t bytes() const { return own_.bytes; }
  int device() const { return device_; }
  uint64_t address() const { return static_cast<uint64_t>(own_.ptr); }

  // A file descriptor for this rank's allocation; the receiver (another process) imports it and
  // both sides close their copy afterwards.
  int export_fd() const {
    int fd = -1;
    check(driver().export_handle(&fd, own_.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
    return fd;
  }

  // Map a peer's allocation (same size as ours) into this process for this device; closes `fd`.
  // Returns the index under which its address and tensor view are available.
  int import_peer(int fd) {
    c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device_));
    Mapping m;
    m.bytes = own_.bytes;
    const CUresult r = driver().import_handle(&m.handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    ::close(fd);
    check(r, "cuMemImportFromShareableHandle");
    map_here(m);
    peers_.push_back(m);
    return static_cast<int>(peers_.size()) - 1;
  }

  uint64_t peer_address(int index) const {
    TORCH_CHECK(index >= 0 && index < (int)peers_.size(), "symmetric memory: no such peer mapping");
    return static_cast<uint64_t>(peers_[index].ptr);
  }

  // uint8 views; they borrow the mapping, so the arena must outlive them (the Python wrapper keeps it).
  at::Tensor tensor() const { return view(own_); }
  at::Tensor peer_tensor(int index) const {
    TORCH_CHECK(index >= 0 && index < (int)peers_.size(), "symmetric memory: no such peer mapping");
    return view(peers_[index]);
  }

 private:
  void map_here(Mapping& m) {
    CUresult r = driver().reserve(&m.ptr, m.bytes, granularity_, 0, 0);
    if (r != CUDA_SUCCESS) {
      driver().release(m.handle);
      m.handle = 0;
      check(r, "cuMemAddressReserve");
    }
    r = driver().map(m.ptr, m.bytes, 0, m.handle, 0);
    if (r == CUDA_SUCCESS) {
      CUmemAccessDesc access = {};
      access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      access.location.id = device_;
      access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      r = driver().set_access(m.ptr, m.bytes, &access, 1);
      if (r != CUDA_SUCCESS) driver().unmap(m.ptr, m.bytes);
    }
    if (r != CUDA_SUCCESS) {
      driver().address_free(m.ptr, m.bytes);
      driver().release(m.handle);
      m = Mapping{};
      check(r, "cuMemMap / cuMemSetAccess");
    }
  }
  void unmap(Mapping& m) {
    if (m.ptr != 0) {
      driver().unmap(m.ptr, m.bytes);
      driver().address_free(m.ptr, m.bytes);
    }
    if (m.handle != 0) driver().release(m.handle);
    m = Mapping{};
  }
  at::Tensor view(const Mapping& m) const {
    // The view belongs to THIS rank's device whichever GPU holds the memory: a peer's allocation is
    // physically elsewhere, and work on the view runs here and crosses NVLink.  Naming the target
    // device keeps from_blob from asking the driver where the pointer lives and rejecting the answer.
    const c10::Device here(at::kCUDA, static_cast<c10::DeviceIndex>(device_));
    return at::for_blob(reinterpret_cast<void*>(m.ptr), {static_cast<int64_t>(m.bytes)})
        .deleter([](void*) {})
        .options(at::TensorOptions().dtype(at::kByte).device(here))
        .target_device(here)
        .make_tensor();
  }

  int device_;
  size_t granularity_ = 0;
  Mapping own_;
  std::vector<Mapping> peers_;
};

}  // namespace

void register_symm_runtime(pybind11::module_& m) {
  py::class_<VmmArena>(m, "VmmArena", "one rank's end of a symmetric buffer on CUDA virtual memory (see elf_b200/parallel/symm.py)")
      .def(py::init<size_t, int>(), py::arg("bytes"), py::arg("device"))
      .def_property_readonly("bytes", &VmmArena::bytes)
      .def_property_readonly("device", &VmmArena::device)
      .def_property_readonly("address", &VmmArena::address)
      .def("export_fd", &VmmArena::export_fd)
      .def("import_peer", &VmmArena::import_peer, py::arg("fd"))
      .def("peer_address", &VmmArena::peer_address, py::arg("index"))
      .def("tensor", &VmmArena::tensor)
      .def("peer_tensor", &VmmArena::peer_tensor, py::arg("index"));
}
