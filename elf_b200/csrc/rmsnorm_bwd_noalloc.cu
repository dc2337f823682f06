// Allocation-free RMSNorm backward (see rmsnorm_bwd_noalloc.h for the contract).
//
// The kernels are the regular ones (fused_ops.cu); only the source of the scratch differs: a
// file-scope __device__ array.  In host code the array's name is merely a handle for the
// runtime, not a device address, so the address is obtained once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels get.
#include "rmsnorm_bwd_noalloc.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <mutex>

#include "fused_ops.h"

namespace {

constexpr int kMaxDevices = 64;

// Column-sum partials: rmsnorm_backward_blocks() row groups x dim floats.
static __device__ __align__(256) float g_rms_dw_scratch[ELFB_NOALLOC_SCRATCH_BYTES / sizeof(float)];

float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;
thread_local char g_error[256] = "";

int fail(int code, const char* what, const char* detail = "") {
  snprintf(g_error, sizeof(g_error), "elfb_rmsnorm_backward_noalloc: %s%s", what, detail);
  return code;
}

// Device address of the scratch array on the current device (looked up on first use).
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ELFB_NOALLOC_CUDA_ERROR, "cudaGetDevice failed: ", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(ELFB_NOALLOC_CUDA_ERROR, "device index out of the supported range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rms_dw_scratch);
    if (e != cudaSuccess || p == nullptr) return fail(ELFB_NOALLOC_CUDA_ERROR, "cudaGetSymbolAddress failed: ", cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return ELFB_NOALLOC_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int elfb_rmsnorm_backward_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, int rows, int dim,
                                             void* stream) {
  g_error[0] = '\0';
  if (rows < 0 || dim <= 0) return fail(ELFB_NOALLOC_BAD_SIZE, "rows must be >= 0 and dim > 0");
  if (dim % 8 != 0) return fail(ELFB_NOALLOC_BAD_SIZE, "dim must be a multiple of 8");
  if (dim > ELFB_NOALLOC_MAX_DIM) {
    char detail[96];
    snprintf(detail, sizeof(detail), "dim %d exceeds the built-in scratch (maximum %d)", dim, ELFB_NOALLOC_MAX_DIM);
    return fail(ELFB_NOALLOC_BAD_SIZE, detail);
  }
  if ((size_t)elfb::rmsnorm_backward_min_blocks() * (size_t)dim * sizeof(float) > (size_t)ELFB_NOALLOC_SCRATCH_BYTES)
    return fail(ELFB_NOALLOC_BAD_SIZE, "problem does not fit the built-in scratch");
  if (rows == 0) return ELFB_NOALLOC_OK;
  if (!dy || !x || !w || !rstd || !dx || !dw) return fail(ELFB_NOALLOC_BAD_POINTER, "null pointer argument");
  if (!aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx) || !aligned16(dw))
    return fail(ELFB_NOALLOC_BAD_POINTER, "dy, x, w, dx and dw must be 16-byte aligned");
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != ELFB_NOALLOC_OK) return rc;
  const cudaError_t e = elfb::rmsnorm_backward(dy, x, w, rstd, /*dres_in=*/nullptr, dx, scratch, /*scratch_rows=*/(int)((size_t)ELFB_NOALLOC_SCRATCH_BYTES / sizeof(float) / (size_t)dim), dw, /*dw_bf16=*/false,
                                               /*accumulate_dw=*/false, rows, dim,
                                               static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(ELFB_NOALLOC_CUDA_ERROR, "kernel launch failed: ", cudaGetErrorString(e));
  return ELFB_NOALLOC_OK;
}

extern "C" const char* elfb_noalloc_last_error(void) { return g_error; }
