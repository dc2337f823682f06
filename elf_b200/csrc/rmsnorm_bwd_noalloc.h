// RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for two kinds of
// callers of this library:
//   * runtimes that execute a stage under a memory plan fixed in advance (the ILP-planned
//     schedules account for every megabyte of a step; a scratch allocation inside a backward
//     op, which may also make the driver synchronise the device, is outside that plan);
//   * hosts written in plain C/C++ that link the kernels without PyTorch and therefore have no
//     caching allocator to hand scratch buffers out of.
// The regular path (`elfb::rmsnorm_backward` in fused_ops.h, reached from Python through
// `rmsnorm_bwd`) takes its column-sum scratch from the caller or from torch's allocator.  Here
// the scratch lives in a fixed array inside the library instead.
//
// Contract
//   * Computes dx[rows][dim] and dw[dim] (overwritten, fp32) exactly like the regular path
//     without a residual gradient.  dy, x, w, dx are bf16, row-major, contiguous, 16-byte
//     aligned; rstd is the fp32 [rows] vector the forward produced.
//   * Limits: dim must be a multiple of 8 and at most ELFB_NOALLOC_MAX_DIM (8192).  `rows` is
//     not limited.  The scratch array is ELFB_NOALLOC_SCRATCH_BYTES (2 MiB) of device memory
//     per GPU that has this library loaded, held until the process exits.
//   * Calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on
//     each device looks up the device address of the scratch array (cudaGetSymbolAddress) and
//     caches it; make that first call before starting any stream capture on that device.
//   * All calls on a device share the one scratch array.  Nothing in it needs to be zero on
//     entry (every call rewrites the part it reads), but two calls whose kernels overlap on
//     the GPU - different streams, or different host threads on different streams - race on
//     it.  Serialise them on one stream or with events.
//   * Returns 0 on success, a negative code otherwise; `elfb_noalloc_last_error()` describes
//     the most recent failure of the calling thread.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ELFB_NOALLOC_MAX_DIM 8192
#define ELFB_NOALLOC_SCRATCH_BYTES (64 * ELFB_NOALLOC_MAX_DIM * 4)

#define ELFB_NOALLOC_OK 0
#define ELFB_NOALLOC_BAD_SIZE (-1)
#define ELFB_NOALLOC_BAD_POINTER (-2)
#define ELFB_NOALLOC_CUDA_ERROR (-3)

// `stream` is a cudaStream_t (0 for the default stream).
__attribute__((visibility("default"))) int elfb_rmsnorm_backward_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                                                        void* dx, float* dw, int rows, int dim, void* stream);

__attribute__((visibility("default"))) const char* elfb_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
