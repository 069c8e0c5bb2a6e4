// Entry points of libntb_kernels.so that never allocate device memory.
//
// This header has no counterpart in the reference framework (which has no native kernels at all); it exists for callers of
// this library that are not allowed to allocate: hooks called from inside another allocator, and serving / embedded runtimes
// that reserve all device memory up front.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest `cols` accepted by ntb_rmsnorm_bwd_noalloc (8192).
int ntb_rmsnorm_bwd_noalloc_max_cols();

// RMSNorm backward with the dW partial-sum scratch held in a fixed 4.6 MiB array inside the library image instead of a
// caller buffer.  The CUDA runtime loads kernel modules lazily, so a GPU starts to hold those 4.6 MiB when this library's
// module is first loaded on it (at the latest: the first call of this entry point there) and keeps them until the process exits.  Same maths and argument meaning as ntb_norm_bwd(is_rms = 1):
//   dtype : 0 fp32, 1 bf16, 2 fp16 (dy, pre, w, dres, dx)
//   dy, pre, dres (nullable), dx : [rows, cols];  w : [cols];  rstd : fp32 [rows];  dw_out : fp32 [cols]
// Returns 0 on success, 1 for unsupported sizes (cols > 8192, cols % 8 != 0, empty), 2 for a CUDA error.
// Calls no cudaMalloc / cudaFree and no allocating library routine.  The first call on a device resolves the array's
// device address (cudaGetSymbolAddress), which may load the module and so reserve the array: make that call once per device
// at start-up, while memory can still be reserved (otherwise it can fail with code 2) and before any stream capture.
// The address cache is a plain per-device table without locks: concurrent first calls from several host threads all
// resolve the same address, so they are harmless, but make the start-up call from one thread if in doubt.
// All calls share the array: launches that may overlap on the GPU must be ordered by the caller.
int ntb_rmsnorm_bwd_noalloc(int dtype, const void* dy, const void* pre, const void* w, const float* rstd, const void* dres, void* dx, float* dw_out, int rows,
                            int cols, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
