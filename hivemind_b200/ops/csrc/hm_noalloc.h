// Allocation-free entry point of libhm_kernels. It has no counterpart in the reference: it is offered to
// callers of this library that are not in a position to allocate device memory at call time, for example a host
// runtime that gave all HBM to its own pool at start-up and forbids cudaMalloc afterwards, or an embedding
// program written in C that wants gradient clipping without pulling in a tensor allocator.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of tensors one call may cover. The scratch array that backs the call is sized for it:
// (HM_NOALLOC_MAX_TENSORS + 1) floats = 16 388 bytes of device memory, resident on every GPU that loads the
// library, from load until the process exits.
#define HM_NOALLOC_MAX_TENSORS 4096

// Global-norm gradient clipping over a multi-tensor table, like hm_mt_sumsq + hm_mt_clip, but the per-tensor
// sums of squares live in a fixed device array inside the library instead of a buffer the caller allocates.
//
//   tensors, chunks, num_chunks : the multi-tensor table (see multi_tensor.cu); slot 0 of every row is scaled in place
//   num_tensors                 : rows of the table; more than HM_NOALLOC_MAX_TENSORS is refused with -20 and a
//                                 message on stderr, and nothing is launched
//   max_norm                    : tensors are multiplied by min(1, max_norm / (global L2 norm + 1e-6))
//   total_norm_out              : optional device pointer; receives the norm before clipping
//   returns 0, a CUDA error code (> 0) or a negative argument error
//
// The call makes no cudaMalloc / cudaFree and calls no allocating library routine. The first call on a device
// looks up the device address of the scratch array (cudaGetSymbolAddress) and keeps it; make that first call
// outside of any stream capture. All calls share the one array: it is cleared at the start of every call (the
// previous call's sums are still in it), and two calls whose kernels overlap on the GPU — different streams, or
// different host threads — would race on it, so serialise them.
int hm_mt_clip_grad_norm_noalloc(const void* tensors, const void* chunks, int num_chunks, int num_tensors,
                                 float max_norm, float* total_norm_out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
