// Entry point for callers that cannot allocate device memory.
//
// This function has no counterpart in the reference implementation; it exists only in this library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a plug-in that executes inside
// another framework's stream callback or graph-building phase, a real-time loop that may not touch the
// allocator once it is running, and a host that has handed all device memory to its own pool and gives
// guests no way to get more.  Such callers can still own the tensors they pass in, but they cannot hand us
// the extra workspace that llmq_rmsnorm_backward() asks for.
//
// What it does: exactly what llmq_rmsnorm_backward() does (dinp += norm gradient, dweight (+)= sum over
// rows, optional abs-max of dinp), but the per-CTA partial sums of the weight gradient are kept in a
// fixed array inside the library (LLMQ_NOALLOC_SCRATCH_FLOATS floats, about 9.3 MiB, resident on every
// GPU that loads the library, until the process ends).  It calls neither cudaMalloc nor cudaFree nor any
// allocating library routine.
//
// Limits and rules:
//  * C must be at most LLMQ_NOALLOC_MAX_C (and a multiple of the 16-byte vector width: 8 for bf16, 4 for
//    fp32); a larger C is refused with LLMQ_NOALLOC_ERR_TOO_LARGE and nothing is launched.  Any row count works.
//  * The first call on each device looks up the device address of the array (cudaGetSymbolAddress, with
//    that device current).  Make that first call before starting any stream capture on that device.
//  * All calls on one device share the array.  Nothing in it has to start at zero: every slot is written
//    by the first kernel of a call before the second kernel of the same call reads it, so leftovers of an
//    earlier call are harmless.  Two calls whose kernels overlap on the GPU (different streams) would
//    overwrite each other's partial sums: run calls on one stream, or order them with events.
//  * dtype: 0 = bf16, 3 = fp32.  Returns 0 on success, a CUDA error code, or one of the negative codes below.
#pragma once
#include <cuda_runtime.h>

#define LLMQ_NOALLOC_MAX_C 8192
#define LLMQ_NOALLOC_SCRATCH_FLOATS (296 * LLMQ_NOALLOC_MAX_C)
#define LLMQ_NOALLOC_ERR_TOO_LARGE (-20)
#define LLMQ_NOALLOC_ERR_DEVICE (-21)

extern "C" int llmq_rmsnorm_backward_noalloc(void* dinp, void* dweight, const void* dout, const void* inp,
                                             const void* weight, const float* rstd, int rows, int C, int dtype,
                                             float* absmax, int accumulate_dweight, cudaStream_t stream);
