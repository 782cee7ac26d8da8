// Allocation-free C entry point for the per-expert bias gradient.
//
// This entry point has no counterpart in the reference: FastMoE computes the bias gradient
// with its column_reduce kernel inside linear_backward and always goes through torch's
// allocator.  It exists for callers that are not allowed to allocate device memory when they
// need the result: code that runs while a stream is being captured, code inside a memory
// pool that is closed for the step, a serving runtime with a fixed memory plan, or a plugin
// loaded through the C ABI without access to torch's allocator.  The regular path
// (ops/grouped_gemm.py::bias_grad) asks torch for an fp32 accumulation buffer on every call;
// here that buffer is a fixed array inside the library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest num_groups * n the built-in accumulation array can hold (fp32 elements, 256 KiB).
// Every GPU that loads the library keeps this array until the process exits.
#define FMOE_NOALLOC_MAX_ELEMS 65536

// out[g, :] = sum of the rows x[offs[g] : offs[g + 1], :]   for g in [0, num_groups)
//
//   x         device, [rows_cap, n], bf16 (dtype 0) or fp16 (dtype 1), 16-byte aligned, n % 8 == 0
//   offs      device, int32 [num_groups + 1], ascending row offsets; rows at or past rows_cap
//             are not read, whatever the offsets say
//   out       device, [num_groups, n], same dtype as x
//   stream    stream of the CURRENT device on which the three kernels (clear, accumulate,
//             convert) are enqueued
//
// Misaligned pointers, a stream of another device and sizes the launch cannot express
// (n > 16,776,960) are refused with -1 before anything is launched.
//
// Returns 0 on success, a negative value otherwise (fmoe_noalloc_last_error() describes it):
//   -1 bad argument, -2 num_groups * n exceeds FMOE_NOALLOC_MAX_ELEMS, -3 CUDA error.
//
// Nothing is allocated: no cudaMalloc/cudaFree, no library routine that allocates.  The first
// call on a device looks up the address of the built-in array (cudaGetSymbolAddress with that
// device current); make that first call before starting any stream capture.  All calls on a
// device share the one array: it is cleared at the start of each call, and two calls whose
// kernels can overlap on the GPU (different streams without an ordering) race on it.
int fmoe_bias_grad_noalloc(const void* x, const int* offs, int num_groups, long rows_cap, int n,
                           int dtype, void* out, cudaStream_t stream);

const char* fmoe_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
