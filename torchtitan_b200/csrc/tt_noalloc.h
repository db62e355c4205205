/* Allocation-free entry point of libtt_b200.so.
 *
 * This function has no counterpart in the reference (torchtitan); it exists for embedders of this
 * library that are not allowed to allocate device memory when they call into it: code running under
 * a memory budget fixed at start-up, inside a CUDA-graph-style capture window of the host
 * application, or in a process whose allocator is owned by another runtime (so neither cudaMalloc
 * nor the PyTorch caching allocator may be touched from the call site).
 *
 *   int tt_rmsnorm_bwd_noalloc(dy, x, w, rstd, dx, dw, rows, D, dtype, stream)
 *
 * Same computation and argument meaning as tt_rmsnorm_bwd() (RMSNorm backward: dx, and dw when w is
 * given; dtype 0 = bf16, 1 = fp32; rstd is the per-row 1/rms saved by the forward), except that the
 * fp32 [blocks, D] partial sums for dw live in an array built into the library instead of a buffer
 * supplied by the caller. The caller still passes every input and output.
 *
 * Limits and rules
 *  - D must be a multiple of 8 and at most tt_rmsnorm_bwd_noalloc_max_dim() (4096). Larger D is
 *    refused with -20 before anything is launched; tt_noalloc_strerror(code) gives the text.
 *  - The built-in array is 2 * 148 * 4096 floats (about 4.6 MiB) and is part of the library image:
 *    every GPU that loads the library holds it until the process exits.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress with
 *    that device current). Make that first call before starting any stream capture.
 *  - No cudaMalloc, cudaFree or other allocating routine is called, on any call.
 *  - All calls on a device share the one array. It keeps the previous call's partial sums, which is
 *    harmless because each call overwrites every row it later reads; but two calls that overlap on
 *    the GPU (different streams, no ordering between them) race on it. Serialise them.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int tt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                           long long rows, int D, int dtype, cudaStream_t stream);
int tt_rmsnorm_bwd_noalloc_max_dim(void);
const char* tt_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
