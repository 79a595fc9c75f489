// LayerNorm backward without any allocation.  (This entry point has no counterpart in the reference, which
// has no native code at all; it exists for embedders of this library.)
//
// Who needs it: code that drives these kernels from a place where allocating device memory is forbidden or
// impossible - a plug-in running inside a host application that owns the whole memory pool and hands out only
// the input and output buffers, a real-time loop that may not take the allocator's lock, or a region of a
// program (a stream-ordered section, a signal-driven callback) in which cudaMalloc / cudaFree and every
// allocating library routine - the tensor allocator of the Python framework included - are off limits.
// tsp_layernorm_bwd() needs a scratch buffer for its per-block partial sums of dw and db, and its callers
// usually get that buffer from an allocator; this variant keeps the scratch in a fixed array inside the
// library instead.
//
// int tsp_layernorm_bwd_noalloc(dy, x, w, mean, rstd, dx, dw, db, rows, d, dtype, stream)
//   Same math and argument meaning as tsp_layernorm_bwd (minus its `partial` argument):
//     dy, x   [rows, d] activations (dtype: TSP_DTYPE_F32 or TSP_DTYPE_BF16), w [d] fp32 weight,
//     mean, rstd [rows] fp32 statistics saved by the forward pass,
//     dx      [rows, d] output, same dtype;  dw, db [d] fp32 outputs.
//   The caller still passes all inputs and outputs; all must be device memory of the current device.
//   Returns 0 on success, a cudaError_t value (> 0) if the runtime refused something, -3 for a shape or dtype
//   the kernel does not support (d not a multiple of 8, unknown dtype), and
//   TSP_NOALLOC_ERR_TOO_LARGE (-4) when the request does not fit the built-in scratch: d larger than
//   TSP_NOALLOC_LN_MAX_D, or a device ordinal of TSP_NOALLOC_MAX_DEVICES or more.  `rows` has no limit of its
//   own: more rows only mean more rows per block.
//
// Limits and rules:
//   * The scratch is TSP_NOALLOC_LN_MAX_BLOCKS * 2 * TSP_NOALLOC_LN_MAX_D floats = 148 * 2 * 1024 * 4 B
//     = 1.16 MiB of device memory.  Every GPU on which the library gets loaded holds it until the process ends,
//     whether or not this function is ever called.
//   * It calls no cudaMalloc, cudaFree or other allocating routine.
//   * The first call on each device looks up the device address of the scratch array (one runtime query,
//     result cached per device).  Make that first call with the right device current and before starting
//     any stream capture; later calls only launch kernels.
//   * All calls on a device share the one array and it keeps whatever the last call wrote.  No call relies on
//     its previous contents (each block rewrites its own slice before the reduction reads it), but two calls
//     whose kernels overlap in time on the GPU - different streams, no ordering between them - race on it and
//     give wrong dw/db.  Order such calls on one stream or with events.
//   * Results match tsp_layernorm_bwd up to floating-point summation order (it may use fewer, larger blocks).
#pragma once
#include <cuda_runtime.h>

#define TSP_NOALLOC_LN_MAX_D 1024
#define TSP_NOALLOC_LN_MAX_BLOCKS 148
#define TSP_NOALLOC_MAX_DEVICES 64
#define TSP_NOALLOC_ERR_TOO_LARGE (-4)

#ifdef __cplusplus
extern "C" {
#endif

int tsp_layernorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* mean, const float* rstd,
                              void* dx, float* dw, float* db, int rows, int d, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
