// Entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference: it exists for programs that embed these
// kernels somewhere cudaMalloc is off the table.  Examples: a serving process that
// handed every byte of device memory to its weight and cache pools at start-up, so a
// later cudaMalloc simply fails; a step loop with a latency budget, where cudaMalloc or
// cudaFree would stall every stream of the device; a plug-in whose host forbids
// allocation after initialisation.  Such a caller cannot provide the scratch buffers the
// many-block argmax needs, and cannot let the library allocate them either.
//
// ifx_argmax_no_alloc does the same work as ifx_argmax_chunks (argmax of each row of
// float32 logits, ties to the lower index) but keeps its scratch in a fixed array that
// is part of the library image: 67,584 bytes per GPU that loads the library, held until
// the process exits.  The caller passes only the input and the output.
//
//   logits  float32 [rows, vocab] on the current device
//   out     int32 [rows] on the current device
//   rows    1 .. 256   (IFX_NO_ALLOC_MAX_ROWS); more is refused with IFX_E_TOOBIG (-4)
//   vocab   1 .. 2^30
//   returns 0, a negative IFX_E_* code for refused arguments, or a positive cudaError_t
//
// Set-up: the first call on each device looks up the device address of the scratch
// array (cudaGetSymbolAddress) with that device current.  Make that first call during
// start-up, outside any stream capture; later calls only launch work on `stream`.
// Neither the first nor later calls call cudaMalloc, cudaFree or any allocating routine.
//
// Sharing: every call on a device uses the same array, and the array keeps what the last
// call left in it.  The part that must start at zero (one counter per row) is cleared on
// `stream` at the start of each call.  Two calls that can overlap on the GPU (different
// streams without an ordering between them) race on the array and give wrong results:
// order them.
#pragma once

#include <cuda_runtime.h>

#define IFX_NO_ALLOC_MAX_ROWS 256
#define IFX_NO_ALLOC_CHUNKS 32
#define IFX_NO_ALLOC_SCRATCH_BYTES (IFX_NO_ALLOC_MAX_ROWS * IFX_NO_ALLOC_CHUNKS * 8 + IFX_NO_ALLOC_MAX_ROWS * 8)

#ifdef __cplusplus
extern "C"
#endif
int ifx_argmax_no_alloc(const float* logits, int* out, int rows, int vocab, cudaStream_t stream);
