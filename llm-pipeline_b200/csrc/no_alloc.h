// An entry point of this library that never allocates device memory.
//
// It has no counterpart in DavidAkinpelu/llm-pipeline: it exists for hosts of this library, not for
// parity with the reference.
//
// Who needs it. Some programs that embed these kernels cannot ask the CUDA runtime for memory at
// the moment they call us: a server that handed every free byte of the GPU to its own page pool at
// start-up (a later cudaMalloc simply fails there), or a caller on a path where an allocation's
// device-wide synchronisation, or its possible failure, is not acceptable. The regular argmax entry
// point (llmp_argmax) takes a scratch buffer that somebody has to allocate; this one brings its own.
//
// What it does. llmp_argmax_no_alloc computes, for each of M rows of float32 logits, the index of the
// largest value (the lowest index among equal values), exactly like llmp_argmax with a scratch
// buffer. Its scratch (the per-slice winners of the first pass) is a fixed array inside the library
// image: LLMP_NO_ALLOC_MAX_ROWS rows x 32 slices x 8 bytes = 256 KiB, which every GPU that loads the
// library holds until the process exits. Inputs and outputs are still the caller's.
//
// Rules.
// * M must be in 1..LLMP_NO_ALLOC_MAX_ROWS and V in 1..2^31-1, else the call returns non-zero and
//   llmp_last_error() says why; nothing is launched.
// * The first call on a device looks up the device address of the array (cudaGetSymbolAddress, with
//   that device current) and remembers it; make this first call before you start any stream capture.
// * All calls on one GPU share the one array, and it keeps what the last call left. Nothing in it has
//   to start at zero: a call writes every slot it later reads. But two calls that overlap on the GPU
//   (different streams, no dependency between them) race on it and may both return wrong indices:
//   order such calls yourself.
// * It calls no cudaMalloc, cudaFree or any allocating library routine.
#pragma once

#include <cuda_runtime.h>

#define LLMP_NO_ALLOC_MAX_ROWS 1024

extern "C" __attribute__((visibility("default")))
int llmp_argmax_no_alloc(const float* logits, long row_stride, int M, int V, int* out, cudaStream_t stream);
