// airun_gemm_tcgen05_static: the split-K tensor-core matrix product for callers that
// cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for users of
// this library.  Some of them run where cudaMalloc is off limits: inside a region that is
// being captured into a CUDA graph, in a process whose memory is handed out once by a
// framework's pool, or in a plug-in that is only given input and output buffers.  The
// regular entry point (airun_gemm_tcgen05) needs two scratch buffers from its caller when
// the product is cut into K slices: float partial tiles and one counter per tile.  This
// variant brings its own: two file-scope arrays in device memory that belong to the
// library.
//
//   out[M][N] = x[M][K] * W[N][K]^T        (same arguments and modes as airun_gemm_tcgen05,
//                                           without the scratch and counter pointers)
//
// Limits.  The arrays hold AIRUN_STATIC_SCRATCH_FLOATS floats (16 MiB) and
// AIRUN_STATIC_COUNTERS counters; every GPU on which the library is loaded keeps that much
// memory until the process ends.  Of the two builds of gemm_tcgen05.cu only the plain one (without
// AIRUN_FOLD_NORM) carries the arrays and exports this symbol, so a process that loads both
// libraries still holds them once.  A call that would need more (tiles * ksplit * bn * 128
// floats, or more tiles than counters) is refused with AIRUN_ERR_STATIC_TOO_LARGE before
// anything is launched; use fewer slices or the regular entry point.
//
// First call.  The device addresses of the arrays are looked up with
// cudaGetSymbolAddress the first time the function is called on a device (with that
// device current).  Make that first call outside any stream capture.
//
// Sharing.  All calls on a device use the same arrays.  The function clears the counters
// it is about to use (a memset on the caller's stream) and the kernel overwrites the
// partial tiles before it reads them, so calls that follow one another on one stream are
// independent.  Calls that overlap on the GPU (two streams, two threads, two processes
// sharing a context) would write the same scratch at once: do not overlap them.
//
// It calls no cudaMalloc, cudaFree or other allocating routine.
#pragma once
#include <cuda_runtime.h>

#define AIRUN_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define AIRUN_STATIC_COUNTERS 4096
#define AIRUN_ERR_STATIC_TOO_LARGE 1002
#define AIRUN_ERR_STATIC_SETUP 1003

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or AIRUN_ERR_ARG (1000) / AIRUN_ERR_UNSUPPORTED (1001) as the regular entry
// point does, AIRUN_ERR_STATIC_TOO_LARGE when the launch needs more scratch than the
// library holds, AIRUN_ERR_STATIC_SETUP when the address lookup failed, or a CUDA error
// code from the launch.
int airun_gemm_tcgen05_static(const void* x, const void* W, void* out, int M, int N, int K,
                              long long ldx, long long ldw, long long ldc, int epi, int swap, int bn,
                              int ksplit, int* err, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
