// b200_skinny_gemm_static: the weight-streaming matrix product for callers that cannot allocate.
//
// This entry point has no counterpart in the reference project; it exists for embedders of
// this library. Some callers run where device allocation is off the table: inside a stream
// capture, inside another runtime's allocator-owned region, in a process whose memory plan
// was fixed at start-up, or in a real-time loop where cudaMalloc's implicit synchronisation
// is not acceptable. b200_skinny_gemm (gemm_skinny.cu) makes such callers provide scratch
// memory for the partial sums of blocks that split K. This variant brings its own: a
// file-scope device array of kStaticScratchFloats 32-bit words (512 KiB) plus
// kStaticCounters arrival counters, which every GPU that loads the library holds until
// the process exits.
//
//   Y[M,N] = X[M,K] * W[N,K]^T,  M <= 16, K a multiple of 8, bfloat16 operands 16-byte aligned;
//   epilogue 0 = bfloat16 Y, 1 = float32 Y, 2 = SwiGLU over interleaved gate/up rows of W.
//
// Rules for callers:
//  * Inputs and the output are the caller's; the function calls no cudaMalloc, cudaFree or
//    any allocating library routine.
//  * A shape whose partial sums do not fit the static array is refused with an error that
//    names the need and the limit (b200_last_error()); nothing is launched.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current). Make that first call outside any
//    stream capture.
//  * The kernel starts only after everything before it on the stream has finished (it is not
//    launched for programmatic overlap), so W, like X, may be written by the work just before it.
//  * All calls on a device share the one array. It keeps whatever the last call left; the
//    arrival counters, the only part that must start at zero, are cleared on the stream
//    before every launch. Two calls whose kernels can overlap on the GPU (different streams,
//    or kernels allowed to overlap on one stream) would race on it: serialise them.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, a negative value after storing a message for b200_last_error().
int b200_skinny_gemm_static(const void* W, const void* X, void* Y, int M, int N, int K, int epilogue,
                            cudaStream_t stream);

// The static scratch's capacity, for callers that want to check a shape up front.
long long b200_skinny_gemm_static_capacity_floats(void);

#ifdef __cplusplus
}
#endif
