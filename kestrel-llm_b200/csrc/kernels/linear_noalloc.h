// kestrel_linear_bf16_noalloc - a matrix product for callers that must not allocate.
//
// This entry point has no counterpart in the reference engine (which runs on CPUs and has no
// device memory to manage).  It exists for users of this library who cannot call cudaMalloc at
// the moment they need a product: a host application that handed the whole device to an arena
// of its own at start-up and gives libraries no way to ask for more; or a latency-bound loop in
// which an allocation is unacceptable because cudaMalloc may synchronise the device and takes
// driver locks.  The library's usual route, kestrel_gemm_tc, writes split-K slices into a
// scratch buffer that the caller (in this package: the Python layer, through torch) allocates
// per call.  Here the scratch is a fixed array inside the library instead.
//
//   out[t, n] = sum_k x[t, k] * w[n, k] (+ bias[n])
//
//   x    bfloat16 [T, K], row stride ldx elements      w   bfloat16 [N, K], row stride ldw
//   bias float32 [N] or NULL                            out [T, N] contiguous, float32 (out_dtype 0)
//                                                           or bfloat16 (out_dtype 1)
//
// The caller passes inputs and the output; the function calls no cudaMalloc, cudaFree or any
// allocating routine of a library.  Returns 0, or a negative code with the text in
// kestrel_last_error().
//
// Limits and rules
//  * Scratch: KESTREL_NOALLOC_SCRATCH_BYTES (16 MiB) in a file-scope __device__ array.  Every
//    GPU on which this library is loaded holds these 16 MiB until the process exits.  A product
//    whose slices need more (slices * T * N * 4 bytes, slices as kestrel_gemm_tc_splits gives
//    them) is refused with an error that names the sizes; nothing is launched then.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and keeps it.  Make this first call before any stream capture begins.
//  * All calls share the one array, and it keeps what the last call left.  Nothing in it has to
//    start at zero: the product writes every slice element it later reads.  Two calls whose
//    kernels can overlap on the GPU (different streams without an ordering between them) race
//    on the array; keep calls on one stream, or order them with events.
//  * Operand rules are those of kestrel_gemm_tc: K, ldx and ldw multiples of 8, x and w 16-byte
//    aligned.
#pragma once
#include <cuda_runtime.h>

#define KESTREL_NOALLOC_SCRATCH_BYTES (16u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int kestrel_linear_bf16_noalloc(const void *x, const void *w, const float *bias, void *out, int out_dtype,
                                int T, int N, int K, long long ldx, long long ldw, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
