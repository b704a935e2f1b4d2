// Shared declarations of the sm_100a kernel library: storage types, error reporting and the
// conventions of the exported C entry points.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and a CUDA stream,
// launches on that stream without synchronising, and returns 0 or a negative code; the
// message of the last failure on the calling thread is read with kestrel_last_error().
// Storage type codes: 0 = float32, 1 = bfloat16.  Sums, norms, softmax, rotation angles and
// the residual stream are float32 whatever the storage type.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// every exported entry point is declared in the package's one C header; a definition that
// differs from its declaration there does not compile
#include "../../include/kestrel.h"

int kestrel_fail(int code, const char *fmt, ...);
// multiprocessors of the current device (cost models and grids size themselves by it); a
// B200's 148 where no device can be asked, as when a cost model is called on a host without one
static inline int kestrel_sms() {
    int n = kestrel_sm_count();
    return n > 0 ? n : 148;
}
int kestrel_check_launch(const char *what);

#define KESTREL_REQUIRE(cond, ...)                       \
    do {                                                 \
        if (!(cond)) return kestrel_fail(-2, __VA_ARGS__); \
    } while (0)

// Programmatic dependent launch.  Every kernel of the library is launched with the attribute
// that lets it start while its predecessor on the stream is still draining, calls
// pdl_launch_dependents() first thing (so that its own successor may be scheduled as soon as
// all of its blocks are resident) and pdl_wait() before it touches global memory (which
// returns once the predecessor has completed and its writes are visible).  Because every
// kernel waits, completion is transitive along the stream.  What runs before the wait - barrier
// set-up, TMEM allocation, descriptor prefetch, index arithmetic - overlaps the predecessor's
// tail.  kestrel_set_pdl(0) switches the attribute off; the instructions are then no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

extern int g_kestrel_pdl;

template <typename... KArgs, typename... Args>
static inline cudaError_t kestrel_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_kestrel_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
