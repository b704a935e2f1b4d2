// The allocation-free matrix product declared in linear_noalloc.h: the tcgen05 split-K
// product followed by the fixed-order sum of its slices, with the slices kept in an array
// that is part of the library image instead of a buffer allocated per call.
#include "linear_noalloc.h"
#include "common.cuh"

// (the entry points of the other translation units that do the work are declared in kestrel.h)

#define NOALLOC_FLOATS (KESTREL_NOALLOC_SCRATCH_BYTES / sizeof(float))
#define NOALLOC_MAX_DEVICES 64

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; it is
// NOT a device pointer and must never be passed to a kernel as one.
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_FLOATS];

// device address of the array on each device, looked up at the first call there
static float *g_scratch_addr[NOALLOC_MAX_DEVICES];

static int scratch_for_current_device(float **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return kestrel_fail(-3, "linear_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return kestrel_fail(-2, "linear_noalloc: device index %d is beyond %d", dev, NOALLOC_MAX_DEVICES);
    if (!g_scratch_addr[dev]) {
        float *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_noalloc_scratch);     // with device `dev` current
        if (e != cudaSuccess || !p)
            return kestrel_fail(-3, "linear_noalloc: cudaGetSymbolAddress on device %d: %s", dev, cudaGetErrorString(e));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

KESTREL_API int kestrel_linear_bf16_noalloc(const void *x, const void *w, const float *bias, void *out, int out_dtype,
                                            int T, int N, int K, long long ldx, long long ldw, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && N > 0 && K > 0, "linear_noalloc: bad sizes T=%d N=%d K=%d", T, N, K);
    KESTREL_REQUIRE(out_dtype == KESTREL_F32 || out_dtype == KESTREL_BF16, "linear_noalloc: unknown output dtype %d", out_dtype);
    KESTREL_REQUIRE(kestrel_gemm_tc_supported(x, w, T, N, K, ldx, ldw),
                    "linear_noalloc: K=%d, ldx=%lld, ldw=%lld must be multiples of 8 and x, w 16-byte aligned", K, ldx, ldw);
    int splits = kestrel_gemm_tc_splits(T, N, K);
    unsigned long long need = (unsigned long long)splits * (unsigned long long)T * (unsigned long long)N;
    if (need > NOALLOC_FLOATS && splits > 1) {       // one slice is always possible, if slower
        splits = 1;
        need = (unsigned long long)T * (unsigned long long)N;
    }
    KESTREL_REQUIRE(need <= NOALLOC_FLOATS,
                    "linear_noalloc: %d slices of T=%d x N=%d float32 need %llu bytes of scratch; the built-in array holds %u",
                    splits, T, N, need * 4ull, (unsigned)KESTREL_NOALLOC_SCRATCH_BYTES);
    float *scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    long long slice = (long long)T * N;
    rc = kestrel_gemm_tc(x, w, scratch, T, N, K, ldx, ldw, N, splits, slice, stream);
    if (rc) return rc;
    return kestrel_reduce_partials(scratch, splits, slice, bias, out, out_dtype, T, N, stream);
}
