// Error reporting shared by all entry points, and the library's identity.
#include "tcgen05.cuh"
#include <stdarg.h>
#include <stdio.h>

static thread_local char g_error[512] = "";

int kestrel_fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int kestrel_check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return kestrel_fail(-3, "%s: %s", what, cudaGetErrorString(e));
    return 0;
}

int g_kestrel_pdl = 1;

// 1: kernels are launched with programmatic dependent launch (the default); 0: plain stream order
KESTREL_API void kestrel_set_pdl(int on) { g_kestrel_pdl = on ? 1 : 0; }

KESTREL_API const char *kestrel_last_error(void) { return g_error; }

// Compute capability of the current device as major*10+minor, or a negative code.
KESTREL_API int kestrel_device_arch(void) {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return kestrel_fail(-3, "no CUDA device");
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    return major * 10 + minor;
}

// Streaming multiprocessors of the current device, asked once per device; cost models and grids
// size themselves by it.
KESTREL_API int kestrel_sm_count(void) {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return kestrel_fail(-3, "no CUDA device");
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
        return kestrel_fail(-3, "cannot read the device's multiprocessor count");
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

// Error words of all kernels with bounded waits in one call: bit 0 the tensor-core product,
// bit 1 the prompt-portion attention, bit 2 the decode attention.  Synchronises the device and
// clears the words.
KESTREL_API int kestrel_kernel_errors(void) {
    int bits = 0;
    if (kestrel_gemm_tc_error() != 0) bits |= 1;
    if (kestrel_attention_tc_error() != 0) bits |= 2;
    if (kestrel_attention_decode_error() != 0) bits |= 4;
    return bits;
}

// ------------------------------------------------------------------------------------------
// What the kernels' bounded waits do when nothing ever arrives: one block waits on an mbarrier
// that no one completes, with the same wait the tensor-core kernels use.  The wait gives up
// after its limit (about two seconds), the kernel records that and returns; the context stays
// usable.  Returns 1 if the wait gave up, 0 if it claimed success, negative on an API error;
// *elapsed_ms is the kernel's duration.
// ------------------------------------------------------------------------------------------
__global__ void wait_probe_kernel(int *result) {
    __shared__ __align__(8) unsigned long long barrier_word;
    const uint32_t bar = smem_u32(&barrier_word);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *result = mbar_wait(bar, 0) ? 0 : 1;
    }
}

KESTREL_API int kestrel_wait_probe(float *elapsed_ms) {
    int *flag = nullptr;
    cudaEvent_t a, b;
    if (cudaMalloc(&flag, sizeof(int)) != cudaSuccess) return kestrel_fail(-3, "wait_probe: no memory");
    cudaMemset(flag, 0xff, sizeof(int));
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    cudaEventRecord(a, 0);
    wait_probe_kernel<<<1, 32>>>(flag);
    cudaEventRecord(b, 0);
    cudaError_t e = cudaDeviceSynchronize();
    int result = -1;
    if (e == cudaSuccess) e = cudaMemcpy(&result, flag, sizeof(int), cudaMemcpyDeviceToHost);
    if (elapsed_ms) cudaEventElapsedTime(elapsed_ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    cudaFree(flag);
    if (e != cudaSuccess) return kestrel_fail(-3, "wait_probe: %s", cudaGetErrorString(e));
    return result;
}
