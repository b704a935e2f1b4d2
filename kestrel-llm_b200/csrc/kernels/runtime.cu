// Error reporting shared by all entry points, and the library's identity.
#include "common.cuh"
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
