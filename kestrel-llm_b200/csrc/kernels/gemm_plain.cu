// Plain matrix product on the CUDA cores: out[t, n] = sum_k x[t, k] * w[n, k], float32
// accumulation by FMA in ascending k for every output, whatever T is (the reference's
// float32 product, st.c:8880-8892, is the same sum row by row).  It is the whole product of
// the true 32-bit path, the fallback of the bfloat16 path for sizes the tensor-core kernel
// refuses, and the twin that the tensor-core kernel is tested against.  Any T, N, K.
//
// Tile 64x64, 256 threads, 4x4 outputs per thread, K in steps of 16 through shared memory.
#include "common.cuh"

#define PG_BM 64
#define PG_BN 64
#define PG_BK 16

template <typename T>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const T *__restrict__ x, const T *__restrict__ w, float *__restrict__ out,
                  int Tn, int N, int K, long long ldx, long long ldw, long long ldo) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float xs[PG_BK][PG_BM + 4];
    __shared__ float ws[PG_BK][PG_BN + 4];
    int tid = threadIdx.x;
    int t0 = blockIdx.y * PG_BM, n0 = blockIdx.x * PG_BN;
    int ty = tid / 16, tx = tid % 16;          // 16 x 16 threads, each 4 rows x 4 cols
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += PG_BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int idx = tid + 256 * e;
            int r = idx / PG_BK, kk = idx % PG_BK;
            int gk = k0 + kk;
            float xv = 0.f, wv = 0.f;
            if (gk < K) {
                if (t0 + r < Tn) xv = to_f32<T>(x[(size_t)(t0 + r) * ldx + gk]);
                if (n0 + r < N) wv = to_f32<T>(w[(size_t)(n0 + r) * ldw + gk]);
            }
            xs[kk][r] = xv;
            ws[kk][r] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < PG_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int t = t0 + ty * 4 + i;
        if (t >= Tn) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + tx * 4 + j;
            if (n < N) out[(size_t)t * ldo + n] = acc[i][j];
        }
    }
}

KESTREL_API int kestrel_gemm_plain(const void *x, const void *w, float *out, int dtype, int T, int N,
                                   int K, long long ldx, long long ldw, long long ldo,
                                   cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && N > 0 && K > 0, "gemm_plain: bad sizes T=%d N=%d K=%d", T, N, K);
    dim3 grid((N + PG_BN - 1) / PG_BN, (T + PG_BM - 1) / PG_BM);
    KESTREL_REQUIRE(grid.y <= 65535, "gemm_plain: T=%d needs more than 65535 row tiles", T);
    if (dtype == KESTREL_F32)
        kestrel_launch(gemm_plain_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float *)x, (const float *)w, out, T, N, K, ldx, ldw, ldo);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(gemm_plain_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)w, out, T, N, K, ldx, ldw, ldo);
    else
        return kestrel_fail(-2, "gemm_plain: unknown dtype %d", dtype);
    return kestrel_check_launch("gemm_plain");
}
