// Plain causal attention over the paged cache, one block per (token, query head).
//
// For the token at position p of its request the keys are positions lo..p of the same
// request, lo = 0 or p - window + 1 for a windowed layer; the mask is this loop bound, as in
// the reference (st.c:1974, st.c:10833-10849).  kv head = (h * nkv) / nq (st.c:10782);
// score = dot * scale (st.c:10846); softmax in float32 with a running maximum (the
// reference's tiled online form, st.c:9762-9859); out = sum_s w_s V_s.
//
// The four warps of a block take keys lo+w, lo+w+4, ... in groups of four; their running
// (max, sum, out) states are merged in warp order.  The order of every sum depends on
// (lo, p) alone: a token's result is bit-identical however the step was cut or batched.
// Works for any head size up to 256 and any numbers of heads.  It is the attention of the
// true 32-bit path and the twin that the fast kernels are tested against.
#include "common.cuh"
#include <math.h>

#define PA_WARPS 4
#define PA_MAX_PER_LANE 8     // head size up to 256
#define PA_KEYS 4

template <typename T>
__global__ void __launch_bounds__(PA_WARPS * 32)
attention_plain_kernel(const T *__restrict__ q, const T *__restrict__ k_cache, const T *__restrict__ v_cache,
                       const int *__restrict__ positions, const int *__restrict__ seq_of_token,
                       const int *__restrict__ block_table, int table_stride, int page_size,
                       T *__restrict__ out, int nq, int nkv, int hd, int window, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x, h = blockIdx.y;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int kvh = (h * nkv) / nq;
    int pos = positions[t];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int *table = block_table + (size_t)seq_of_token[t] * table_stride;
    int per_lane = (hd + 31) / 32;

    float qv[PA_MAX_PER_LANE], acc[PA_MAX_PER_LANE];
    const T *qrow = q + ((size_t)t * nq + h) * hd;
#pragma unroll
    for (int c = 0; c < PA_MAX_PER_LANE; ++c) {
        int i = lane + 32 * c;
        qv[c] = (c < per_lane && i < hd) ? to_f32<T>(qrow[i]) : 0.f;
        acc[c] = 0.f;
    }
    float m = -INFINITY, l = 0.f;

    for (int base = lo + warp * PA_KEYS; base <= pos; base += PA_WARPS * PA_KEYS) {
        float sc[PA_KEYS];
        const T *vrow[PA_KEYS];
#pragma unroll
        for (int u = 0; u < PA_KEYS; ++u) {
            int s = base + u;
            float dot = 0.f;
            vrow[u] = nullptr;
            if (s <= pos) {
                int page = table[s / page_size];
                size_t off = (((size_t)page * nkv + kvh) * page_size + (s % page_size)) * hd;
                const T *krow = k_cache + off;
                vrow[u] = v_cache + off;
#pragma unroll
                for (int c = 0; c < PA_MAX_PER_LANE; ++c) {
                    int i = lane + 32 * c;
                    if (c < per_lane && i < hd) dot = fmaf(qv[c], to_f32<T>(krow[i]), dot);
                }
            }
            dot = warp_sum(dot);
            sc[u] = (s <= pos) ? dot * scale : -INFINITY;
        }
        float mn = m;
#pragma unroll
        for (int u = 0; u < PA_KEYS; ++u) mn = fmaxf(mn, sc[u]);
        float corr = expf(m - mn);          // m = -inf on the first group: exp(-inf) = 0
        l *= corr;
#pragma unroll
        for (int c = 0; c < PA_MAX_PER_LANE; ++c) acc[c] *= corr;
#pragma unroll
        for (int u = 0; u < PA_KEYS; ++u) {
            if (vrow[u]) {
                float p = expf(sc[u] - mn);
                l += p;
#pragma unroll
                for (int c = 0; c < PA_MAX_PER_LANE; ++c) {
                    int i = lane + 32 * c;
                    if (c < per_lane && i < hd) acc[c] = fmaf(p, to_f32<T>(vrow[u][i]), acc[c]);
                }
            }
        }
        m = mn;
    }

    // merge the warps' states in warp order
    __shared__ float sm_m[PA_WARPS], sm_l[PA_WARPS];
    __shared__ float sm_acc[PA_WARPS][PA_MAX_PER_LANE * 32];
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int c = 0; c < PA_MAX_PER_LANE; ++c) sm_acc[warp][lane + 32 * c] = acc[c];
    __syncthreads();
    if (warp == 0) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < PA_WARPS; ++w) M = fmaxf(M, sm_m[w]);
        float L = 0.f;
        float o[PA_MAX_PER_LANE];
#pragma unroll
        for (int c = 0; c < PA_MAX_PER_LANE; ++c) o[c] = 0.f;
#pragma unroll
        for (int w = 0; w < PA_WARPS; ++w) {
            if (sm_m[w] == -INFINITY) continue;     // a warp that saw no key
            float f = expf(sm_m[w] - M);
            L += sm_l[w] * f;
#pragma unroll
            for (int c = 0; c < PA_MAX_PER_LANE; ++c) o[c] += sm_acc[w][lane + 32 * c] * f;
        }
        float inv = 1.0f / L;
        T *orow = out + ((size_t)t * nq + h) * hd;
#pragma unroll
        for (int c = 0; c < PA_MAX_PER_LANE; ++c) {
            int i = lane + 32 * c;
            if (c < per_lane && i < hd) orow[i] = from_f32<T>(o[c] * inv);
        }
    }
}

KESTREL_API int kestrel_attention_plain(const void *q, const void *k_cache, const void *v_cache,
                                        const int *positions, const int *seq_of_token,
                                        const int *block_table, int table_stride, int page_size,
                                        void *out, int dtype, int T, int nq, int nkv, int hd, int window,
                                        float scale, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && nq > 0 && nkv > 0 && hd > 0, "attention_plain: bad sizes");
    KESTREL_REQUIRE(hd <= 32 * PA_MAX_PER_LANE, "attention_plain: head size %d exceeds %d", hd, 32 * PA_MAX_PER_LANE);
    KESTREL_REQUIRE(nq <= 65535, "attention_plain: %d query heads exceed the grid", nq);
    dim3 grid(T, nq);
    if (dtype == KESTREL_F32)
        kestrel_launch(attention_plain_kernel<float>, dim3(grid), dim3(PA_WARPS * 32), 0, stream, (const float *)q, (const float *)k_cache, (const float *)v_cache, positions, seq_of_token,
            block_table, table_stride, page_size, (float *)out, nq, nkv, hd, window, scale);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(attention_plain_kernel<__nv_bfloat16>, dim3(grid), dim3(PA_WARPS * 32), 0, stream, (const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_cache, (const __nv_bfloat16 *)v_cache, positions,
            seq_of_token, block_table, table_stride, page_size, (__nv_bfloat16 *)out, nq, nkv, hd, window, scale);
    else
        return kestrel_fail(-2, "attention_plain: unknown dtype %d", dtype);
    return kestrel_check_launch("attention_plain");
}
