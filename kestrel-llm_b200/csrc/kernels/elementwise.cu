// Row-wise kernels of the decoder: embedding gather, residual-add + RMSNorm, gated
// activation, and the step between the QKV projection and attention (bias, per-head RMSNorm,
// rotary position encoding, write of K and V into cache pages).
//
// A projection's output reaches these kernels as `S` float32 partial results of shape
// [S, T, N] (split-K slices of a matrix product; S = 1 for an unsplit product).  The consumer
// sums the slices in ascending s, so the result does not depend on scheduling, and the sum
// never makes a round trip through memory.  Formulas follow the reference's float32 path:
// RMSNorm st.c:8811-8827, per-head norm st.c:9541-9561, rotation st.c:8950-8991, SiLU
// st.c:3605-3607 (st.c = src/model/vllm_safetensors.c).
#include "common.cuh"

// ------------------------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :] widened to float32 (st.c:16392-16393)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T *__restrict__ table, const int *__restrict__ ids,
                             float *__restrict__ out, int d) {
    pdl_launch_dependents();
    pdl_wait();
    int t = blockIdx.x;
    const T *row = table + (size_t)ids[t] * d;
    float *o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_f32<T>(row[i]);
}

KESTREL_API int kestrel_embed(const void *table, int dtype, const int *ids, float *out, int T,
                              int d, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && d > 0, "embed: bad sizes T=%d d=%d", T, d);
    if (dtype == KESTREL_F32)
        kestrel_launch(embed_kernel<float>, dim3(T), dim3(256), 0, stream, (const float *)table, ids, out, d);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16 *)table, ids, out, d);
    else
        return kestrel_fail(-2, "embed: unknown dtype %d", dtype);
    return kestrel_check_launch("embed");
}

// ------------------------------------------------------------------------------------------
// residual add + RMSNorm
//   src row t = rows ? rows[r] : r
//   x = residual[t] + (sum_s partial[s, t] + bias)      (partial may be null: x = residual[t])
//   if write_back: residual[t] = x
//   out[r] = (x * rsqrt(mean(x^2) + eps)) * w
// One block of 256 threads per row; the sum of squares is reduced in a fixed tree, so a
// row's result does not depend on what else is in the batch.
// ------------------------------------------------------------------------------------------
#define NORM_THREADS 256

template <typename TOut>
__global__ void add_rmsnorm_kernel(float *__restrict__ residual, const float *__restrict__ partial,
                                   int S, size_t slice_stride, const float *__restrict__ bias,
                                   const int *__restrict__ rows, const float *__restrict__ w,
                                   float eps, TOut *__restrict__ out, int d, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float xs[];
    __shared__ float red[NORM_THREADS / 32];
    int r = blockIdx.x;
    int t = rows ? rows[r] : r;
    float *res = residual + (size_t)t * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += NORM_THREADS) {
        float x = res[i];
        if (partial) {
            float delta = 0.f;
            for (int s = 0; s < S; ++s) delta += partial[(size_t)s * slice_stride + (size_t)t * d + i];
            if (bias) delta += bias[i];
            x += delta;
            if (write_back) res[i] = x;
        }
        xs[i] = x;
        ss += x * x;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_THREADS / 32; ++k) tot += red[k];
    float rinv = 1.0f / sqrtf(tot / (float)d + eps);
    TOut *o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += NORM_THREADS) o[i] = from_f32<TOut>((xs[i] * rinv) * w[i]);
}

// The same for widths that are a multiple of 4: 1024 threads, float4 accesses, and the loads
// of the slices issued four at a time (they are independent; the adds stay in ascending s).
// With few rows in the batch (decode) the kernel is latency-bound, so the work of a row is
// spread over as many threads as there are vectors.
#define NORMV_THREADS 1024

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ void store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t *>(&lo);
    u.y = *reinterpret_cast<uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(p) = u;
}

// THREADS is 1024 or 256.  With 256 threads a thread plays four of the 1024 "virtual lanes"
// (t, t + 256, ...): vector i always belongs to virtual lane i mod 1024 and the sums of
// squares are combined in the same tree, so both variants give the same bits and the choice
// can follow the number of rows (few rows: spread a row wide; many rows: more blocks per SM).
template <typename TOut, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_vec_kernel(float *__restrict__ residual, const float *__restrict__ partial, int S, size_t slice_stride,
                       const float *__restrict__ bias, const int *__restrict__ rows, const float *__restrict__ w,
                       float eps, TOut *__restrict__ out, int d, int write_back) {
    pdl_launch_dependents();
    // the norm's weight is a model weight: this thread's first vector of it is fetched while the
    // kernel before this one still runs, not after the row's sum is known
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    const float4 g0 = (int)threadIdx.x < (d >> 2) ? w4[threadIdx.x] : make_float4(0.f, 0.f, 0.f, 0.f);
    pdl_wait();
    constexpr int VL = NORMV_THREADS / THREADS;
    extern __shared__ float xs[];
    __shared__ float red[NORMV_THREADS / 32];
    int r = blockIdx.x;
    int t = rows ? rows[r] : r;
    int d4 = d >> 2;
    float4 *res = reinterpret_cast<float4 *>(residual + (size_t)t * d);
    const float4 *bias4 = reinterpret_cast<const float4 *>(bias);
    float ss[VL];
#pragma unroll
    for (int k = 0; k < VL; ++k) ss[k] = 0.f;
    for (int base = 0; base < d4; base += NORMV_THREADS) {
#pragma unroll
        for (int k = 0; k < VL; ++k) {
            int i = base + threadIdx.x + k * THREADS;
            if (i >= d4) continue;
            float4 x = res[i];
            if (partial) {
                const float4 *p4 = reinterpret_cast<const float4 *>(partial + (size_t)t * d) + i;
                size_t st4 = slice_stride >> 2;
                float4 delta = make_float4(0.f, 0.f, 0.f, 0.f);
                int s = 0;
                for (; s + 4 <= S; s += 4) {
                    float4 a = p4[(size_t)s * st4], b = p4[(size_t)(s + 1) * st4], c = p4[(size_t)(s + 2) * st4], e = p4[(size_t)(s + 3) * st4];
                    delta = add4(add4(add4(add4(delta, a), b), c), e);
                }
                for (; s < S; ++s) delta = add4(delta, p4[(size_t)s * st4]);
                if (bias) delta = add4(delta, bias4[i]);
                x = add4(x, delta);
                if (write_back) res[i] = x;
            }
            reinterpret_cast<float4 *>(xs)[i] = x;
            ss[k] += x.x * x.x;
            ss[k] += x.y * x.y;
            ss[k] += x.z * x.z;
            ss[k] += x.w * x.w;
        }
    }
#pragma unroll
    for (int k = 0; k < VL; ++k) {
        float v = warp_sum(ss[k]);
        if ((threadIdx.x & 31) == 0) red[(threadIdx.x >> 5) + k * (THREADS / 32)] = v;
    }
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < NORMV_THREADS / 32; ++k) tot += red[k];
    float rinv = 1.0f / sqrtf(tot / (float)d + eps);
    TOut *o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d4; i += THREADS) {
        float4 x = reinterpret_cast<float4 *>(xs)[i], g = i == (int)threadIdx.x ? g0 : w4[i];
        store4(o + 4 * i, make_float4((x.x * rinv) * g.x, (x.y * rinv) * g.y, (x.z * rinv) * g.z, (x.w * rinv) * g.w));
    }
}

// Many rows: one WARP per row, the row's vectors in registers (lane l holds vectors l, l + 32,
// ...), no shared memory and no block barrier; all of a row's loads are in flight at once and
// several rows a block keep the memory system busy, where one block per row waits out its own
// chain of load, barrier, store (2,048 rows of 4,096: 17.4 us before).  The sums are the SAME
// tree as above - vector i is virtual lane i mod 1024, its squares are added in the order x, y,
// z, w, virtual lanes 32 g .. 32 g + 31 are combined by the same shuffle tree and the 32 group
// sums in ascending order - so a row's bits do not depend on which variant ran.
// NV: vectors per lane, 32 NV >= d / 4.
// Rows from which the norm takes a warp a row, where it only reads the stream (the products
// added themselves already).  With slices to add and the stream to write back the block-a-row
// kernel is twice as fast (measured, 4,096 rows of two slices: 52 against 106 us; 1,536 rows of
// three: 29 against 58), so the warp kernel is not taken then unless a test asks for it.
static int g_norm_warp_rows = 1024, g_norm_warp_slices = 0;
KESTREL_API void kestrel_set_norm_warp_rows(int rows, int with_slices) {
    g_norm_warp_rows = rows > 0 ? rows : 1024;
    g_norm_warp_slices = with_slices ? 1 : 0;
}

template <typename TOut, int NV>
__global__ void __launch_bounds__(128)
add_rmsnorm_warp_kernel(float *__restrict__ residual, const float *__restrict__ partial, int S, size_t slice_stride,
                        const float *__restrict__ bias, const int *__restrict__ rows, const float *__restrict__ w,
                        float eps, TOut *__restrict__ out, int R, int d, int write_back) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= R) return;
    const int t = rows ? rows[r] : r;
    const int d4 = d >> 2;
    float4 *res = reinterpret_cast<float4 *>(residual + (size_t)t * d);
    float4 x[NV];
    if (partial) {
        // delta = ((0 + P[0]) + P[1]) + ... + bias, then residual + delta: the other norm kernels'
        // order.  A pass over the row per slice, so that all of a pass's loads are in flight at
        // once (one element's slices one after the other is a chain of S load latencies, thirty-two
        // times over: measured 80 us instead of 20 for 1,536 rows of three slices).
        const float4 *p4 = reinterpret_cast<const float4 *>(partial + (size_t)t * d);
        const float4 *bias4 = reinterpret_cast<const float4 *>(bias);
        const size_t st4 = slice_stride >> 2;
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = 32 * j + lane;
            x[j] = i < d4 ? add4(zero, p4[i]) : zero;
        }
        for (int s = 1; s < S; ++s) {
            const float4 *ps = p4 + (size_t)s * st4;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int i = 32 * j + lane;
                if (i < d4) x[j] = add4(x[j], ps[i]);
            }
        }
        if (bias) {
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int i = 32 * j + lane;
                if (i < d4) x[j] = add4(x[j], bias4[i]);
            }
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = 32 * j + lane;
            if (i >= d4) continue;
            x[j] = add4(res[i], x[j]);
            if (write_back) res[i] = x[j];
        }
    } else {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int i = 32 * j + lane;
            x[j] = i < d4 ? res[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float tot = 0.f;
#pragma unroll
    for (int g = 0; g < 32; ++g) {
        float ss = 0.f;
        if (g < NV) {
            ss += x[g].x * x[g].x;
            ss += x[g].y * x[g].y;
            ss += x[g].z * x[g].z;
            ss += x[g].w * x[g].w;
        }
        if (g + 32 < NV) {              // widths beyond 4096: the second vector of this virtual lane
            ss += x[(g + 32) % NV].x * x[(g + 32) % NV].x;
            ss += x[(g + 32) % NV].y * x[(g + 32) % NV].y;
            ss += x[(g + 32) % NV].z * x[(g + 32) % NV].z;
            ss += x[(g + 32) % NV].w * x[(g + 32) % NV].w;
        }
        tot += warp_sum(ss);
    }
    const float rinv = 1.0f / sqrtf(tot / (float)d + eps);
    TOut *o = out + (size_t)r * d;
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = 32 * j + lane;
        if (i >= d4) continue;
        const float4 g = w4[i];
        store4(o + 4 * i, make_float4((x[j].x * rinv) * g.x, (x[j].y * rinv) * g.y, (x[j].z * rinv) * g.z, (x[j].w * rinv) * g.w));
    }
}

template <typename TOut>
static void launch_add_rmsnorm(float *residual, const float *partial, int S, long long slice_stride, const float *bias,
                               const int *rows, const float *w, float eps, TOut *out, int R, int d, int write_back,
                               size_t smem, cudaStream_t stream) {
    // the vector kernel for widths of at least 2048 that are multiples of 4 (and slices and
    // pointers that keep float4 alignment); which kernel runs depends on the width alone, so a
    // row's result does not depend on the batch
    bool vec = d % 4 == 0 && d >= 2048 && slice_stride % 4 == 0 &&
               ((((uintptr_t)residual | (uintptr_t)partial | (uintptr_t)bias | (uintptr_t)w) & 15) == 0) &&
               (((uintptr_t)out & 7) == 0);
    if (vec && R >= g_norm_warp_rows && d <= 48 * 128 && (!partial || g_norm_warp_slices)) {
        // very many rows: a warp a row (widths up to 6144 fit a lane's registers; measured faster from about a thousand rows on)
        const dim3 grid((R + 3) / 4), block(128);
        if (d <= 16 * 128)
            kestrel_launch(add_rmsnorm_warp_kernel<TOut, 16>, grid, block, 0, stream, residual, partial, S, (size_t)slice_stride, bias, rows, w, eps, out, R, d, write_back);
        else if (d <= 32 * 128)
            kestrel_launch(add_rmsnorm_warp_kernel<TOut, 32>, grid, block, 0, stream, residual, partial, S, (size_t)slice_stride, bias, rows, w, eps, out, R, d, write_back);
        else if (d <= 40 * 128)
            kestrel_launch(add_rmsnorm_warp_kernel<TOut, 40>, grid, block, 0, stream, residual, partial, S, (size_t)slice_stride, bias, rows, w, eps, out, R, d, write_back);
        else
            kestrel_launch(add_rmsnorm_warp_kernel<TOut, 48>, grid, block, 0, stream, residual, partial, S, (size_t)slice_stride, bias, rows, w, eps, out, R, d, write_back);
    } else if (vec && R >= 296) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_vec_kernel<TOut, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kestrel_launch(add_rmsnorm_vec_kernel<TOut, 256>, dim3(R), dim3(256), smem, stream, residual, partial, S, (size_t)slice_stride, bias, rows, w, eps, out, d, write_back);
    } else if (vec) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_vec_kernel<TOut, NORMV_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kestrel_launch(add_rmsnorm_vec_kernel<TOut, NORMV_THREADS>, dim3(R), dim3(NORMV_THREADS), smem, stream, residual, partial, S, (size_t)slice_stride, bias, rows, w, eps, out, d, write_back);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kestrel_launch(add_rmsnorm_kernel<TOut>, dim3(R), dim3(NORM_THREADS), smem, stream, residual, partial, S, (size_t)slice_stride, bias, rows, w, eps, out, d, write_back);
    }
}

KESTREL_API int kestrel_add_rmsnorm(float *residual, const float *partial, int S,
                                    long long slice_stride, const float *bias, const int *rows,
                                    const float *w, float eps, void *out, int out_dtype, int R,
                                    int d, int write_back, cudaStream_t stream) {
    if (R == 0) return 0;
    KESTREL_REQUIRE(R > 0 && d > 0, "add_rmsnorm: bad sizes R=%d d=%d", R, d);
    KESTREL_REQUIRE(!(rows && write_back), "add_rmsnorm: write_back with gathered rows");
    KESTREL_REQUIRE(!partial || S >= 1, "add_rmsnorm: a product of %d slices", S);
    size_t smem = (size_t)d * sizeof(float);
    KESTREL_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: width %d exceeds the 51200 the kernel holds in shared memory", d);
    if (out_dtype == KESTREL_F32)
        launch_add_rmsnorm<float>(residual, partial, S, slice_stride, bias, rows, w, eps, (float *)out, R, d, write_back, smem, stream);
    else if (out_dtype == KESTREL_BF16)
        launch_add_rmsnorm<__nv_bfloat16>(residual, partial, S, slice_stride, bias, rows, w, eps, (__nv_bfloat16 *)out, R, d, write_back, smem, stream);
    else
        return kestrel_fail(-2, "add_rmsnorm: unknown dtype %d", out_dtype);
    return kestrel_check_launch("add_rmsnorm");
}

// ------------------------------------------------------------------------------------------
// gated activation: out[t, i] = silu(g) * u,  g = sum_s P[s, t, i],  u = sum_s P[s, t, ff + i]
// ------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void swiglu_kernel(const float *__restrict__ partial, int S, size_t slice_stride,
                              TOut *__restrict__ out, int T, int ff) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)T * ff) return;
    int t = (int)(idx / ff), i = (int)(idx % ff);
    const float *row = partial + (size_t)t * 2 * ff;
    float g = 0.f, u = 0.f;
    for (int s = 0; s < S; ++s) {
        g += row[(size_t)s * slice_stride + i];
        u += row[(size_t)s * slice_stride + ff + i];
    }
    float a = g / (1.0f + expf(-g));
    out[idx] = from_f32<TOut>(a * u);
}

KESTREL_API int kestrel_swiglu(const float *partial, int S, long long slice_stride, void *out,
                               int out_dtype, int T, int ff, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && ff > 0, "swiglu: bad sizes T=%d ff=%d", T, ff);
    size_t n = (size_t)T * ff;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == KESTREL_F32)
        kestrel_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, partial, S, (size_t)slice_stride, (float *)out, T, ff);
    else if (out_dtype == KESTREL_BF16)
        kestrel_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, partial, S, (size_t)slice_stride, (__nv_bfloat16 *)out, T, ff);
    else
        return kestrel_fail(-2, "swiglu: unknown dtype %d", out_dtype);
    return kestrel_check_launch("swiglu");
}

// ------------------------------------------------------------------------------------------
// between the QKV projection and attention
//   input  : partial [S, T, nq*hd + 2*nkv*hd] float32 (q heads, then k heads, then v heads),
//            optional bias of the same width
//   q head : + bias, per-head RMSNorm (if q_norm_w), rotation, -> q_out [T, nq*hd]
//   k head : + bias, per-head RMSNorm (if k_norm_w), rotation, -> K page slot of the token
//   v head : + bias                                           -> V page slot of the token
// Rotation turns pairs of dimensions inside the first `rot` dimensions of a head (rot = head size
// for Qwen3) by angle = (float)pos * inv_freq[j], cosf/sinf in float32, both multiplied by
// rot_scale (1 for Qwen3).  rot_mode 0 pairs dimension j with j + rot/2 (rotate-half, the
// reference's pairing, st.c:8963-8989); rot_mode 1 pairs 2j with 2j + 1 (interleaved).
// The page of a token is block_table[seq, pos / page_size]; cache planes are laid out
// [page][kv_head][slot][hd].  One warp per (token, head).
// ------------------------------------------------------------------------------------------
#define PREP_MAX_PER_LANE 8   // head size up to 8 * 32 = 256

// rotation when half the rotary size is HP * 32: the pair (j, j + half) sits in registers c and c + HP
template <int HP>
__device__ __forceinline__ void rotate_in_registers(float *x, int pos, const float *__restrict__ inv_freq, int lane, float rot_scale) {
#pragma unroll
    for (int c = 0; c < HP; ++c) {
        float ang = (float)pos * inv_freq[lane + 32 * c];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        sn *= rot_scale;
        cs *= rot_scale;
        float lo = x[c], hi = x[c + HP];
        x[c] = lo * cs - hi * sn;
        x[c + HP] = hi * cs + lo * sn;
    }
}

template <typename T>
__global__ void attn_prepare_kernel(const float *__restrict__ partial, int S, size_t slice_stride,
                                    const float *__restrict__ bias, const float *__restrict__ q_norm_w,
                                    const float *__restrict__ k_norm_w, float norm_eps,
                                    const float *__restrict__ inv_freq, int rot, int rot_mode, float rot_scale,
                                    const int *__restrict__ positions, const int *__restrict__ seq_of_token,
                                    const int *__restrict__ block_table, int table_stride, int page_size,
                                    T *__restrict__ k_cache, T *__restrict__ v_cache, T *__restrict__ q_out,
                                    int Tn, int nq, int nkv, int hd, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    int warp = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    int lane = threadIdx.x & 31;
    int heads = nq + 2 * nkv;
    if (warp >= Tn * heads) return;
    int t = warp / heads, h = warp % heads;
    bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    if (!is_q && !write_kv) return;
    int width = heads * hd;
    const float *row = partial + (size_t)t * width + (size_t)h * hd;
    const float *b = bias ? bias + (size_t)h * hd : nullptr;

    float x[PREP_MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < PREP_MAX_PER_LANE; ++c) x[c] = 0.f;
    // the loads of a slice's elements are issued together, four slices at a time; the adds
    // stay in ascending s
    int s0 = 0;
    for (; s0 + 4 <= S; s0 += 4) {
        float v[4][PREP_MAX_PER_LANE];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
                int i = lane + 32 * c;
                v[u][c] = i < hd ? row[(size_t)(s0 + u) * slice_stride + i] : 0.f;
            }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int c = 0; c < PREP_MAX_PER_LANE; ++c) x[c] += v[u][c];
    }
    for (; s0 < S; ++s0) {
#pragma unroll
        for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
            int i = lane + 32 * c;
            if (i < hd) x[c] += row[(size_t)s0 * slice_stride + i];
        }
    }
#pragma unroll
    for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
        int i = lane + 32 * c;
        if (b && i < hd) x[c] += b[i];
        ss += x[c] * x[c];
    }
    const float *nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    if (nw) {
        ss = warp_sum(ss);
        float rinv = 1.0f / sqrtf(ss / (float)hd + norm_eps);
#pragma unroll
        for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
            int i = lane + 32 * c;
            if (i < hd) x[c] = (x[c] * rinv) * nw[i];
        }
    }
    int pos = positions[t];
    if ((is_q || is_k) && rot > 0) {
        int half = rot >> 1;
        if (rot_mode == 0 && (half & 31) == 0 && half <= 128) {
            // element lane + 32 c pairs with lane + 32 (c + half / 32): both are in this lane
            // (half = 32, 64, 96 or 128: the entry point refuses head sizes beyond 256)
            switch (half >> 5) {
                case 1: rotate_in_registers<1>(x, pos, inv_freq, lane, rot_scale); break;
                case 2: rotate_in_registers<2>(x, pos, inv_freq, lane, rot_scale); break;
                case 3: rotate_in_registers<3>(x, pos, inv_freq, lane, rot_scale); break;
                case 4: rotate_in_registers<4>(x, pos, inv_freq, lane, rot_scale); break;
            }
        } else {
            // the partner lives in another lane: exchange through a per-warp row of shared memory
            __shared__ float stage[4][PREP_MAX_PER_LANE * 32];
            float *st = stage[threadIdx.x >> 5];
#pragma unroll
            for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
                int i = lane + 32 * c;
                if (i < hd) st[i] = x[c];
            }
            __syncwarp();
#pragma unroll
            for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
                int i = lane + 32 * c;
                if (i < rot) {
                    // pair index j; its first member `lo`, its second `hi`
                    int j = rot_mode == 0 ? (i < half ? i : i - half) : (i >> 1);
                    bool first = rot_mode == 0 ? i < half : !(i & 1);
                    float ang = (float)pos * inv_freq[j];
                    float sn, cs;
                    sincosf(ang, &sn, &cs);
                    sn *= rot_scale;
                    cs *= rot_scale;
                    float lo = rot_mode == 0 ? st[j] : st[2 * j], hi = rot_mode == 0 ? st[j + half] : st[2 * j + 1];
                    x[c] = first ? lo * cs - hi * sn : hi * cs + lo * sn;
                }
            }
        }
    }
    if (is_q) {
        T *o = q_out + (size_t)t * nq * hd + (size_t)h * hd;
#pragma unroll
        for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
            int i = lane + 32 * c;
            if (i < hd) o[i] = from_f32<T>(x[c]);
        }
    } else {
        int kvh = is_k ? h - nq : h - nq - nkv;
        int seq = seq_of_token[t];
        int page = block_table[(size_t)seq * table_stride + pos / page_size];
        int slot = pos % page_size;
        T *plane = is_k ? k_cache : v_cache;
        T *o = plane + (((size_t)page * nkv + kvh) * page_size + slot) * hd;
#pragma unroll
        for (int c = 0; c < PREP_MAX_PER_LANE; ++c) {
            int i = lane + 32 * c;
            if (i < hd) o[i] = from_f32<T>(x[c]);
        }
    }
}

// The same for head size 128 with all 128 dims rotated by rotate-half pairing (the common case).
// A warp takes FOUR heads of one token: eight lanes a head, sixteen values a lane - dimensions
// 8 l' .. 8 l' + 7 and 64 + 8 l' .. 64 + 8 l' + 7 for lane l' of the eight, so that both members
// of every rotation pair sit in the same lane and the sum of squares needs three shuffle steps.
// With one head a warp and four values a lane the kernel spent about an instruction per value on
// addresses, shuffles and bookkeeping and ran at 2.5 TB/s, bound by instruction issue; this form
// needs about a third of the instructions.  A block of 256 threads takes 32 heads of a token
// (the token's cosines and sines are computed once per block, by 64 threads, into shared memory).
template <typename T>
__global__ void __launch_bounds__(256)
attn_prepare_hd128_kernel(const float *__restrict__ partial, int S, size_t slice_stride,
                          const float *__restrict__ bias, const float *__restrict__ q_norm_w,
                          const float *__restrict__ k_norm_w, float norm_eps, const float *__restrict__ inv_freq, float rot_scale,
                          const int *__restrict__ positions, const int *__restrict__ seq_of_token,
                          const int *__restrict__ block_table, int table_stride, int page_size,
                          T *__restrict__ k_cache, T *__restrict__ v_cache, T *__restrict__ q_out,
                          int nq, int nkv, int write_kv) {
    pdl_launch_dependents();
    constexpr int hd = 128;
    __shared__ __align__(16) float cs_s[64], sn_s[64];
    const int t = blockIdx.x;
    const int sub = threadIdx.x & 7;                       // lane of the eight that share a head
    const int heads = nq + 2 * nkv;
    const int h = blockIdx.y * 32 + (threadIdx.x >> 3);
    const bool live = h < heads;
    // What does not come from the kernel before this one - the step's description (positions, block
    // tables: copied before the step's first kernel), the rotation's frequencies, norm weights and
    // bias - is read, and the cosines and sines are made, while that kernel still runs.
    const int pos = positions[t];
    const bool is_q = h < nq, is_k = !is_q && h < nq + nkv;
    int page = 0;
    if (live && !is_q && write_kv)          // where the key or value goes: two dependent loads
        page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_size];
    if (threadIdx.x < 64) {
        float ang = (float)pos * inv_freq[threadIdx.x];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        cs_s[threadIdx.x] = cs * rot_scale;
        sn_s[threadIdx.x] = sn * rot_scale;
    }
    const float *nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    float4 g[4], bv[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) g[v] = bv[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && nw) {
        const float4 *g4 = reinterpret_cast<const float4 *>(nw) + 2 * sub;
        g[0] = g4[0]; g[1] = g4[1]; g[2] = g4[16]; g[3] = g4[17];
    }
    if (live && bias) {
        const float4 *b4 = reinterpret_cast<const float4 *>(bias + (size_t)h * hd) + 2 * sub;
        bv[0] = b4[0]; bv[1] = b4[1]; bv[2] = b4[16]; bv[3] = b4[17];
    }
    pdl_wait();
    // the head's values: their loads are in flight while the block meets at the barrier
    float4 x[4];             // x[0], x[1]: dimensions 8 sub .. 8 sub + 7; x[2], x[3]: the same 64 further
#pragma unroll
    for (int v = 0; v < 4; ++v) x[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        const float4 *row = reinterpret_cast<const float4 *>(partial + (size_t)t * heads * hd + (size_t)h * hd) + 2 * sub;
        const size_t st4 = slice_stride >> 2;
        for (int s = 0; s < S; ++s) {
            const float4 *r = row + (size_t)s * st4;
            float4 a = r[0], b = r[1], c = r[16], e = r[17];
            x[0] = add4(x[0], a); x[1] = add4(x[1], b); x[2] = add4(x[2], c); x[3] = add4(x[3], e);
        }
    }
    __syncthreads();
    // from here on the eight lanes of a head stay together: shuffles name them by their own mask
    if (!live || (!is_q && !write_kv)) return;
    const unsigned mask = 0xffu << (threadIdx.x & 24);
    if (bias) {
#pragma unroll
        for (int v = 0; v < 4; ++v) x[v] = add4(x[v], bv[v]);
    }
    if (nw) {
        float ss = 0.f;
#pragma unroll
        for (int v = 0; v < 4; ++v) ss += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(mask, ss, o);
        const float rinv = 1.0f / sqrtf(ss / (float)hd + norm_eps);
#pragma unroll
        for (int v = 0; v < 4; ++v)
            x[v] = make_float4((x[v].x * rinv) * g[v].x, (x[v].y * rinv) * g[v].y, (x[v].z * rinv) * g[v].z, (x[v].w * rinv) * g[v].w);
    }
    if (is_q || is_k) {
        // pair j = 8 sub + i: low member x[i / 4], high member x[2 + i / 4]
        const float4 *c4 = reinterpret_cast<const float4 *>(cs_s) + 2 * sub, *s4 = reinterpret_cast<const float4 *>(sn_s) + 2 * sub;
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            const float4 cs = c4[v], sn = s4[v], lo = x[v], hi = x[2 + v];
            x[v] = make_float4(lo.x * cs.x - hi.x * sn.x, lo.y * cs.y - hi.y * sn.y, lo.z * cs.z - hi.z * sn.z, lo.w * cs.w - hi.w * sn.w);
            x[2 + v] = make_float4(hi.x * cs.x + lo.x * sn.x, hi.y * cs.y + lo.y * sn.y, hi.z * cs.z + lo.z * sn.z, hi.w * cs.w + lo.w * sn.w);
        }
    }
    T *o;
    if (is_q) {
        o = q_out + ((size_t)t * nq + h) * hd;
    } else {
        const int kvh = is_k ? h - nq : h - nq - nkv;
        o = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * hd;
    }
    store4(o + 8 * sub, x[0]);
    store4(o + 8 * sub + 4, x[1]);
    store4(o + 64 + 8 * sub, x[2]);
    store4(o + 64 + 8 * sub + 4, x[3]);
}

KESTREL_API int kestrel_attn_prepare(const float *partial, int S, long long slice_stride,
                                     const float *bias, const float *q_norm_w, const float *k_norm_w,
                                     float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale,
                                     const int *positions, const int *seq_of_token,
                                     const int *block_table, int table_stride, int page_size,
                                     void *k_cache, void *v_cache, void *q_out, int dtype, int T,
                                     int nq, int nkv, int hd, int write_kv, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(T > 0 && nq > 0 && nkv > 0 && hd > 0, "attn_prepare: bad sizes");
    KESTREL_REQUIRE(hd <= 32 * PREP_MAX_PER_LANE, "attn_prepare: head size %d exceeds %d", hd, 32 * PREP_MAX_PER_LANE);
    KESTREL_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0, "attn_prepare: rotary size %d does not fit head size %d", rot, hd);
    KESTREL_REQUIRE(rot_mode == 0 || rot_mode == 1, "attn_prepare: rotation mode %d is neither 0 (rotate-half) nor 1 (interleaved)", rot_mode);
    KESTREL_REQUIRE(page_size > 0, "attn_prepare: page size %d", page_size);
    long long warps = (long long)T * (nq + 2 * nkv);
    unsigned blocks = (unsigned)((warps + 3) / 4);
    bool fast = hd == 128 && rot == 128 && rot_mode == 0 && slice_stride % 4 == 0 && (nq + 2 * nkv + 31) / 32 <= 65535 &&
                ((((uintptr_t)partial | (uintptr_t)bias | (uintptr_t)q_norm_w | (uintptr_t)k_norm_w | (uintptr_t)q_out |
                   (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0);
    if (fast) {
        dim3 grid(T, (nq + 2 * nkv + 31) / 32);
        if (dtype == KESTREL_F32)
            kestrel_launch(attn_prepare_hd128_kernel<float>, grid, dim3(256), 0, stream, partial, S, (size_t)slice_stride, bias, q_norm_w,
                           k_norm_w, norm_eps, inv_freq, rot_scale, positions, seq_of_token, block_table, table_stride, page_size,
                           (float *)k_cache, (float *)v_cache, (float *)q_out, nq, nkv, write_kv);
        else if (dtype == KESTREL_BF16)
            kestrel_launch(attn_prepare_hd128_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, partial, S, (size_t)slice_stride, bias,
                           q_norm_w, k_norm_w, norm_eps, inv_freq, rot_scale, positions, seq_of_token, block_table, table_stride, page_size,
                           (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache, (__nv_bfloat16 *)q_out, nq, nkv, write_kv);
        else
            return kestrel_fail(-2, "attn_prepare: unknown dtype %d", dtype);
        return kestrel_check_launch("attn_prepare");
    }
    if (dtype == KESTREL_F32)
        kestrel_launch(attn_prepare_kernel<float>, dim3(blocks), dim3(128), 0, stream, partial, S, (size_t)slice_stride, bias, q_norm_w, k_norm_w, norm_eps, inv_freq, rot, rot_mode, rot_scale, positions,
            seq_of_token, block_table, table_stride, page_size, (float *)k_cache, (float *)v_cache,
            (float *)q_out, T, nq, nkv, hd, write_kv);
    else if (dtype == KESTREL_BF16)
        kestrel_launch(attn_prepare_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, partial, S, (size_t)slice_stride, bias, q_norm_w, k_norm_w, norm_eps, inv_freq, rot, rot_mode, rot_scale, positions,
            seq_of_token, block_table, table_stride, page_size, (__nv_bfloat16 *)k_cache,
            (__nv_bfloat16 *)v_cache, (__nv_bfloat16 *)q_out, T, nq, nkv, hd, write_kv);
    else
        return kestrel_fail(-2, "attn_prepare: unknown dtype %d", dtype);
    return kestrel_check_launch("attn_prepare");
}

// ------------------------------------------------------------------------------------------
// sum of partial slices (+ bias) into a tensor of the storage type; for consumers that have
// no fused form of their own
// ------------------------------------------------------------------------------------------
template <typename TOut>
__global__ void reduce_partials_kernel(const float *__restrict__ partial, int S, size_t slice_stride,
                                       const float *__restrict__ bias, TOut *__restrict__ out,
                                       size_t n, int width) {
    pdl_launch_dependents();
    pdl_wait();
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    float v = 0.f;
    for (int s = 0; s < S; ++s) v += partial[(size_t)s * slice_stride + idx];
    if (bias) v += bias[idx % width];
    out[idx] = from_f32<TOut>(v);
}

KESTREL_API int kestrel_reduce_partials(const float *partial, int S, long long slice_stride,
                                        const float *bias, void *out, int out_dtype, int T, int width,
                                        cudaStream_t stream) {
    if (T == 0) return 0;
    size_t n = (size_t)T * width;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == KESTREL_F32)
        kestrel_launch(reduce_partials_kernel<float>, dim3(blocks), dim3(256), 0, stream, partial, S, (size_t)slice_stride, bias, (float *)out, n, width);
    else if (out_dtype == KESTREL_BF16)
        kestrel_launch(reduce_partials_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, partial, S, (size_t)slice_stride, bias, (__nv_bfloat16 *)out, n, width);
    else
        return kestrel_fail(-2, "reduce_partials: unknown dtype %d", out_dtype);
    return kestrel_check_launch("reduce_partials");
}
