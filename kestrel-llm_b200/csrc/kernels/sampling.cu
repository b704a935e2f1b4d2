// Token selection on the device: argmax, and sampling with temperature, top-k, min-p and
// top-p, one block per row of float32 logits.  Only token ids leave the GPU.
//
// Meaning of the options follows the reference's host sampler
// (src/core/vllm_transformer.c:357-479): temperature <= 0 or top_p <= 0 selects the first
// maximum (:362-367); else p = exp((l - max)/T) / sum (:393-404); top-k keeps the k most
// probable (:413); min-p drops p < min_p * max p (:418-423); top-p keeps the shortest
// descending prefix whose mass reaches top_p, without renormalising in between (:426-458);
// the draw is the first index whose running sum of kept p reaches u * total (:464-471).  The
// reference's zeroing of ids 0, 1 and 3 (:406-409) belongs to its toy tokenizer and is not
// taken over.  The uniform number u in (0, 1] comes from the caller, one per row, so a
// request's draws do not depend on what else is in the batch.
//
// No sort: the k-th largest logit and the top-p cut are found by building the threshold's
// bit pattern from the top bit down, one counting (or mass) pass per bit.  Entries equal to a
// threshold are all kept, where the reference's heap keeps the lower indices; the two differ
// only on exact ties at a cut.
#include "common.cuh"
#include <math.h>

#define SP_THREADS 1024

__device__ __forceinline__ unsigned ordered_key(float f) {
    unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) tot += red[k];
    return tot;
}

__device__ float block_max(float v, float *red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = -INFINITY;
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) tot = fmaxf(tot, red[k]);
    return tot;
}

// first maximum of a row; ties go to the lower index
__device__ int block_argmax(const float *__restrict__ row, int V, float *red, int *redi) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        float v = row[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = best; redi[threadIdx.x >> 5] = bi; }
    __syncthreads();
    float b = red[0];
    int idx = redi[0];
    for (int k = 1; k < (int)(blockDim.x >> 5); ++k)
        if (red[k] > b || (red[k] == b && redi[k] < idx)) { b = red[k]; idx = redi[k]; }
    return idx == 0x7fffffff ? 0 : idx;   // a row of NaN or -inf: index 0, as a strict > scan gives
}

__global__ void __launch_bounds__(SP_THREADS)
argmax_kernel(const float *__restrict__ logits, long long ld, int V, int *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[SP_THREADS / 32];
    __shared__ int redi[SP_THREADS / 32];
    int idx = block_argmax(logits + (size_t)blockIdx.x * ld, V, red, redi);
    if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

// A large vocabulary in two passes, so that a row is read by many SMs: each block finds the
// first maximum of a chunk of ARGMAX_CHUNK entries and writes (value, index) to scratch; then
// one thread per row takes the first maximum over the chunks in ascending order.
#define ARGMAX_CHUNK 8192

__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float *__restrict__ logits, long long ld, int V, float *__restrict__ cand_v,
                     int *__restrict__ cand_i) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[8];
    __shared__ int redi[8];
    int row = blockIdx.x, chunk = blockIdx.y, chunks = gridDim.y;
    int b = chunk * ARGMAX_CHUNK, n = min(ARGMAX_CHUNK, V - b);
    int idx = block_argmax(logits + (size_t)row * ld + b, n, red, redi);
    if (threadIdx.x == 0) {
        cand_v[(size_t)row * chunks + chunk] = logits[(size_t)row * ld + b + idx];
        cand_i[(size_t)row * chunks + chunk] = b + idx;
    }
}

__global__ void argmax_final_kernel(const float *__restrict__ cand_v, const int *__restrict__ cand_i, int chunks,
                                    int R, int *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= R) return;
    const float *v = cand_v + (size_t)row * chunks;
    int best = 0;
    for (int c = 1; c < chunks; ++c)
        if (v[c] > v[best]) best = c;
    out[row] = cand_i[(size_t)row * chunks + best];
}

// scratch (used for V > ARGMAX_CHUNK): float [R * chunks] and int [R * chunks], chunks = ceil(V / 8192)
KESTREL_API int kestrel_argmax(const float *logits, long long ld, int R, int V, int *out, float *cand_v, int *cand_i,
                               cudaStream_t stream) {
    if (R == 0) return 0;
    KESTREL_REQUIRE(R > 0 && V > 0, "argmax: bad sizes R=%d V=%d", R, V);
    int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    if (chunks == 1 || !cand_v || !cand_i) {
        kestrel_launch(argmax_kernel, dim3(R), dim3(SP_THREADS), 0, stream, logits, ld, V, out);
        return kestrel_check_launch("argmax");
    }
    KESTREL_REQUIRE(chunks <= 65535, "argmax: vocabulary %d too large", V);
    kestrel_launch(argmax_chunks_kernel, dim3(dim3(R, chunks)), dim3(256), 0, stream, logits, ld, V, cand_v, cand_i);
    kestrel_launch(argmax_final_kernel, dim3((R + 63) / 64), dim3(64), 0, stream, cand_v, cand_i, chunks, R, out);
    return kestrel_check_launch("argmax");
}

KESTREL_API int kestrel_argmax_chunks(int V) { return (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK; }

__global__ void __launch_bounds__(SP_THREADS)
sample_kernel(const float *__restrict__ logits, long long ld, int V, const float *__restrict__ temperature,
              const int *__restrict__ top_k, const float *__restrict__ top_p, const float *__restrict__ min_p,
              const float *__restrict__ uniform, int *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[SP_THREADS / 32];
    __shared__ int redi[SP_THREADS / 32];
    __shared__ float scan[SP_THREADS];
    __shared__ int pick;
    const float *row = logits + (size_t)blockIdx.x * ld;
    float temp = temperature[blockIdx.x], tp = top_p[blockIdx.x], mp = min_p[blockIdx.x];
    int tk = top_k[blockIdx.x];
    if (temp <= 0.f || tp <= 0.f) {
        int idx = block_argmax(row, V, red, redi);
        if (threadIdx.x == 0) out[blockIdx.x] = idx;
        return;
    }
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += SP_THREADS) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += SP_THREADS) z += expf((row[i] - mx) / temp);
    z = block_sum(z, red);
    float inv_z = 1.0f / z;

    // top-k: largest key x with count(key >= x) >= k
    unsigned key_k = 0u;
    if (tk > 0 && tk < V) {
        for (int bit = 31; bit >= 0; --bit) {
            unsigned cand = key_k | (1u << bit);
            float cnt = 0.f;
            for (int i = threadIdx.x; i < V; i += SP_THREADS) cnt += ordered_key(row[i]) >= cand ? 1.f : 0.f;
            cnt = block_sum(cnt, red);
            if (cnt >= (float)tk) key_k = cand;
        }
    }
    // min-p against the largest probability, which is exp(0)/z
    float floor_p = mp > 0.f ? mp * inv_z : 0.f;
    // top-p: largest key x whose mass(key >= x) reaches top_p among the entries still kept
    unsigned key_p = 0u;
    if (tp < 1.0f) {
        for (int bit = 31; bit >= 0; --bit) {
            unsigned cand = key_p | (1u << bit);
            float mass = 0.f;
            for (int i = threadIdx.x; i < V; i += SP_THREADS) {
                unsigned key = ordered_key(row[i]);
                float p = expf((row[i] - mx) / temp) * inv_z;
                if (key >= key_k && !(p < floor_p) && key >= cand) mass += p;
            }
            mass = block_sum(mass, red);
            if (mass >= tp) key_p = cand;
        }
    }
    unsigned cut = key_k > key_p ? key_k : key_p;

    // draw: contiguous chunk per thread, scan of the chunk sums, then a walk inside one chunk
    int chunk = (V + SP_THREADS - 1) / SP_THREADS;
    int b = threadIdx.x * chunk, e = min(V, b + chunk);
    float s = 0.f;
    for (int i = b; i < e; ++i) {
        float p = expf((row[i] - mx) / temp) * inv_z;
        if (ordered_key(row[i]) >= cut && !(p < floor_p)) s += p;
    }
    scan[threadIdx.x] = s;
    if (threadIdx.x == 0) pick = SP_THREADS;
    __syncthreads();
    for (int off = 1; off < SP_THREADS; off <<= 1) {
        float add = threadIdx.x >= off ? scan[threadIdx.x - off] : 0.f;
        __syncthreads();
        scan[threadIdx.x] += add;
        __syncthreads();
    }
    float total = scan[SP_THREADS - 1];
    float r = uniform[blockIdx.x] * total;
    float incl = scan[threadIdx.x];
    if (s > 0.f && incl >= r) atomicMin(&pick, (int)threadIdx.x);
    __syncthreads();
    if ((int)threadIdx.x == pick) {
        float c = threadIdx.x ? scan[threadIdx.x - 1] : 0.f;
        int chosen = -1, last = -1;
        for (int i = b; i < e && chosen < 0; ++i) {
            float p = expf((row[i] - mx) / temp) * inv_z;
            if (ordered_key(row[i]) >= cut && !(p < floor_p)) {
                c += p;
                last = i;
                if (c >= r) chosen = i;
            }
        }
        out[blockIdx.x] = chosen >= 0 ? chosen : last;
    }
    if (pick == SP_THREADS) {            // nothing kept (a row of NaN): first maximum
        int idx = block_argmax(row, V, red, redi);
        if (threadIdx.x == 0) out[blockIdx.x] = idx;
    }
}

KESTREL_API int kestrel_sample(const float *logits, long long ld, int R, int V, const float *temperature,
                               const int *top_k, const float *top_p, const float *min_p,
                               const float *uniform, int *out, cudaStream_t stream) {
    if (R == 0) return 0;
    KESTREL_REQUIRE(R > 0 && V > 0, "sample: bad sizes R=%d V=%d", R, V);
    kestrel_launch(sample_kernel, dim3(R), dim3(SP_THREADS), 0, stream, logits, ld, V, temperature, top_k, top_p, min_p, uniform, out);
    return kestrel_check_launch("sample");
}
