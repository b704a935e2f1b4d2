// Token selection on the device: argmax, and sampling with temperature, top-k, min-p and
// top-p over rows of float32 logits.  Only token ids leave the GPU.  A row is sampled by the
// CTAs of a cluster that keep it in shared memory (sample_cluster_kernel, further down), or,
// where it does not fit, by one block over global memory (sample_kernel).
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
// bit pattern from the top bits down, one counting (or mass) pass per bit (sample_kernel) or
// per four bits (sample_cluster_kernel).  Entries equal to a
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

// ------------------------------------------------------------------------------------------
// The same selection for vocabularies that fit the shared memory of a cluster: the row is cut
// over the CTAs of a cluster (up to 8), each CTA keeps its slice - logits and, where they fit
// too, probabilities - in shared memory, reads global memory once, and every further pass runs
// from there.  Thresholds are built 4 bits at a time: one pass fills 16 buckets (counts for
// top-k, probability mass for top-p) for the entries that match the bits found so far, the
// buckets are summed over the block and then over the cluster in rank order through
// distributed shared memory, and every CTA takes the same digit from them.  8 + 8 passes and
// about 20 cluster barriers instead of 65 passes of one block over global memory (the
// vocabulary of 151,936, 8 rows, all filters: 1,380 -> 82 us).  Many rows run two CTAs on an SM
// where leaving the probabilities out lets them fit.  Sums are taken in a fixed order
// (thread, warp, block, rank), so a row's token does not depend on what else is in the batch.
// ------------------------------------------------------------------------------------------
#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)
#define SC_BINS 16
#define SC_MAX_CLUSTER 8
#define SC_SMEM_LIMIT (200 * 1024)

__device__ __forceinline__ uint32_t sc_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t sc_ranks() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the float at the same shared-memory address in CTA `rank` of this cluster
__device__ __forceinline__ float sc_remote(const float *local, uint32_t rank) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(local), remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

struct ScShared {
    float wred[SC_WARPS][SC_BINS];      // per-warp partial sums of the 16 buckets
    float xch[2][SC_BINS];              // this CTA's sums, read by the other ranks; two turns
    float res[SC_BINS];                 // the cluster's sums
    float scan[SC_THREADS];
    int pick;
};

// v[0..n) summed over the block (lane tree, then warps in ascending order) and over the
// cluster (ranks in ascending order); every thread of every CTA gets the same totals in sh.res.
// One cluster barrier a call; `turn` alternates so that a slot is not overwritten while a
// slower CTA still reads it.
template <int N>
__device__ __forceinline__ void sc_reduce(float (&v)[N], ScShared &sh, int &turn) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int b = 0; b < N; ++b) v[b] = warp_sum(v[b]);
    if (lane == 0) {
#pragma unroll
        for (int b = 0; b < N; ++b) sh.wred[warp][b] = v[b];
    }
    __syncthreads();
    if (threadIdx.x < N) {
        float t = 0.f;
        for (int w = 0; w < SC_WARPS; ++w) t += sh.wred[w][threadIdx.x];
        sh.xch[turn][threadIdx.x] = t;
    }
    sc_cluster_sync();
    if (threadIdx.x < N) {
        float t = 0.f;
        const uint32_t n = sc_ranks();
        for (uint32_t r = 0; r < n; ++r) t += sc_remote(&sh.xch[turn][threadIdx.x], r);
        sh.res[threadIdx.x] = t;
    }
    __syncthreads();
    turn ^= 1;
}

template <bool STORE_P>
__global__ void __launch_bounds__(SC_THREADS, 2)
sample_cluster_kernel(const float *__restrict__ logits, long long ld, int V, int S, const float *__restrict__ temperature,
                      const int *__restrict__ top_k, const float *__restrict__ top_p, const float *__restrict__ min_p,
                      const float *__restrict__ uniform, int *__restrict__ out) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) float sc_dyn[];
    __shared__ ScShared sh;
    float *vals = sc_dyn;                           // [S] this CTA's logits
    float *probs = sc_dyn + (STORE_P ? S : 0);      // [S] their probabilities (unnormalised), if kept
    const int tid = threadIdx.x;
    const uint32_t rank = sc_rank();
    const int rowi = blockIdx.y;
    const int base = (int)rank * S, n = max(0, min(S, V - base));
    pdl_wait();
    const float temp = temperature[rowi], tp = top_p[rowi], mp = min_p[rowi], u = uniform[rowi];
    const int tk = top_k[rowi];
    const float *row = logits + (size_t)rowi * ld + base;
    int turn = 0;

    // the slice into shared memory; its first maximum on the way
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < n; i += SC_THREADS) {
        float v = row[i];
        vals[i] = v;
        if (v > best) { best = v; bi = base + i; }          // ascending i per thread: the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, best, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { sh.wred[tid >> 5][0] = best; sh.wred[tid >> 5][1] = __int_as_float(bi); }
    __syncthreads();
    if (tid == 0) {
        float b = sh.wred[0][0];
        int idx = __float_as_int(sh.wred[0][1]);
        for (int w = 1; w < SC_WARPS; ++w) {
            float wv = sh.wred[w][0];
            int wi = __float_as_int(sh.wred[w][1]);
            if (wv > b || (wv == b && wi < idx)) { b = wv; idx = wi; }
        }
        sh.xch[turn][0] = b;
        sh.xch[turn][1] = __int_as_float(idx);
    }
    sc_cluster_sync();
    float mx = -INFINITY;
    int arg = 0x7fffffff;
    {
        const uint32_t nr = sc_ranks();
        for (uint32_t r = 0; r < nr; ++r) {             // ranks in ascending order hold ascending indices
            float rv = sc_remote(&sh.xch[turn][0], r);
            int ri = __float_as_int(sc_remote(&sh.xch[turn][1], r));
            if (rv > mx || (rv == mx && ri < arg)) { mx = rv; arg = ri; }
        }
    }
    turn ^= 1;
    if (arg == 0x7fffffff) arg = 0;                     // a row of NaN or -inf
    const bool greedy = temp <= 0.f || tp <= 0.f;
    bool done = greedy;
    float inv_z = 0.f, floor_p = 0.f;
    unsigned cut = 0u;
    if (!greedy) {
        // probabilities and their sum
        float z[1] = {0.f};
        for (int i = tid; i < n; i += SC_THREADS) {
            float e = expf((vals[i] - mx) / temp);
            if (STORE_P) probs[i] = e;
            z[0] += e;
        }
        sc_reduce<1>(z, sh, turn);
        inv_z = 1.0f / sh.res[0];
        floor_p = mp > 0.f ? mp * inv_z : 0.f;
        auto prob = [&](int i) { return (STORE_P ? probs[i] : expf((vals[i] - mx) / temp)) * inv_z; };

        // top-k: the largest key x with count(key >= x) >= k, 4 bits a pass
        unsigned key_k = 0u;
        if (tk > 0 && tk < V) {
            float above = 0.f;                          // entries whose key lies above the prefix's range
            for (int shift = 28; shift >= 0; shift -= 4) {
                float c[SC_BINS];
#pragma unroll
                for (int b = 0; b < SC_BINS; ++b) c[b] = 0.f;
                for (int i = tid; i < n; i += SC_THREADS) {
                    unsigned key = ordered_key(vals[i]);
                    if (shift == 28 || (key >> (shift + 4)) == (key_k >> (shift + 4))) {
                        unsigned d = (key >> shift) & 15u;
#pragma unroll
                        for (int b = 0; b < SC_BINS; ++b) c[b] += d == (unsigned)b ? 1.f : 0.f;
                    }
                }
                sc_reduce<SC_BINS>(c, sh, turn);
                // the highest bucket with which the count reaches k; none (k beyond the entries that are
                // left) means the lowest
                float run = above;
                int d = 0;
                for (int b = SC_BINS - 1; b >= 1; --b) {
                    float with_b = run + sh.res[b];
                    if (with_b >= (float)tk) { d = b; break; }
                    run = with_b;
                }
                above = run;
                key_k |= (unsigned)d << shift;
            }
        }
        // top-p: the largest key x whose mass(key >= x) reaches top_p among the entries still kept
        unsigned key_p = 0u;
        if (tp < 1.0f) {
            float above = 0.f;
            for (int shift = 28; shift >= 0; shift -= 4) {
                float m[SC_BINS];
#pragma unroll
                for (int b = 0; b < SC_BINS; ++b) m[b] = 0.f;
                for (int i = tid; i < n; i += SC_THREADS) {
                    unsigned key = ordered_key(vals[i]);
                    if (key >= key_k && (shift == 28 || (key >> (shift + 4)) == (key_p >> (shift + 4)))) {
                        float p = prob(i);
                        if (!(p < floor_p)) {
                            unsigned d = (key >> shift) & 15u;
#pragma unroll
                            for (int b = 0; b < SC_BINS; ++b) m[b] += d == (unsigned)b ? p : 0.f;
                        }
                    }
                }
                sc_reduce<SC_BINS>(m, sh, turn);
                float run = above;
                int d = 0;
                for (int b = SC_BINS - 1; b >= 1; --b) {
                    float with_b = run + sh.res[b];
                    if (with_b >= tp) { d = b; break; }
                    run = with_b;
                }
                above = run;                            // if the mass never reaches top_p every digit is 0: all is kept
                key_p |= (unsigned)d << shift;
            }
        }
        cut = key_k > key_p ? key_k : key_p;

        // draw: a contiguous chunk per thread, scan of the chunk sums over the block, the CTAs'
        // totals over the cluster, then a walk inside one chunk
        const int chunk = (S + SC_THREADS - 1) / SC_THREADS;
        const int b0 = min(n, tid * chunk), e0 = min(n, b0 + chunk);
        float s = 0.f;
        for (int i = b0; i < e0; ++i) {
            float p = prob(i);
            if (ordered_key(vals[i]) >= cut && !(p < floor_p)) s += p;
        }
        sh.scan[tid] = s;
        if (tid == 0) sh.pick = SC_THREADS;
        __syncthreads();
        for (int off = 1; off < SC_THREADS; off <<= 1) {
            float add = tid >= off ? sh.scan[tid - off] : 0.f;
            __syncthreads();
            sh.scan[tid] += add;
            __syncthreads();
        }
        const float cta_total = sh.scan[SC_THREADS - 1];
        if (tid == 0) sh.xch[turn][0] = cta_total;
        sc_cluster_sync();
        // the CTA in which the running sum of kept probability first reaches u * total: every CTA
        // finds the same one from the same sums
        float total = 0.f;
        const uint32_t nr = sc_ranks();
        for (uint32_t r = 0; r < nr; ++r) total += sc_remote(&sh.xch[turn][0], r);
        const float target = u * total;
        float before = 0.f, run = 0.f;
        int owner_rank = -1;
        for (uint32_t r = 0; r < nr; ++r) {
            float t = sc_remote(&sh.xch[turn][0], r);
            float end = run + t;
            if (owner_rank < 0 && t > 0.f && end >= target) { owner_rank = (int)r; before = run; }
            run = end;
        }
        turn ^= 1;
        if (total > 0.f && owner_rank >= 0) {
            done = true;
            const bool owner = owner_rank == (int)rank;
            const float rl = fminf(target - before, cta_total);
            if (owner) {
                const float incl = sh.scan[tid];
                if (s > 0.f && incl >= rl) atomicMin(&sh.pick, tid);
            }
            __syncthreads();
            if (owner && tid == sh.pick) {
                float c = tid ? sh.scan[tid - 1] : 0.f;
                int chosen = -1, last = -1;
                for (int i = b0; i < e0 && chosen < 0; ++i) {
                    float p = prob(i);
                    if (ordered_key(vals[i]) >= cut && !(p < floor_p)) {
                        c += p;
                        last = i;
                        if (c >= rl) chosen = i;
                    }
                }
                out[rowi] = base + (chosen >= 0 ? chosen : last);
            }
        }
    }
    if ((greedy || !done) && rank == 0 && tid == 0) out[rowi] = arg;    // greedy, or nothing kept (a row of NaN): first maximum
    sc_cluster_sync();                  // nobody leaves while its shared memory may still be read
}

// CTAs of a cluster for a vocabulary of V and whether the probabilities fit beside the logits;
// 0 if the row does not fit a cluster's shared memory (the one-block kernel takes it then)
static int sample_cluster_shape(int V, int R, int *slice, int *store_p) {
    for (int cl = 1; cl <= SC_MAX_CLUSTER; cl *= 2) {
        int S = (((V + cl - 1) / cl) + 3) & ~3;
        bool last = cl == SC_MAX_CLUSTER;
        if (!last && S > 8192) continue;               // more CTAs while a slice is long
        // many rows: two CTAs on an SM, if leaving the probabilities out lets them fit
        bool crowded = (long long)R * cl > kestrel_sms() && (size_t)S * 8 > 100 * 1024 && (size_t)S * 4 <= 100 * 1024;
        if (!crowded && (size_t)S * 8 <= SC_SMEM_LIMIT) { *slice = S; *store_p = 1; return cl; }
        if ((size_t)S * 4 <= SC_SMEM_LIMIT) { *slice = S; *store_p = 0; return cl; }
    }
    return 0;
}

// ------------------------------------------------------------------------------------------
// Repetition penalty of the reference's streaming harness (src/main.c:3741-3782): for each of
// the last `window` tokens a request generated, most recent first, the token's logit l becomes
// l / p if l >= 0, else l * p - once per occurrence, so a token that appears twice in the window
// is penalised twice.  history int32 [R, width]: row r holds that request's last tokens (entries
// beyond counts[r], or outside the vocabulary, are skipped); penalty float [R], <= 1 = off.
// One thread a row: the steps on one token follow each other, and there are 64 at most.
// ------------------------------------------------------------------------------------------
__global__ void repetition_penalty_kernel(float *__restrict__ logits, long long ld, int V, const int *__restrict__ history,
                                          int width, const int *__restrict__ counts, const float *__restrict__ penalty, int R) {
    pdl_launch_dependents();
    pdl_wait();
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    float p = penalty[r];
    if (!(p > 1.0f)) return;
    float *row = logits + (size_t)r * ld;
    int n = min(counts[r], width);
    for (int h = 0; h < n; ++h) {
        int tok = history[(size_t)r * width + h];
        if (tok < 0 || tok >= V) continue;
        float l = row[tok];
        row[tok] = l >= 0.0f ? l / p : l * p;
    }
}

KESTREL_API int kestrel_repetition_penalty(float *logits, long long ld, int R, int V, const int *history, int width,
                                           const int *counts, const float *penalty, cudaStream_t stream) {
    if (R == 0) return 0;
    KESTREL_REQUIRE(R > 0 && V > 0 && width > 0, "repetition_penalty: bad sizes R=%d V=%d width=%d", R, V, width);
    kestrel_launch(repetition_penalty_kernel, dim3((R + 63) / 64), dim3(64), 0, stream, logits, ld, V, history, width, counts, penalty, R);
    return kestrel_check_launch("repetition_penalty");
}

static int g_sample_cluster = 1;    // 0: always the one-block kernel (for tests of it)
KESTREL_API void kestrel_sample_set_cluster(int on) { g_sample_cluster = on ? 1 : 0; }

KESTREL_API int kestrel_sample(const float *logits, long long ld, int R, int V, const float *temperature,
                               const int *top_k, const float *top_p, const float *min_p,
                               const float *uniform, int *out, cudaStream_t stream) {
    if (R == 0) return 0;
    KESTREL_REQUIRE(R > 0 && V > 0, "sample: bad sizes R=%d V=%d", R, V);
    int S = 0, store_p = 0;
    int cl = g_sample_cluster && R <= 65535 && V < (1 << 24) ? sample_cluster_shape(V, R, &S, &store_p) : 0;
    if (cl > 0) {
        size_t smem = (size_t)S * 4 * (store_p ? 2 : 1);
        static bool attr_set = false;
        if (!attr_set) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SC_SMEM_LIMIT);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_cluster_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SC_SMEM_LIMIT);
            if (e != cudaSuccess) return kestrel_fail(-3, "sample: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
            attr_set = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(cl, R);
        cfg.blockDim = dim3(SC_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = cl;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_kestrel_pdl ? 2 : 1;
        if (store_p) cudaLaunchKernelEx(&cfg, sample_cluster_kernel<true>, logits, ld, V, S, temperature, top_k, top_p, min_p, uniform, out);
        else cudaLaunchKernelEx(&cfg, sample_cluster_kernel<false>, logits, ld, V, S, temperature, top_k, top_p, min_p, uniform, out);
        return kestrel_check_launch("sample");
    }
    kestrel_launch(sample_kernel, dim3(R), dim3(SP_THREADS), 0, stream, logits, ld, V, temperature, top_k, top_p, min_p, uniform, out);
    return kestrel_check_launch("sample");
}
