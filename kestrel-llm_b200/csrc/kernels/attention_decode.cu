// Attention of decode tokens over the paged cache: few rows, many keys, bound by the stream of
// keys and values from HBM.  Head sizes 64 and 128.
//
// As in the KEYS mode of attention_mma.cu a CTA takes the (token, query head) rows of one
// (request, kv head) - at most 16 - and one slice of the key range; its four consumer warps
// share the rows, each takes 16 keys of every 64-key tile (mma.sync.m16n8k16, float32 softmax
// statistics and accumulators in registers) and the four running (max, sum, out) states are
// merged in warp order at the end; up to 4 slices of a key range are the CTAs of a cluster and
// merge their results over distributed shared memory, more go through scratch and
// attention_merge_kernel (clusters of 8 were measured to be placed badly among the kernels of a
// step: twice the time at 4 requests).  What differs further is how the tiles arrive: a fifth warp fetches
// them with TMA (boxes of one page - or 64 keys of a larger page - by 64 dims, 128-byte swizzle)
// into a ring of stages and runs ahead of the consumers as far as the ring allows; full/empty
// mbarriers couple the two sides, so no warp issues copies between its products and the CTA
// never meets at a block-wide barrier inside the loop.  Tiles that end before the request's
// first new position hold only what earlier steps wrote; the loader fetches those before it
// waits for the predecessor kernel (which writes the new tokens' keys and values), so the
// stream is already running when that kernel ends.
//
// TMA brings whole pages: keys outside [first key, last key] of the rows are masked in the
// scores, and their V rows are zeroed in shared memory before the product reads them (a page may
// hold another request's stale values there, and 0 x NaN would not be 0).  ldmatrix addresses
// follow the swizzle: 16-byte chunk c of row r of a 64-dim panel lies at r * 128 + ((c ^ r % 8) << 4).
// Every mbarrier wait is bounded; the error word is read by kestrel_attention_decode_error.
// Formulas as in attention_plain.cu (reference: st.c:10779-10911, st.c:9762-9859).
#include "attention_params.cuh"
#include "mma_sync.cuh"
#include "tcgen05.cuh"
#include <math.h>

#define AD_THREADS 160          // 4 consumer warps + the loader
#define AD_BN 64                // keys per tile
#ifndef AD_STAGES
#define AD_STAGES 3               // stages of the ring: 3 x 32 KB at head size 128, two CTAs per SM
#endif
#define AD_PANEL (AD_BN * 128)  // bytes of a panel: 64 keys x 64 dims
#ifndef AD_MAX_CLUSTER
#define AD_MAX_CLUSTER 4        // slices merged by one cluster
#endif

__device__ int g_ad_error = 0;

// a float of CTA `rank` of this cluster, at the shared-memory address `addr` of this CTA's window
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr, int rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

template <int HD, bool CLUSTER>
__global__ void __launch_bounds__(AD_THREADS)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const AttnParams p, int cache_pages) {
    pdl_launch_dependents();
    constexpr int PANELS = HD / 64;
    constexpr uint32_t TILE_BYTES = PANELS * AD_PANEL;          // K (or V) of one tile
    constexpr uint32_t STAGE_BYTES = 2 * TILE_BYTES;
    constexpr int LDQ = HD + 8;                                 // padded Q row, in elements
    constexpr int KS = HD / 16;                                 // k-steps of the QK product
    constexpr int NT_O = HD / 8;                                // 8-dim tiles of the output
    constexpr uint32_t FIN_OFFSET = 4 * 16 * HD * 4 + 1024;     // behind the four warps' states in the ring's memory
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *ring = smem_raw + (base - smem_u32(smem_raw));     // [AD_STAGES][K tile | V tile]
    __nv_bfloat16 *Qs = reinterpret_cast<__nv_bfloat16 *>(ring + AD_STAGES * STAGE_BYTES);        // [16][LDQ]
    const uint32_t bars = base + AD_STAGES * STAGE_BYTES + 16 * LDQ * 2;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (AD_STAGES + s); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < AD_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // The step's description (lengths, tables, slice length) was copied to the device before the
    // step's first kernel began; reading it does not have to wait for the predecessor kernel.
    const int tile = blockIdx.x, kvh = blockIdx.y, slice = blockIdx.z;
    const int seq = p.tile_seq[tile], row0 = p.tile_row0[tile];
    const int G = p.nq / p.nkv;
    const int tok_begin = p.cu_seqlens[seq], n_tok = p.cu_seqlens[seq + 1] - tok_begin;
    const int kv_len = p.kv_lens[seq];
    const int pos_begin = kv_len - n_tok;             // position of the request's first token of this step
    const int rows_here = min(16, n_tok * G - row0);
    const int *table = p.block_table + (size_t)seq * p.table_stride;
    const int slice_len = attn_slice_len(p);
    const int first_tok = row0 / G, last_tok = (row0 + rows_here - 1) / G;
    int k_hi = min(pos_begin + last_tok + 1, (slice + 1) * slice_len);          // exclusive
    const int k_first = max(p.window > 0 ? max(0, pos_begin + first_tok - p.window + 1) : 0, slice * slice_len);
    const int k_lo = (k_first / AD_BN) * AD_BN;
    const int n_tiles = k_hi > k_lo ? (k_hi - k_lo + AD_BN - 1) / AD_BN : 0;

    if (warp == 4) {
        // ------------------------------------------------------------------ loader
        // lane l fetches the l-th page of a tile: every panel of K, then of V
        const int box_rows = min(p.page_size, AD_BN);
        const int boxes = AD_BN / box_rows;
        bool waited = false;
        for (int t = 0; t < n_tiles; ++t) {
            const int stage = t % AD_STAGES;
            const uint32_t par = (uint32_t)(t / AD_STAGES) & 1u;
            const int kb = k_lo + t * AD_BN;
            if (!waited && kb + AD_BN > pos_begin) {        // this tile may hold keys the predecessor writes
                pdl_wait();
                waited = true;
            }
            int row = 0;
            if (lane < boxes) {
                int s0 = kb + lane * box_rows;
                int idx = s0 / p.page_size;
                int page = idx < p.table_width ? table[idx] : 0;
                if (page < 0 || page >= cache_pages) page = 0;      // a released or absent page: its keys are masked, its values zeroed
                row = (page * p.nkv + kvh) * p.page_size + s0 % p.page_size;
            }
            if (!mbar_wait(empty_bar(stage), par ^ 1u)) { atomicExch(&g_ad_error, 1); break; }
            if (lane == 0) mbar_expect_tx(full_bar(stage), STAGE_BYTES);
            __syncwarp();
            if (lane < boxes) {
                const uint32_t dst = base + stage * STAGE_BYTES + lane * box_rows * 128;
#pragma unroll
                for (int pn = 0; pn < PANELS; ++pn) {
                    tma_load_2d(dst + pn * AD_PANEL, &map_k, full_bar(stage), 64 * pn, row);
                    tma_load_2d(dst + TILE_BYTES + pn * AD_PANEL, &map_v, full_bar(stage), 64 * pn, row);
                }
            }
        }
    } else {
    // ---------------------------------------------------------------------- consumers
    pdl_wait();                                       // the queries are the predecessor's output
    for (int idx = tid; idx < 16 * (HD / 8); idx += 128) {
        int r = idx / (HD / 8), c = idx % (HD / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows_here) {
            int row = row0 + r;
            v = *reinterpret_cast<const uint4 *>(p.q + ((size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G) * HD + c * 8);
        }
        *reinterpret_cast<uint4 *>(Qs + r * LDQ + c * 8) = v;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");

    int pos_r[2], lo_r[2];
    int min_pos = 0x7fffffff, max_lo = 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        int r = (lane >> 2) + 8 * i;                  // the rows this thread holds
        bool ok = r < rows_here;
        int ps = pos_begin + (row0 + r) / G;
        pos_r[i] = ok ? ps : -1;                      // an absent row sees no key
        lo_r[i] = p.window > 0 ? max(0, ps - p.window + 1) : 0;
        min_pos = min(min_pos, pos_r[i]);
        max_lo = max(max_lo, lo_r[i]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {          // over the warp: tiles every row sees whole need no mask
        min_pos = min(min_pos, __shfl_xor_sync(0xffffffffu, min_pos, off));
        max_lo = max(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, off));
    }
    float o[NT_O][4];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
    bool ok = true;             // after a wait gave up the loop runs on without waiting, so that the warps still meet below

    for (int t = 0; t < n_tiles; ++t) {
        const int stage = t % AD_STAGES;
        if (ok && !mbar_wait(full_bar(stage), (uint32_t)(t / AD_STAGES) & 1u)) { atomicExch(&g_ad_error, 2); ok = false; }
        const int kbase = k_lo + t * AD_BN + 16 * warp;                 // this warp's 16 keys
        const uint32_t Kt = base + stage * STAGE_BYTES + (16 * warp) * 128;
        const uint32_t Vt = Kt + TILE_BYTES;
        if (ok && kbase < k_hi && kbase <= pos_begin + last_tok && kbase + 16 > k_first) {
            if (kbase < k_first || kbase + 16 > k_hi) {
                // V rows of keys outside the range become zero: 16 rows x HD / 8 chunks over the lanes
                uint8_t *vrows = ring + stage * STAGE_BYTES + TILE_BYTES + (16 * warp) * 128;
                for (int idx = lane; idx < 16 * (HD / 8); idx += 32) {
                    int r = idx / (HD / 8), c = idx % (HD / 8);
                    int key = kbase + r;
                    if (key < k_first || key >= k_hi)
                        *reinterpret_cast<uint4 *>(vrows + (c >> 3) * AD_PANEL + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            float s[2][4];
            s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t a[4], b0, b1, b2, b3;
                // A fragments of Q: rows lane % 16, columns 16 ks + 8 (lane / 16)
                ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Qs + (lane & 15) * LDQ + ks * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
                // keys (lane % 8) + 8 (lane / 16), dims 16 ks + 8 ((lane / 8) % 2)
                const int kr = (lane & 7) + ((lane >> 4) << 3);
                const int kc = 2 * ks + ((lane >> 3) & 1);                  // 16-byte chunk of the row
                ldmatrix_x4(Kt + (kc >> 3) * AD_PANEL + kr * 128 + (((kc & 7) ^ (kr & 7)) << 4), b0, b1, b2, b3);
                mma_bf16(s[0], a, b0, b1);
                mma_bf16(s[1], a, b2, b3);
            }
            // scale, mask (only on tiles that some row does not see whole), running maximum
            const bool whole = kbase >= k_first && kbase + 16 <= k_hi && kbase + 15 <= min_pos && kbase >= max_lo;
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    int i = e >> 1;
                    float v = s[nt][e] * p.scale_log2;
                    if (!whole) {
                        int key = kbase + nt * 8 + 2 * (lane & 3) + (e & 1);
                        bool vis = key <= pos_r[i] && key >= lo_r[i] && key < k_hi && key >= k_first;
                        v = vis ? v : -INFINITY;
                    }
                    s[nt][e] = v;
                    mx[i] = fmaxf(mx[i], v);
                }
            float alpha[2], m_use[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                float mn = fmaxf(m_r[i], mx[i]);
                m_use[i] = mn == -INFINITY ? 0.f : mn;             // a row that has seen no key yet
                alpha[i] = fast_exp2(m_r[i] - m_use[i]);           // exp2(-inf) = 0 on the first keys
                m_r[i] = mn;
                l_r[i] *= alpha[i];
            }
#pragma unroll
            for (int nt = 0; nt < NT_O; ++nt) {
                o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
                o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float pv = fast_exp2(s[nt][e] - m_use[e >> 1]);
                    s[nt][e] = pv;
                    l_r[e >> 1] += pv;
                }
            // out += P V
            uint32_t a[4];
            a[0] = pack_bf16(s[0][0], s[0][1]);
            a[1] = pack_bf16(s[0][2], s[0][3]);
            a[2] = pack_bf16(s[1][0], s[1][1]);
            a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int dp = 0; dp < NT_O / 2; ++dp) {
                uint32_t b0, b1, b2, b3;
                // keys (lane % 8) + 8 ((lane / 8) % 2), dims 16 dp + 8 (lane / 16), transposed
                const int vr = (lane & 7) + (((lane >> 3) & 1) << 3);
                const int vc = 2 * dp + (lane >> 4);
                ldmatrix_x4_trans(Vt + (vc >> 3) * AD_PANEL + vr * 128 + (((vc & 7) ^ (vr & 7)) << 4), b0, b1, b2, b3);
                mma_bf16(o[2 * dp], a, b0, b1);
                mma_bf16(o[2 * dp + 1], a, b2, b3);
            }
            if (kbase < k_first || kbase + 16 > k_hi)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the zeroed rows before the next copy into them
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage));
    }

    // row sums across the four threads of a row
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 1);
        l_r[i] += __shfl_xor_sync(0xffffffffu, l_r[i], 2);
    }

    // merge the four warps' states in warp order through shared memory (the ring is free: every
    // tile the loader fetched has been consumed)
    asm volatile("bar.sync 1, 128;" ::: "memory");
    float *mo = reinterpret_cast<float *>(ring);                // [4][16][HD]
    float *mml = mo + 4 * 16 * HD;                              // [4][16][2]
    float *fin = reinterpret_cast<float *>(ring + FIN_OFFSET);  // [16][HD], then [16][2]: this CTA's merged slice (clusters)
    float *finml = fin + 16 * HD;
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
        int d = nt * 8 + 2 * (lane & 3);
        *reinterpret_cast<float2 *>(mo + ((size_t)warp * 16 + (lane >> 2)) * HD + d) = make_float2(o[nt][0], o[nt][1]);
        *reinterpret_cast<float2 *>(mo + ((size_t)warp * 16 + (lane >> 2) + 8) * HD + d) = make_float2(o[nt][2], o[nt][3]);
    }
    if ((lane & 3) == 0) {
        mml[(warp * 16 + (lane >> 2)) * 2] = m_r[0];
        mml[(warp * 16 + (lane >> 2)) * 2 + 1] = l_r[0];
        mml[(warp * 16 + (lane >> 2) + 8) * 2] = m_r[1];
        mml[(warp * 16 + (lane >> 2) + 8) * 2 + 1] = l_r[1];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // thread -> (row, 8-dim group): 16 rows x HD/8 groups
    for (int idx = tid; idx < 16 * (HD / 8); idx += 128) {
        int r = idx / (HD / 8), d0 = (idx % (HD / 8)) * 8;
        if (r >= rows_here) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
        float L = 0.f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            float mw = mml[(w * 16 + r) * 2];
            if (mw == -INFINITY) continue;
            float f = exp2f(mw - M);
            L += mml[(w * 16 + r) * 2 + 1] * f;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += mo[((size_t)w * 16 + r) * HD + d0 + j] * f;
        }
        int row = row0 + r;
        size_t qrow = (size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G;
        if (CLUSTER) {
            // this slice's unnormalised out, maximum and sum stay in shared memory for the cluster's merge
            *reinterpret_cast<float4 *>(fin + r * HD + d0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4 *>(fin + r * HD + d0 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            if (d0 == 0) { finml[2 * r] = M; finml[2 * r + 1] = L; }
        } else if (!ok) {
            // a wait gave up: nothing is written
        } else if (p.slices > 1) {
            float *po = p.part_o + (qrow * p.slices + slice) * HD + d0;
            *reinterpret_cast<float4 *>(po) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4 *>(po + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            if (d0 == 0) { p.part_ml[(qrow * p.slices + slice) * 2] = M; p.part_ml[(qrow * p.slices + slice) * 2 + 1] = L; }
        } else {
            float inv = 1.0f / L;
            uint4 u;
            u.x = pack_bf16(acc[0] * inv, acc[1] * inv);
            u.y = pack_bf16(acc[2] * inv, acc[3] * inv);
            u.z = pack_bf16(acc[4] * inv, acc[5] * inv);
            u.w = pack_bf16(acc[6] * inv, acc[7] * inv);
            *reinterpret_cast<uint4 *>(p.out + qrow * HD + d0) = u;
        }
    }
    }   // consumers

    if (CLUSTER) {
        // The slices of one (request, kv head) are the CTAs of one cluster (1, 1, slices): their
        // results are merged over distributed shared memory, in ascending order of the slices, and
        // the rows are shared out among the CTAs.  Every thread of every CTA takes part in the
        // cluster barriers; no CTA leaves while its shared memory may still be read.
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
        const uint32_t fin_s = base + FIN_OFFSET, finml_s = fin_s + 16 * HD * 4;
        if (warp < 4) {
            for (int idx = tid; idx < 16 * (HD / 8); idx += 128) {
                int r = idx / (HD / 8), d0 = (idx % (HD / 8)) * 8;
                if (r >= rows_here || r % p.slices != slice) continue;
                float M = -INFINITY;
                for (int s = 0; s < p.slices; ++s) M = fmaxf(M, ld_cluster_f32(finml_s + 8 * r, s));
                float L = 0.f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int s = 0; s < p.slices; ++s) {
                    float ms = ld_cluster_f32(finml_s + 8 * r, s);
                    if (ms == -INFINITY) continue;
                    float f = exp2f(ms - M);
                    L += ld_cluster_f32(finml_s + 8 * r + 4, s) * f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] += ld_cluster_f32(fin_s + (r * HD + d0 + j) * 4, s) * f;
                }
                int row = row0 + r;
                size_t qrow = (size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G;
                uint4 u;
                u.x = pack_bf16(acc[0] / L, acc[1] / L);
                u.y = pack_bf16(acc[2] / L, acc[3] / L);
                u.z = pack_bf16(acc[4] / L, acc[5] / L);
                u.w = pack_bf16(acc[6] / L, acc[7] / L);
                *reinterpret_cast<uint4 *>(p.out + qrow * HD + d0) = u;
            }
        }
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
}

template <int HD>
static size_t decode_smem() { return (size_t)AD_STAGES * 2 * (HD / 64) * AD_PANEL + 16 * (HD + 8) * 2 + 16 * AD_STAGES + 1024; }

template <int HD, bool CLUSTER>
static int launch_decode(const CUtensorMap &mk, const CUtensorMap &mv, const AttnParams &p, int tiles, int cache_pages,
                         cudaStream_t stream) {
    size_t smem = decode_smem<HD>();
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return kestrel_fail(-3, "attention_decode: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    if (CLUSTER) {
        // the slices of a (request, kv head) form a cluster; programmatic dependent launch as everywhere
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(tiles, p.nkv, p.slices);
        cfg.blockDim = dim3(AD_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = p.slices;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_kestrel_pdl ? 2 : 1;
        cudaLaunchKernelEx(&cfg, attention_decode_kernel<HD, CLUSTER>, mk, mv, p, cache_pages);
    } else {
        kestrel_launch(attention_decode_kernel<HD, CLUSTER>, dim3(tiles, p.nkv, p.slices), dim3(AD_THREADS), smem, stream, mk, mv, p, cache_pages);
    }
    return kestrel_check_launch("attention_decode");
}

// Whether the kernel takes this head size and page size.
KESTREL_API int kestrel_attention_decode_supported(int hd, int page_size) {
    return (hd == 64 || hd == 128) && page_size > 0 && page_size % 8 == 0 && (AD_BN % page_size == 0 || page_size % AD_BN == 0);
}

// CTAs of the kernel that the GPU's SMs hold at once, by shared memory
KESTREL_API int kestrel_attention_decode_slots(int hd) {
    size_t smem = hd == 64 ? decode_smem<64>() : decode_smem<128>();
    int per_sm = (int)((227 * 1024) / (smem + 1024));
    return kestrel_sms() * (per_sm < 1 ? 1 : per_sm);
}

// Tiles of at most 16 rows (tile_seq / tile_row0): decode tokens.  The key range is cut into
// `slices` slices of slice_len keys, a multiple of 64 - or a length that follows the longest
// request at max_kv_ptr on the device - which are merged in ascending order; part_o / part_ml
// are scratch of T * nq * slices * hd and T * nq * slices * 2 floats.  cache_pages is the number of pages the cache tensors hold.
KESTREL_API int kestrel_attention_decode(const void *q, const void *k_cache, const void *v_cache, void *out,
                                         float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0,
                                         int tiles, const int *cu_seqlens, const int *kv_lens, const int *block_table,
                                         int table_width, int table_stride, int page_size, int cache_pages, int T, int nq,
                                         int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr,
                                         float scale, cudaStream_t stream) {
    if (T == 0 || tiles == 0) return 0;
    KESTREL_REQUIRE(kestrel_attention_decode_supported(hd, page_size),
                    "attention_decode: head size %d with pages of %d keys; the head size must be 64 or 128 and the page size a multiple of 8 that divides 64 or is a multiple of it", hd, page_size);
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && nq / nkv <= 16, "attention_decode: %d query heads over %d kv heads", nq, nkv);
    KESTREL_REQUIRE(slices >= 1 && slice_len > 0 && slice_len % AD_BN == 0, "attention_decode: slice length %d must be a positive multiple of %d", slice_len, AD_BN);
    KESTREL_REQUIRE(slices <= AD_MAX_CLUSTER || (part_o && part_ml), "attention_decode: %d slices without scratch", slices);
    KESTREL_REQUIRE(nkv <= 65535 && slices <= 65535, "attention_decode: grid too large");
    KESTREL_REQUIRE(cache_pages > 0 && (long long)cache_pages * nkv * page_size < (1ll << 31), "attention_decode: a cache of %d pages is beyond the 32-bit row coordinate", cache_pages);
    CUtensorMap mk, mv;
    const long long cache_rows = (long long)cache_pages * nkv * page_size;
    const int box_rows = page_size < AD_BN ? page_size : AD_BN;
    int rc = kestrel_tensor_map_bf16(&mk, k_cache, cache_rows, hd, hd, box_rows);
    if (rc) return rc;
    rc = kestrel_tensor_map_bf16(&mv, v_cache, cache_rows, hd, hd, box_rows);
    if (rc) return rc;
    AttnParams p = {};
    p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out; p.part_o = part_o; p.part_ml = part_ml; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
    p.cu_seqlens = cu_seqlens; p.kv_lens = kv_lens; p.block_table = block_table; p.table_width = table_width;
    p.table_stride = table_stride; p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.hd = hd; p.window = window;
    p.slices = slices; p.slice_len = slice_len; p.max_kv_ptr = max_kv_ptr;
    p.scale_log2 = scale * 1.4426950408889634f;
    // up to AD_MAX_CLUSTER slices are merged inside the kernel by a cluster; more go through scratch
    const bool cluster = slices > 1 && slices <= AD_MAX_CLUSTER;
    if (cluster) rc = hd == 64 ? launch_decode<64, true>(mk, mv, p, tiles, cache_pages, stream) : launch_decode<128, true>(mk, mv, p, tiles, cache_pages, stream);
    else rc = hd == 64 ? launch_decode<64, false>(mk, mv, p, tiles, cache_pages, stream) : launch_decode<128, false>(mk, mv, p, tiles, cache_pages, stream);
    if (rc || slices == 1 || cluster) return rc;
    return kestrel_attention_merge(part_o, part_ml, out, tile_seq, tile_row0, tiles, 16, cu_seqlens, slices, hd, nq, nkv, stream);
}

// Error word of the kernel's bounded waits: 0 = none, 1 = the loader waited for a free stage,
// 2 = a consumer waited for a tile.  Synchronises the device and clears the word.
// Slices that are merged without scratch and without a second kernel.
KESTREL_API int kestrel_attention_decode_cluster_slices(void) { return AD_MAX_CLUSTER; }

KESTREL_API int kestrel_attention_decode_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_ad_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_ad_error, &zero, sizeof(int));
    return v;
}
