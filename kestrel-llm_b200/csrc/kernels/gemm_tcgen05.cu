// bfloat16 matrix product on the 5th-generation tensor cores: out[t, n] = sum_k x[t, k] w[n, k].
//
// The weight matrix is the MMA's M operand: a CTA owns 128 output features (TMEM lanes) by BN
// tokens (TMEM columns), BN from 16 to 256.  So one kernel serves decode (few tokens, the
// product is a stream of weights from HBM) and prefill (many tokens, tensor-core bound), and an
// output element is accumulated in the same k order whatever the number of tokens.
//
//   warp 0   : one thread issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the
//              weight tile [128 x 64] and the activation tile [BN x 64] into a ring of stages;
//   warp 1   : allocates TMEM; one thread issues tcgen05.mma (M=128, N=BN, K=16, bf16 in,
//              float32 accumulate in TMEM) and releases stages with tcgen05.commit;
//   warps 2-5: epilogue - tcgen05.ld the accumulator (each warp its 32 lanes) and store.
//
// Epilogues: PARTIAL writes float32 [split, t, n] - the K range can be split over blockIdx.z
// so that few-token products still fill 148 SMs, and the consumer kernel sums the slices in a
// fixed order; SWIGLU runs two accumulators (gate rows n and up rows ff + n of a fused weight)
// and writes silu(gate) * up as bfloat16, so the gate/up product never reaches memory.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets an error word that the host
// reads (kestrel_gemm_tc_error) and the CTA leaves through the common exit, which frees TMEM.
// Sizes: K and the row strides must be multiples of 8 elements and the bases 16-byte aligned
// (TMA); N, T and K need not be multiples of the tile - TMA fills out-of-range rows and
// columns with zeros and stores are predicated.  Anything else is refused
// (kestrel_gemm_tc_supported) and takes the CUDA-core kernel.
#include "tcgen05.cuh"
#include <mutex>
#include <unordered_map>

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

enum { TC_PARTIAL = 0, TC_SWIGLU = 1, TC_PARTIAL2 = 2, TC_SWIGLU_T = 3, TC_QKV_PREP = 4 };     // PARTIAL2: two weight tiles a CTA, as SWIGLU, both written as float32 slices
// QKV_PREP (CTA pairs only): the q, k, v product with the tokens as the M operand and, in its
// epilogue, everything the prepare kernel does between that product and attention for head
// size 128: bias, per-head RMSNorm, rotate-half rotation, queries out, keys and values into their
// cache pages.  A tile is 256 tokens x 2 heads (one head's 128 weight rows from each rank), so a
// TMEM lane holds one token's whole head: the product's float32 plane (50 MB at 2,048 tokens of
// 8B size) is neither written nor read back, and the prepare kernel's 20 us a layer go.
// SWIGLU_T (CTA pairs only): the roles of the operands swapped - tokens are the MMA's M operand,
// the weights its N operand (128 gate rows from one rank, the 128 up rows of the same features
// from the other) - so that ONE accumulator of 256 columns holds gate and up of a (token,
// feature) in the same TMEM lane, two accumulators fit TMEM and the epilogue of a tile overlaps
// the main loop of the next, and a tile is 256 tokens x 128 features: twice as many, half as
// large, which fills the last round of tiles better.

__device__ int g_tc_error = 0;

// what the QKV_PREP epilogue needs beside the product's own arguments
struct QkvPrepParams {
    const float *bias, *q_norm_w, *k_norm_w, *inv_freq;
    float norm_eps, rot_scale;
    const int *positions, *seq_of_token, *block_table;
    int table_stride, page_size;
    __nv_bfloat16 *k_cache, *v_cache, *q_out;
    int nq, nkv, write_kv;
};

// ------------------------------------------------------------------------------- kernel
template <int BN, int MODE>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               void *__restrict__ out, int T, int N, int K, int kb_per_split, long long slice_stride,
               long long ldo, int stages, int up_row_offset, int early_w) {
    pdl_launch_dependents();
    constexpr int A_TILES = MODE == TC_PARTIAL ? 1 : 2;
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = (A_TILES * BN) < 32 ? 32 : (A_TILES * BN);
    // M = 128, N = BN, bf16 x bf16 -> f32, both operands K-major
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint32_t bars = base + (uint32_t)stages * STAGE_BYTES;          // full[stages], empty[stages], accum, tmem slot
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (stages + s); };
    uint32_t accum_bar = bars + 16u * stages;
    uint32_t tmem_slot = accum_bar + 8;
    volatile uint32_t *tmem_slot_ptr = (volatile uint32_t *)(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int n0 = blockIdx.x * TC_BM, t0 = blockIdx.y * BN;
    int total_kb = (K + TC_BK - 1) / TC_BK;
    int kb0 = blockIdx.z * kb_per_split;
    int num_kb = min(kb_per_split, total_kb - kb0);

    // Prologue, before the wait on the predecessor kernel.  Warp 0 sets up the barriers and
    // fetches the tensor maps; after the first block-wide sync its loader thread starts the
    // copies at once.  TMEM is allocated by warp 1 meanwhile and its address published to the
    // MMA and epilogue warps by a second barrier that the loader does not take part in.
    if (warp == 0) {
        if (lane < stages) { mbar_init(full_bar(lane), 1); mbar_init(empty_bar(lane), 1); }
        if (lane == 31) mbar_init(accum_bar, 1);
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t tmem = 0;
    if (warp != 0) {
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(TC_THREADS - 32) : "memory");
        tc_fence_after();
        tmem = *tmem_slot_ptr;
    }
    if (warp == 0) {
        if (lane == 0) {
            // Weights that were complete before the predecessor kernel began do not depend on it:
            // the weight tiles of the first ring of stages are on their way while it still runs,
            // and only the activation tiles wait for it.
            const int pre = early_w ? min(stages, num_kb) : 0;
            for (int kb = 0; kb < pre; ++kb) {
                mbar_expect_tx(full_bar(kb), STAGE_BYTES);
                uint32_t sa = base + (uint32_t)kb * STAGE_BYTES;
                int kc = (kb0 + kb) * TC_BK;
                tma_load_2d(sa, &map_w, full_bar(kb), kc, n0);
                if (A_TILES == 2) tma_load_2d(sa + A_BYTES, &map_w, full_bar(kb), kc, up_row_offset + n0);
            }
            pdl_wait();                               // the activations are the predecessor's output
            for (int kb = 0; kb < pre; ++kb)
                tma_load_2d(base + (uint32_t)kb * STAGE_BYTES + A_TILES * A_BYTES, &map_x, full_bar(kb), (kb0 + kb) * TC_BK, t0);
            int stage = pre == stages ? 0 : pre;
            uint32_t phase = pre == stages ? 1 : 0;
            for (int kb = pre; kb < num_kb; ++kb) {
                if (!mbar_wait(empty_bar(stage), phase ^ 1)) { atomicExch(&g_tc_error, 1); break; }
                mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                int kc = (kb0 + kb) * TC_BK;
                tma_load_2d(sa, &map_w, full_bar(stage), kc, n0);
                if (A_TILES == 2) tma_load_2d(sa + A_BYTES, &map_w, full_bar(stage), kc, up_row_offset + n0);
                tma_load_2d(sa + A_TILES * A_BYTES, &map_x, full_bar(stage), kc, t0);
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        pdl_wait();
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                if (!mbar_wait(full_bar(stage), phase)) { atomicExch(&g_tc_error, 2); ok = false; break; }
                tc_fence_after();
                uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                uint64_t da = smem_desc(sa), db = smem_desc(sa + A_TILES * A_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
                    uint32_t acc = (kb > 0 || k4 > 0) ? 1u : 0u;
                    tc_mma(tmem, da + 2 * k4, db + 2 * k4, IDESC, acc);
                    if (A_TILES == 2) tc_mma(tmem + BN, smem_desc(sa + A_BYTES) + 2 * k4, db + 2 * k4, IDESC, acc);
                }
                tc_commit(empty_bar(stage));
                if (++stage == stages) { stage = 0; phase ^= 1; }
            }
            tc_commit(accum_bar);
        }
    } else {
        pdl_wait();
        int q = warp & 3;                       // TMEM lanes 32q .. 32q+31 belong to this warp
        int n = n0 + 32 * q + lane;
        bool waited = mbar_wait(accum_bar, 0);
        if (!waited && lane == 0) atomicExch(&g_tc_error, 3);
        tc_fence_after();
        if (waited && num_kb > 0) {
            int valid = min(BN, T - t0);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (c >= valid) break;
                float g[16];
                tc_ld16(tmem + ((uint32_t)(32 * q) << 16) + c, g);
                if (MODE == TC_SWIGLU) {
                    float u[16];
                    tc_ld16(tmem + ((uint32_t)(32 * q) << 16) + BN + c, u);
                    __nv_bfloat16 *o = (__nv_bfloat16 *)out;
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c + j < valid) {
                                float a = __fdividef(g[j], 1.0f + __expf(-g[j]));     // bfloat16 output: 2-ulp float32 intrinsics
                                o[(size_t)(t0 + c + j) * ldo + n] = __float2bfloat16_rn(a * u[j]);
                            }
                    }
                } else {
                    float *o = (float *)out + (size_t)blockIdx.z * slice_stride;
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c + j < valid) o[(size_t)(t0 + c + j) * ldo + n] = g[j];
                    }
                    if (MODE == TC_PARTIAL2) {          // the second tile's rows: up_row_offset further on
                        float u[16];
                        tc_ld16(tmem + ((uint32_t)(32 * q) << 16) + BN + c, u);
                        if (n < N) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (c + j < valid) o[(size_t)(t0 + c + j) * ldo + up_row_offset + n] = u[j];
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------- persistent kernel
// Many tokens (T > 128): one CTA per SM walks over output tiles (tile = blockIdx.x + i *
// gridDim.x) and keeps TWO accumulators in TMEM (2 x 256 columns), so that the epilogue warps
// drain tile i while the MMA thread already accumulates tile i+1 and the loader runs ahead
// across tile boundaries.  PARTIAL uses tiles of 128 features x 256 tokens.  SWIGLU uses tiles
// of (128 gate + 128 up) features x 256 tokens, whose two accumulators fill TMEM (the epilogue
// then does not overlap, but operand traffic per FLOP, which bounds the kernel, is a third
// lower than with 128-token tiles and two accumulator pairs).
template <int BN, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          void *__restrict__ out, int T, int N, int K, long long ldo, int stages, int up_row_offset,
                          int tiles_n, int tiles_total) {
    pdl_launch_dependents();
    constexpr int A_TILES = MODE == TC_SWIGLU ? 2 : 1;
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = BN * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
    constexpr uint32_t ACC_COLS = A_TILES * BN;
    static_assert(ACC_COLS == 256 || ACC_COLS == 512, "accumulators of 256 or 512 columns");
    constexpr uint32_t TMEM_COLS = 512;
    constexpr int NBUF = TMEM_COLS / ACC_COLS;          // 2: the epilogue overlaps the next tile; 1: it does not
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint32_t bars = base + (uint32_t)stages * STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (stages + s); };
    auto acc_full = [&](int b) { return bars + 16u * stages + 8u * b; };
    auto acc_empty = [&](int b) { return bars + 16u * stages + 16u + 8u * b; };
    uint32_t tmem_slot = bars + 16u * stages + 32u;
    volatile uint32_t *tmem_slot_ptr = (volatile uint32_t *)(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int num_kb = (K + TC_BK - 1) / TC_BK;

    if (warp == 0) {
        if (lane < stages) { mbar_init(full_bar(lane), 1); mbar_init(empty_bar(lane), 1); }
        if (lane >= 28 && lane < 30) mbar_init(acc_full(lane - 28), 1);
        if (lane >= 30) mbar_init(acc_empty(lane - 30), 4);              // one arrival per epilogue warp
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t tmem = 0;
    if (warp != 0) {
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        tc_fence_before();
        asm volatile("bar.sync 1, %0;" ::"n"(TC_THREADS - 32) : "memory");
        tc_fence_after();
        tmem = *tmem_slot_ptr;
    }
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles_total && ok; tile += gridDim.x) {
                int n0 = (tile % tiles_n) * TC_BM, t0 = (tile / tiles_n) * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1)) { atomicExch(&g_tc_error, 1); ok = false; break; }
                    mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                    uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                    int kc = kb * TC_BK;
                    tma_load_2d(sa, &map_w, full_bar(stage), kc, n0);
                    if (MODE == TC_SWIGLU) tma_load_2d(sa + A_BYTES, &map_w, full_bar(stage), kc, up_row_offset + n0);
                    tma_load_2d(sa + A_TILES * A_BYTES, &map_x, full_bar(stage), kc, t0);
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int j = 0;
            for (int tile = blockIdx.x; tile < tiles_total && ok; tile += gridDim.x, ++j) {
                int b = j % NBUF;
                uint32_t acc_phase = (uint32_t)(j / NBUF) & 1u;
                if (!mbar_wait(acc_empty(b), acc_phase ^ 1)) { atomicExch(&g_tc_error, 4); ok = false; break; }
                tc_fence_after();
                uint32_t d = tmem + (uint32_t)b * ACC_COLS;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase)) { atomicExch(&g_tc_error, 2); ok = false; break; }
                    tc_fence_after();
                    uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                    uint64_t da = smem_desc(sa), db = smem_desc(sa + A_TILES * A_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
                        uint32_t acc = (kb > 0 || k4 > 0) ? 1u : 0u;
                        tc_mma(d, da + 2 * k4, db + 2 * k4, IDESC, acc);
                        if (MODE == TC_SWIGLU) tc_mma(d + BN, smem_desc(sa + A_BYTES) + 2 * k4, db + 2 * k4, IDESC, acc);
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                tc_commit(acc_full(b));
            }
        }
    } else {
        int q = warp & 3;
        int j = 0;
        for (int tile = blockIdx.x; tile < tiles_total; tile += gridDim.x, ++j) {
            int b = j % NBUF;
            uint32_t acc_phase = (uint32_t)(j / NBUF) & 1u;
            int n0 = (tile % tiles_n) * TC_BM, t0 = (tile / tiles_n) * BN;
            int n = n0 + 32 * q + lane;
            if (!mbar_wait(acc_full(b), acc_phase)) { if (lane == 0) atomicExch(&g_tc_error, 3); break; }
            tc_fence_after();
            uint32_t d = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)b * ACC_COLS;
            int valid = min(BN, T - t0);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (c >= valid) break;
                float g[16];
                tc_ld16(d + c, g);
                if (MODE == TC_SWIGLU) {
                    float u[16];
                    tc_ld16(d + BN + c, u);
                    __nv_bfloat16 *o = (__nv_bfloat16 *)out;
                    if (n < N) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj)
                            if (c + jj < valid) {
                                float a = __fdividef(g[jj], 1.0f + __expf(-g[jj]));   // bfloat16 output: 2-ulp float32 intrinsics
                                o[(size_t)(t0 + c + jj) * ldo + n] = __float2bfloat16_rn(a * u[jj]);
                            }
                    }
                } else {
                    float *o = (float *)out;
                    if (n < N) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj)
                            if (c + jj < valid) o[(size_t)(t0 + c + jj) * ldo + n] = g[jj];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(b));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------ CTA-pair kernel
// Many tokens, PARTIAL epilogue: two CTAs of a cluster share one tcgen05.mma (cta_group::2,
// M = 256, N = 256).  Each CTA loads its own 128 weight rows and HALF of the 256 token rows of
// a k-block (32 KB a stage instead of 48), the tensor cores of both SMs read the token rows
// from both CTAs' shared memory, and each CTA ends up with its 128 features x 256 tokens in its
// own TMEM.  Operand traffic per SM - which bounds the one-CTA kernel - drops by a third.
//   * rank 0 ("leader") issues the MMAs; both ranks load; TMA completions of both ranks count
//     on the leader's full barrier (cp.async.bulk.tensor ... cta_group::2);
//   * the leader frees a stage in both CTAs, and publishes an accumulator to both, with
//     tcgen05.commit ... multicast::cluster (a commit, not a load: no operand is multicast);
//   * the epilogue warps of both ranks arrive on the leader's accumulator-empty barrier.
// No TMA load uses cluster multicast.  Persistent over tiles as the one-CTA kernel, two
// accumulators in TMEM.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t leader_bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {       // arrives on `bar` of both CTAs
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

#define TCP_BN 256          // tokens of a pair's tile (128 loaded by each rank)
#ifndef TCP_EPI_GROUPS
#define TCP_EPI_GROUPS 4    // epilogue warps per TMEM lane quarter; each takes 256 / TCP_EPI_GROUPS token columns
#endif
#define TCP_THREADS (64 + 128 * TCP_EPI_GROUPS)     // loader, MMA issuer, 4 x TCP_EPI_GROUPS epilogue warps

// MODE PARTIAL: float32 [T, N], two accumulators (the epilogue overlaps the next tile).  The K
//               range may be cut into slices (tile index = slice * tiles_nt + output tile), each
//               written to its own float32 plane slice_stride elements apart: a few hundred
//               tokens give fewer output tiles than there are CTA pairs.
// MODE SWIGLU : gate rows n and up rows up_row_offset + n, two accumulators that fill TMEM (no
//               overlap), bfloat16 silu(gate) * up out; 48 KB a stage for twice the MMAs.
// The epilogue is spread over 16 warps a CTA (four per TMEM lane quarter, 64 token columns
// each): where it does not overlap the next tile it is on the critical path, and four warps
// alone, one per scheduler, run it at the pace of their own dependent instructions.
template <int MODE>
__global__ void __launch_bounds__(TCP_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    void *__restrict__ out, int T, int N, int K, long long ldo, int stages, int tiles_n, int tiles_total,
                    int up_row_offset, int accumulate, int tiles_nt, int kb_per_split, long long slice_stride,
                    const QkvPrepParams prep) {
    pdl_launch_dependents();
    constexpr bool SWAP = MODE == TC_SWIGLU_T || MODE == TC_QKV_PREP;      // tokens are the M operand
    constexpr int A_TILES = MODE == TC_SWIGLU ? 2 : 1;
    constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
    constexpr uint32_t B_BYTES = (TCP_BN / 2) * TC_BK * 2;
    constexpr uint32_t STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;     // per CTA; a stage of the pair is twice that
    constexpr uint32_t ACC_COLS = A_TILES * TCP_BN, TMEM_COLS = 512;
    constexpr int NBUF = TMEM_COLS / ACC_COLS;
    // M = 256 (two CTAs), N = 256, bf16 x bf16 -> f32, both operands K-major
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TCP_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint32_t bars = base + (uint32_t)stages * STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (stages + s); };
    auto acc_full = [&](int b) { return bars + 16u * stages + 8u * b; };
    auto acc_empty = [&](int b) { return bars + 16u * stages + 16u + 8u * b; };
    uint32_t tmem_slot = bars + 16u * stages + 32u;
    volatile uint32_t *tmem_slot_ptr = (volatile uint32_t *)(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int num_kb = (K + TC_BK - 1) / TC_BK;
    // Output tile w of a slice: the token tiles of one feature tile follow each other, so the pairs
    // that work at the same time share weight rows, which are then fetched from HBM once and found
    // in L2 by the others (with the feature tile running fastest a round of 74 pairs touched 74
    // weight tiles, more than L2 holds, and every token tile fetched the weights anew: 1.08 GB read
    // for the 201 MB of a gate/up matrix at 2,048 tokens).  The activations of a step fit L2.
    const int tiles_t = tiles_nt / tiles_n;
    auto tile_n = [&](int w) { return w / tiles_t; };
    auto tile_t = [&](int w) { return w % tiles_t; };

    if (warp == 0) {
        if (lane < stages) { mbar_init(full_bar(lane), 1); mbar_init(empty_bar(lane), 1); }
        if (lane >= 28 && lane < 30) mbar_init(acc_full(lane - 28), 1);
        if (lane >= 30) mbar_init(acc_empty(lane - 30), 8 * TCP_EPI_GROUPS);    // the epilogue warps of both ranks
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {                                                     // the same warp of both ranks
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync();                   // both ranks' barriers exist before anything arrives on them from afar
    tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles_total && ok; tile += n_pairs) {
                const int split = tile / tiles_nt, tw = tile % tiles_nt;       // a tile of the output and its slice of K
                int n0 = tile_n(tw) * 256 + (int)rank * TC_BM;
                int t0 = tile_t(tw) * TCP_BN + (int)rank * (TCP_BN / 2);
                if (MODE == TC_SWIGLU_T) n0 = tile_n(tw) * TC_BM + (rank ? up_row_offset : 0);     // this rank's half of the N operand: gate rows, or up rows
                if (MODE == TC_QKV_PREP) n0 = (2 * tile_n(tw) + (int)rank) * TC_BM;                  // one head's rows from each rank
                const int kb_end = min(num_kb, (split + 1) * kb_per_split);
                for (int kb = split * kb_per_split; kb < kb_end; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1)) { atomicExch(&g_tc_error, 1); ok = false; break; }
                    uint32_t leader_full = map_to_rank(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
                    uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                    int kc = kb * TC_BK;
                    if (SWAP) {              // tokens are the M operand (this rank's 128), weights the N operand (this rank's half)
                        tma_load_2d_pair(sa, &map_x, leader_full, kc, t0);
                        tma_load_2d_pair(sa + A_BYTES, &map_w, leader_full, kc, n0);
                    } else {
                        tma_load_2d_pair(sa, &map_w, leader_full, kc, n0);
                        if (MODE == TC_SWIGLU) tma_load_2d_pair(sa + A_BYTES, &map_w, leader_full, kc, up_row_offset + n0);
                        tma_load_2d_pair(sa + A_TILES * A_BYTES, &map_x, leader_full, kc, t0);
                    }
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int j = 0;
            for (int tile = pair; tile < tiles_total && ok; tile += n_pairs, ++j) {
                int b = j % NBUF;
                uint32_t acc_phase = (uint32_t)(j / NBUF) & 1u;
                if (!mbar_wait(acc_empty(b), acc_phase ^ 1)) { atomicExch(&g_tc_error, 4); ok = false; break; }
                tc_fence_after();
                uint32_t d = tmem + (uint32_t)b * ACC_COLS;
                const int split = tile / tiles_nt;
                const int kb_begin = split * kb_per_split, kb_end = min(num_kb, (split + 1) * kb_per_split);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase)) { atomicExch(&g_tc_error, 2); ok = false; break; }
                    tc_fence_after();
                    uint32_t sa = base + (uint32_t)stage * STAGE_BYTES;
                    uint64_t da = smem_desc(sa), db = smem_desc(sa + A_TILES * A_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
                        uint32_t acc = (kb > kb_begin || k4 > 0) ? 1u : 0u;
                        tc_mma_pair(d, da + 2 * k4, db + 2 * k4, IDESC, acc);
                        if (MODE == TC_SWIGLU) tc_mma_pair(d + TCP_BN, smem_desc(sa + A_BYTES) + 2 * k4, db + 2 * k4, IDESC, acc);
                    }
                    tc_commit_pair(empty_bar(stage));
                    if (++stage == stages) { stage = 0; phase ^= 1; }
                }
                tc_commit_pair(acc_full(b));
            }
        }
    } else {
        int q = warp & 3;
        int j = 0;
        for (int tile = pair; tile < tiles_total; tile += n_pairs, ++j) {
            int b = j % NBUF;
            uint32_t acc_phase = (uint32_t)(j / NBUF) & 1u;
            const int split = tile / tiles_nt, tw = tile % tiles_nt;
            int n = tile_n(tw) * 256 + (int)rank * TC_BM + 32 * q + lane;
            int t0 = tile_t(tw) * TCP_BN;
            if (!mbar_wait(acc_full(b), acc_phase)) { if (lane == 0) atomicExch(&g_tc_error, 3); break; }
            tc_fence_after();
            uint32_t d = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)b * ACC_COLS;
            if (MODE == TC_QKV_PREP) {
                // lane = token, columns 0..127 = head 2 fn, 128..255 = head 2 fn + 1.  The four warps that
                // share a lane quarter each take sixteen rotation pairs (dimensions 16 g.. and 64 + 16 g..)
                // of both heads; they exchange their parts of the sums of squares through shared memory.
                __shared__ float ss_x[2][2][4][128];                     // [tile parity][head of the tile][group][token]
                const int grp = (warp - 2) >> 2, tl = 32 * q + lane;
                const int t = t0 + (int)rank * (TCP_BN / 2) + tl;
                const bool t_ok = t < T;
                const int heads = prep.nq + 2 * prep.nkv, head0 = 2 * tile_n(tw);
                const int pos = t_ok ? prep.positions[t] : 0;
                int page = 0;
                if (t_ok && prep.write_kv) page = prep.block_table[(size_t)prep.seq_of_token[t] * prep.table_stride + pos / prep.page_size];
                float cs[16], sn[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    sincosf((float)pos * prep.inv_freq[16 * grp + c], &sn[c], &cs[c]);
                    cs[c] *= prep.rot_scale;
                    sn[c] *= prep.rot_scale;
                }
                float (*ssb)[4][128] = ss_x[j & 1];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int head = head0 + hh;
                    float lo[16], hi[16];
                    tc_ld16(d + hh * TC_BM + 16 * grp, lo);
                    tc_ld16(d + hh * TC_BM + 64 + 16 * grp, hi);
                    float ss = 0.f;
                    if (head < heads) {
                        const float *b = prep.bias ? prep.bias + (size_t)head * TC_BM : nullptr;
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            if (b) { lo[c] += b[16 * grp + c]; hi[c] += b[64 + 16 * grp + c]; }
                            ss += lo[c] * lo[c] + hi[c] * hi[c];
                        }
                    }
                    ssb[hh][grp][tl] = ss;
                }
                asm volatile("bar.sync %0, 128;" ::"r"(1 + q) : "memory");       // the four warps of this lane quarter
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int head = head0 + hh;
                    if (head >= heads) continue;
                    const bool is_q = head < prep.nq, is_k = !is_q && head < prep.nq + prep.nkv;
                    if (!is_q && !prep.write_kv) continue;
                    float lo[16], hi[16];
                    tc_ld16(d + hh * TC_BM + 16 * grp, lo);
                    tc_ld16(d + hh * TC_BM + 64 + 16 * grp, hi);
                    if (prep.bias) {
                        const float *b = prep.bias + (size_t)head * TC_BM;
#pragma unroll
                        for (int c = 0; c < 16; ++c) { lo[c] += b[16 * grp + c]; hi[c] += b[64 + 16 * grp + c]; }
                    }
                    const float *nw = is_q ? prep.q_norm_w : (is_k ? prep.k_norm_w : nullptr);
                    if (nw) {
                        const float tot = ((ssb[hh][0][tl] + ssb[hh][1][tl]) + ssb[hh][2][tl]) + ssb[hh][3][tl];
                        const float rinv = 1.0f / sqrtf(tot / (float)TC_BM + prep.norm_eps);
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            lo[c] = (lo[c] * rinv) * nw[16 * grp + c];
                            hi[c] = (hi[c] * rinv) * nw[64 + 16 * grp + c];
                        }
                    }
                    if (is_q || is_k) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const float a = lo[c], b2 = hi[c];
                            lo[c] = a * cs[c] - b2 * sn[c];
                            hi[c] = b2 * cs[c] + a * sn[c];
                        }
                    }
                    if (t_ok) {
                        __nv_bfloat16 *o;
                        if (is_q) {
                            o = prep.q_out + ((size_t)t * prep.nq + head) * TC_BM;
                        } else {
                            const int kvh = is_k ? head - prep.nq : head - prep.nq - prep.nkv;
                            o = (is_k ? prep.k_cache : prep.v_cache) + (((size_t)page * prep.nkv + kvh) * prep.page_size + pos % prep.page_size) * TC_BM;
                        }
                        uint32_t pl[8], ph[8];
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            __nv_bfloat162 a = __floats2bfloat162_rn(lo[2 * c], lo[2 * c + 1]), b2 = __floats2bfloat162_rn(hi[2 * c], hi[2 * c + 1]);
                            pl[c] = *reinterpret_cast<uint32_t *>(&a);
                            ph[c] = *reinterpret_cast<uint32_t *>(&b2);
                        }
                        uint4 *dl = reinterpret_cast<uint4 *>(o + 16 * grp), *dh = reinterpret_cast<uint4 *>(o + 64 + 16 * grp);
                        dl[0] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
                        dl[1] = make_uint4(pl[4], pl[5], pl[6], pl[7]);
                        dh[0] = make_uint4(ph[0], ph[1], ph[2], ph[3]);
                        dh[1] = make_uint4(ph[4], ph[5], ph[6], ph[7]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty(b), 0));
                continue;
            }
            if (SWAP) {
                // lane = token, columns 0..127 = gate of 128 features, 128..255 = up of the same features;
                // each group of four warps takes a quarter of the features
                const int t = t0 + (int)rank * (TCP_BN / 2) + 32 * q + lane;
                const int f0 = tile_n(tw) * TC_BM;
                const int cf = ((warp - 2) >> 2) * (TC_BM / TCP_EPI_GROUPS);
                __nv_bfloat16 *o = (__nv_bfloat16 *)out + (size_t)t * ldo + f0;
#pragma unroll 1
                for (int c = cf; c < cf + TC_BM / TCP_EPI_GROUPS; c += 16) {
                    if (f0 + c >= N) break;
                    float g[16], u[16];
                    tc_ld16(d + c, g);
                    tc_ld16(d + TC_BM + c, u);
                    if (t < T) {
                        if (f0 + c + 16 <= N && (ldo & 7) == 0) {          // 16 features of one token: two 16-byte stores
                            uint32_t pk[8];
#pragma unroll
                            for (int jj = 0; jj < 8; ++jj) {
                                float a0 = __fdividef(g[2 * jj], 1.0f + __expf(-g[2 * jj])) * u[2 * jj];
                                float a1 = __fdividef(g[2 * jj + 1], 1.0f + __expf(-g[2 * jj + 1])) * u[2 * jj + 1];
                                __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1);
                                pk[jj] = *reinterpret_cast<uint32_t *>(&h);
                            }
                            uint4 *dst = reinterpret_cast<uint4 *>(o + c);
                            dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                        } else {
#pragma unroll
                            for (int jj = 0; jj < 16; ++jj)
                                if (f0 + c + jj < N) {
                                    float a = __fdividef(g[jj], 1.0f + __expf(-g[jj]));
                                    o[c + jj] = __float2bfloat16_rn(a * u[jj]);
                                }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty(b), 0));
                continue;
            }
            int valid = min(TCP_BN, T - t0);
            const int c_begin = ((warp - 2) >> 2) * (TCP_BN / TCP_EPI_GROUPS);      // each group of four warps its columns
#pragma unroll 1
            for (int c = c_begin; c < c_begin + TCP_BN / TCP_EPI_GROUPS; c += 16) {
                if (c >= valid) break;
                float g[16];
                tc_ld16(d + c, g);
                if (MODE == TC_SWIGLU) {
                    float u[16];
                    tc_ld16(d + TCP_BN + c, u);
                    __nv_bfloat16 *o = (__nv_bfloat16 *)out;
                    if (n < N) {
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj)
                            if (c + jj < valid) {
                                float a = __fdividef(g[jj], 1.0f + __expf(-g[jj]));
                                o[(size_t)(t0 + c + jj) * ldo + n] = __float2bfloat16_rn(a * u[jj]);
                            }
                    }
                } else if (n < N) {
                    float *o = (float *)out + (size_t)split * slice_stride;
                    if (accumulate) {           // out is the residual stream: the product is added to it in place
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj)
                            if (c + jj < valid) g[jj] += o[(size_t)(t0 + c + jj) * ldo + n];
                    }
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj)
                        if (c + jj < valid) o[(size_t)(t0 + c + jj) * ldo + n] = g[jj];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty(b), 0));
        }
    }
    tc_fence_before();
    cluster_sync();                   // nobody leaves while the other rank may still signal or read it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct MapKey {
    const void *ptr; long long rows, cols, ld; int box_rows;
    bool operator==(const MapKey &o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows; h = h * 1000003u ^ (size_t)k.cols;
        h = h * 1000003u ^ (size_t)k.ld;   h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// bf16 matrix [rows, cols] with row stride ld elements; box = box_rows x 64 columns, 128-byte swizzle
int kestrel_tensor_map_bf16(CUtensorMap *out, const void *ptr, long long rows, long long cols, long long ld, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, ld, box_rows};
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return 0; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return kestrel_fail(-4, "tensor map: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return kestrel_fail(-4, "tensor map: cuTensorMapEncodeTiled failed with %d (rows %lld cols %lld ld %lld)", (int)r, rows, cols, ld);
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}

KESTREL_API int kestrel_gemm_tc_supported(const void *x, const void *w, int T, int N, int K, long long ldx, long long ldw) {
    if (T <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8 || ldx % 8 || ldw % 8) return 0;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return 0;
    return 1;
}

// Tuning of few-token products (T <= 128), which stream the weights once and are bound by HBM:
// g_ctas_per_sm CTAs share an SM's shared memory for their stages; a CTA costs about
// g_overhead_kb k-blocks of time beyond its own k-blocks (launch, barrier set-up, TMEM
// allocation, first tensor-map fetch, pipeline fill, epilogue).
static int g_qkv_fused = 1;        // the q, k, v product of many tokens does the prepare kernel's work in its epilogue
static int g_swiglu_swapped = 1;   // the SwiGLU product on CTA pairs with tokens as the M operand (TC_SWIGLU_T)
static int g_swiglu_bn = 256;      // token tile of the persistent SwiGLU product: 256 (one accumulator pair) or 128 (two)
static int g_pairs = 1;            // many-token PARTIAL products on CTA pairs (cta_group::2)
static int g_persistent = 1;       // many-token products on the persistent kernel (0: one tile per CTA)
static int g_pair_min_tokens = 128; // products of more tokens run on CTA pairs (measured: from 129 tokens on they win)
static int g_pair_overhead_kb = 12;
static int g_overhead_kb = 6;
static int g_ctas_per_sm = 2;

KESTREL_API void kestrel_gemm_tc_set_persistent(int on) { g_persistent = on ? 1 : 0; }
KESTREL_API void kestrel_gemm_tc_set_pairs(int on) { g_pairs = on ? 1 : 0; }
KESTREL_API void kestrel_gemm_tc_set_swiglu_tile(int bn) { if (bn == 128 || bn == 256) g_swiglu_bn = bn; }
KESTREL_API void kestrel_gemm_tc_set_swiglu_swapped(int mode) { if (mode >= 0 && mode <= 2) g_swiglu_swapped = mode; }

KESTREL_API void kestrel_gemm_tc_set_pair_tuning(int min_tokens, int overhead_kb) {
    if (min_tokens >= 0) g_pair_min_tokens = min_tokens;
    if (overhead_kb >= 0) g_pair_overhead_kb = overhead_kb;
}

KESTREL_API void kestrel_gemm_tc_set_tuning(int overhead_kb, int ctas_per_sm) {
    if (overhead_kb >= 0) g_overhead_kb = overhead_kb;
    if (ctas_per_sm >= 1 && ctas_per_sm <= 4) g_ctas_per_sm = ctas_per_sm;
}

// Slices into which a product of T tokens and N output features splits its K range: the
// number that minimises waves x (overhead + k-blocks per slice) over the GPU's SMs.
// Many-token products are not split.
// 33 to 128 tokens: the token tile is half as large as the weight tile or as large, so a third to
// a half of what an SM takes in is the same activations for every CTA.  A CTA then takes two
// weight tiles (rows n and N / 2 + n) against one token tile, as the SwiGLU product does: a
// sixth to a quarter fewer bytes in (measured at 128 tokens: QKV 15.3 -> 12.5 us, attention
// output 13.2 -> 10.2, down projection 24.8 -> 22.7; at 64 tokens 11.8 -> 10.7, 9.7 -> 8.4, 20.9 -> 20.2).
static int g_wide = 1, g_wide_min = 32;
KESTREL_API void kestrel_gemm_tc_set_wide(int on, int more_than_tokens) { g_wide = on ? 1 : 0; if (more_than_tokens >= 0) g_wide_min = more_than_tokens; }
static bool tc_wide(int T, int N) { return g_wide && T > g_wide_min && T <= 128 && T <= g_pair_min_tokens && N % (2 * TC_BM) == 0; }

// Cost of a many-token product on CTA pairs cut into s slices along K, in k-blocks of one
// pair's time (about 0.42 us at these sizes); -1 where s does not divide the k-blocks into slices
// of at least sixteen.  A slice costs about g_pair_overhead_kb k-blocks beyond its own (pipeline
// fill, the last tile's epilogue); the slices' float32 planes cost their write and their read
// by the consumer as far as they no longer fit L2 (measured at 3,072 tokens: the down product in
// three slices 227 + 89 us with its norm, whole 251 + 47).
static long long pair_cost(int T, int N, int K, int s, long long *waves_out = nullptr) {
    const long long tiles = (long long)((N + 255) / 256) * ((T + TCP_BN - 1) / TCP_BN);
    const int total_kb = (K + TC_BK - 1) / TC_BK;
    const int pairs = kestrel_sms() / 2;
    const int per = (total_kb + s - 1) / s;
    if (s > 1 && (per < 16 || (total_kb + per - 1) / per != s)) return -1;
    const long long waves = (tiles * s + pairs - 1) / pairs;
    if (waves_out) *waves_out = waves;
    long long planes = 8ll * T * N * (s - 1) - (64ll << 20);
    if (planes < 0) planes = 0;
    return waves * (g_pair_overhead_kb + per) + planes / 2100000;
}

KESTREL_API int kestrel_gemm_tc_splits(int T, int N, int K) {
    if (T > g_pair_min_tokens) {
        // many tokens on CTA pairs: tiles of 256 x 256 over the pairs of SMs; K is cut only where
        // that fills idle pairs
        if (!g_pairs || !g_persistent) return 1;
        int best = 1;
        long long best_cost = -1;
        for (int s = 1; s <= 8; ++s) {
            long long cost = pair_cost(T, N, K, s);
            if (cost < 0) continue;
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
        }
        return best;
    }
    int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
    const bool wide = tc_wide(T, N);
    long long tiles = (long long)((N + TC_BM - 1) / TC_BM) * ((T + bn - 1) / bn) / (wide ? 2 : 1);
    int total_kb = (K + TC_BK - 1) / TC_BK;
    int slots = kestrel_sms() * (bn <= 64 && !wide ? g_ctas_per_sm : 1);          // wider token tiles take an SM's shared memory alone
    int best = 1;
    long long best_cost = -1;
    int max_s = total_kb / 4 > 0 ? total_kb / 4 : 1;          // at least 4 k-blocks (256 columns) a slice
    if (max_s > 16) max_s = 16;
    for (int s = 1; s <= max_s; ++s) {
        int per = (total_kb + s - 1) / s;
        int real = (total_kb + per - 1) / per;                  // no empty slice
        if (real != s) continue;
        long long waves = (tiles * s + slots - 1) / slots;
        // a CTA also writes its float32 slice [bn, 128] and the consumer reads it back: bn / 16
        // k-blocks' worth of bytes (a k-block of weights is 16 KB)
        long long cost = waves * (g_overhead_kb + (wide ? 2 : 1) * (bn / 16) + per) * (bn <= 64 && !wide ? g_ctas_per_sm : 1);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

// What `linear` asks before a product, in one call: 0 if the operands do not fit the TMA rules,
// else the number of K slices the product should be cut into.
KESTREL_API int kestrel_gemm_tc_plan(const void *x, const void *w, int T, int N, int K, long long ldx, long long ldw) {
    if (!kestrel_gemm_tc_supported(x, w, T, N, K, ldx, ldw)) return 0;
    return kestrel_gemm_tc_splits(T, N, K);
}

template <int BN, int MODE>
static int launch_tc(const CUtensorMap &mw, const CUtensorMap &mx, void *out, int T, int N, int K, int splits,
                     long long slice_stride, long long ldo, int up_off, int early_w, cudaStream_t stream) {
    constexpr int A_TILES = MODE == TC_PARTIAL ? 1 : 2;
    constexpr int STAGE_BYTES = A_TILES * TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    int total_kb = (K + TC_BK - 1) / TC_BK;
    int per = (total_kb + splits - 1) / splits;
    // few tokens: the CTAs that share an SM divide its shared memory; else one CTA takes it all
    int budget = (BN <= 64 && MODE == TC_PARTIAL) ? (216 * 1024) / g_ctas_per_sm - 2048 : 200 * 1024;
    int stages = budget / STAGE_BYTES;
    if (stages > per) stages = per < 2 ? 2 : per;
    if (stages > 12) stages = 12;
    if (stages < 2) stages = 2;
    size_t smem = (size_t)stages * STAGE_BYTES + 16 * stages + 16 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return kestrel_fail(-3, "gemm_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid((N + TC_BM - 1) / TC_BM, (T + BN - 1) / BN, splits);
    if (grid.y > 65535) return kestrel_fail(-2, "gemm_tc: T=%d needs more than 65535 token tiles", T);
    kestrel_launch(gemm_tc_kernel<BN, MODE>, dim3(grid), dim3(TC_THREADS), smem, stream, mw, mx, out, T, N, K, per, slice_stride, ldo, stages, up_off, early_w);
    return kestrel_check_launch("gemm_tc");
}

template <int BN, int MODE>
static int launch_tc_persistent(const CUtensorMap &mw, const CUtensorMap &mx, void *out, int T, int N, int K,
                                long long ldo, int up_off, cudaStream_t stream) {
    constexpr int A_TILES = MODE == TC_SWIGLU ? 2 : 1;
    constexpr int STAGE_BYTES = A_TILES * TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    int stages = (200 * 1024) / STAGE_BYTES;
    if (stages > 8) stages = 8;
    size_t smem = (size_t)stages * STAGE_BYTES + 16 * stages + 48 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return kestrel_fail(-3, "gemm_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    int tiles_n = (N + TC_BM - 1) / TC_BM, tiles_t = (T + BN - 1) / BN;
    long long total = (long long)tiles_n * tiles_t;
    if (total > 0x7fffffff) return kestrel_fail(-2, "gemm_tc: too many tiles");
    const int sms = kestrel_sms();
    int grid = total < sms ? (int)total : sms;
    kestrel_launch(gemm_tc_persistent_kernel<BN, MODE>, dim3(grid), dim3(TC_THREADS), smem, stream, mw, mx, out, T, N, K, ldo,
                   stages, up_off, tiles_n, (int)total);
    return kestrel_check_launch("gemm_tc_persistent");
}

template <int MODE>
static int launch_tc_pair(const CUtensorMap &mw, const CUtensorMap &mx, void *out, int T, int N, int K, long long ldo,
                          int up_off, int accumulate, int splits, long long slice_stride, cudaStream_t stream,
                          const QkvPrepParams &prep = QkvPrepParams()) {
    const int STAGE_BYTES = (MODE == TC_SWIGLU ? 2 : 1) * TC_BM * TC_BK * 2 + (TCP_BN / 2) * TC_BK * 2;
    int stages = (200 * 1024) / STAGE_BYTES;
    if (stages > 8) stages = 8;
    size_t smem = (size_t)stages * STAGE_BYTES + 16 * stages + 48 + 1024;
    static int max_clusters = -1;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(TCP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (max_clusters < 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return kestrel_fail(-3, "gemm_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        cfg.gridDim = dim3(kestrel_sms());
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<MODE>, &cfg);
        if (e != cudaSuccess || n < 1) {
            cudaGetLastError();
            max_clusters = 0;              // pairs cannot be scheduled here: the one-CTA kernel is used
        } else {
            max_clusters = n;
        }
    }
    if (max_clusters == 0) return 1;       // not an error: tells the caller to fall back
    // output tiles: 256 features x 256 tokens; with the operands swapped 128 features x 256 tokens
    // (QKV_PREP: 256 features = two heads of 128 x 256 tokens, N = all heads' rows)
    int tiles_n = MODE == TC_SWIGLU_T ? (N + TC_BM - 1) / TC_BM : (N + 255) / 256, tiles_t = (T + TCP_BN - 1) / TCP_BN;
    long long tiles_nt = (long long)tiles_n * tiles_t, total = tiles_nt * splits;
    if (total > 0x7fffffff) return kestrel_fail(-2, "gemm_tc: too many tiles");
    if (splits > 1 && (MODE != TC_PARTIAL || accumulate)) return kestrel_fail(-2, "gemm_tc_pair: only plain float32 slices can be cut along K");
    int total_kb = (K + TC_BK - 1) / TC_BK;
    int per = (total_kb + splits - 1) / splits;
    int pairs = total < max_clusters ? (int)total : max_clusters;
    cfg.gridDim = dim3(2 * pairs);
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<MODE>, mw, mx, out, T, N, K, ldo, stages, tiles_n, (int)total, up_off, accumulate,
                                       (int)tiles_nt, per, slice_stride, prep);
    if (e != cudaSuccess) return kestrel_fail(-3, "gemm_tc_pair: %s", cudaGetErrorString(e));
    return kestrel_check_launch("gemm_tc_pair");
}

// Which form the SwiGLU product takes on CTA pairs.  With the weights as the M operand a tile is
// 256 features x 256 tokens (gate and up: four units of work) and its epilogue is not overlapped;
// with the tokens as the M operand a tile is 128 features x 256 tokens (two units), the epilogue
// overlaps the next tile and the finer tiles fill the last round better: measured at 8B sizes
// 512 tokens 95.5 -> 78.8 us, 2,048 tokens 294 -> 268 us (1.54 PFLOP/s), 4,096 tokens 551 -> 504 us;
// at 32B sizes 256 tokens 153 -> 111 us.  It fetches a third more operand bytes per multiply-add,
// so where both forms need the same rounds of work for ONE token tile (8B sizes up to 256 tokens:
// 48 tiles in one round against 96 in two) the first form stays ahead, 51.6 against 55.0 us.
// g_swiglu_swapped: 0 never, 1 by this rule, 2 always.
static bool swiglu_swapped_wins(int T, int ff) {
    if (g_swiglu_swapped != 1) return g_swiglu_swapped == 2;
    const long long pairs = kestrel_sms() / 2, tt = (T + TCP_BN - 1) / TCP_BN;
    const long long work_m = 4 * ((((ff + 255) / 256) * tt + pairs - 1) / pairs);       // weights as M: rounds of four units
    const long long work_t = 2 * ((((ff + 127) / 128) * tt + pairs - 1) / pairs);       // tokens as M: rounds of two
    return work_t < work_m || (work_t == work_m && tt > 1);
}

template <int MODE>
static int dispatch_tc(const void *x, const void *w, void *out, int T, int N, int w_rows, int K, long long ldx, long long ldw,
                       long long ldo, int splits, long long slice_stride, int up_off, int early_w, cudaStream_t stream) {
    int bn = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
    bool persistent = T > g_pair_min_tokens && g_persistent && (splits == 1 || (g_pairs && MODE == TC_PARTIAL));
    if (persistent && MODE == TC_SWIGLU) bn = g_swiglu_bn;
    CUtensorMap mw, mx;
    int rc = kestrel_tensor_map_bf16(&mw, w, w_rows, K, ldw, TC_BM);
    if (rc) return rc;
    if (persistent && g_pairs) {
        rc = kestrel_tensor_map_bf16(&mx, x, T, K, ldx, TCP_BN / 2);
        if (rc) return rc;
        if (MODE == TC_SWIGLU && swiglu_swapped_wins(T, N) && ((uintptr_t)out & 15) == 0 && ldo % 8 == 0)
            rc = launch_tc_pair<TC_SWIGLU_T>(mw, mx, out, T, N, K, ldo, up_off, 0, 1, 0, stream);
        else
            rc = launch_tc_pair<MODE>(mw, mx, out, T, N, K, ldo, up_off, 0, splits, slice_stride, stream);
        if (rc <= 0) return rc;            // 1 = pairs cannot be scheduled: go on with one CTA per tile
    }
    if (splits > 1) persistent = false;    // the one-CTA persistent kernel does not cut K
    rc = kestrel_tensor_map_bf16(&mx, x, T, K, ldx, bn);
    if (rc) return rc;
    if (persistent) {
        if (MODE == TC_SWIGLU && bn == 128) return launch_tc_persistent<128, TC_SWIGLU>(mw, mx, out, T, N, K, ldo, up_off, stream);
        if (MODE == TC_SWIGLU) return launch_tc_persistent<256, TC_SWIGLU>(mw, mx, out, T, N, K, ldo, up_off, stream);
        return launch_tc_persistent<256, TC_PARTIAL>(mw, mx, out, T, N, K, ldo, up_off, stream);
    }
    if (MODE == TC_PARTIAL && tc_wide(T, N))
        return bn == 128 ? launch_tc<128, TC_PARTIAL2>(mw, mx, out, T, N / 2, K, splits, slice_stride, ldo, N / 2, early_w, stream)
                         : launch_tc<64, TC_PARTIAL2>(mw, mx, out, T, N / 2, K, splits, slice_stride, ldo, N / 2, early_w, stream);
    switch (bn) {
        case 16: return launch_tc<16, MODE>(mw, mx, out, T, N, K, splits, slice_stride, ldo, up_off, early_w, stream);
        case 32: return launch_tc<32, MODE>(mw, mx, out, T, N, K, splits, slice_stride, ldo, up_off, early_w, stream);
        case 64: return launch_tc<64, MODE>(mw, mx, out, T, N, K, splits, slice_stride, ldo, up_off, early_w, stream);
        case 128: return launch_tc<128, MODE>(mw, mx, out, T, N, K, splits, slice_stride, ldo, up_off, early_w, stream);
        default: return launch_tc<256, MODE>(mw, mx, out, T, N, K, splits, slice_stride, ldo, up_off, early_w, stream);
    }
}

// out float32 [splits, T, N] (slice stride given), x bf16 [T, K], w bf16 [N, K].  weights_static
// says that w was complete before the kernel that precedes this one in the stream began (a
// model's weights): few-token products then fetch their first weight tiles while that kernel
// still runs, and wait for it only before they read x.
KESTREL_API int kestrel_gemm_tc_w(const void *x, const void *w, float *out, int T, int N, int K, long long ldx,
                                  long long ldw, long long ldo, int splits, long long slice_stride, int weights_static,
                                  cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(kestrel_gemm_tc_supported(x, w, T, N, K, ldx, ldw), "gemm_tc: sizes T=%d N=%d K=%d ldx=%lld ldw=%lld do not fit the TMA rules (multiples of 8, 16-byte aligned)", T, N, K, ldx, ldw);
    int total_kb = (K + TC_BK - 1) / TC_BK;
    KESTREL_REQUIRE(splits >= 1 && splits <= total_kb && ((total_kb + splits - 1) / splits) * (splits - 1) < total_kb,
                    "gemm_tc: %d slices over %d k-blocks would leave a slice empty", splits, total_kb);
    return dispatch_tc<TC_PARTIAL>(x, w, out, T, N, N, K, ldx, ldw, ldo, splits, slice_stride, 0, weights_static ? 1 : 0, stream);
}

// The same for a w that the preceding kernel may have written.
KESTREL_API int kestrel_gemm_tc(const void *x, const void *w, float *out, int T, int N, int K, long long ldx,
                                long long ldw, long long ldo, int splits, long long slice_stride, cudaStream_t stream) {
    return kestrel_gemm_tc_w(x, w, out, T, N, K, ldx, ldw, ldo, splits, slice_stride, 0, stream);
}

// residual float32 [T, N] += x w^T, in the product's epilogue (many tokens on CTA pairs only).
// Returns 0 when done, 1 when this product cannot do it (few tokens, or pairs cannot be
// scheduled): the caller then takes the product as slices and lets their consumer add them.
KESTREL_API int kestrel_gemm_tc_add(const void *x, const void *w, float *residual, int T, int N, int K, long long ldx,
                                    long long ldw, long long ldo, cudaStream_t stream) {
    if (T == 0) return 0;
    if (T <= g_pair_min_tokens || !g_persistent || !g_pairs || !kestrel_gemm_tc_supported(x, w, T, N, K, ldx, ldw)) return 1;
    if (kestrel_gemm_tc_splits(T, N, K) > 1) return 1;      // too few output tiles for the CTA pairs: cut along K, as slices
    CUtensorMap mw, mx;
    int rc = kestrel_tensor_map_bf16(&mw, w, N, K, ldw, TC_BM);
    if (rc) return rc;
    rc = kestrel_tensor_map_bf16(&mx, x, T, K, ldx, TCP_BN / 2);
    if (rc) return rc;
    return launch_tc_pair<TC_PARTIAL>(mw, mx, residual, T, N, K, ldo, 0, 1, 1, 0, stream);
}

// The q, k, v product of a prompt portion and everything between it and attention in one kernel
// (QKV_PREP above): x bf16 [T, K], w bf16 [(nq + 2 nkv) * 128, K]; the other arguments as
// kestrel_attn_prepare's.  Returns 0 when done; 1 when this form does not apply - few tokens, a
// product that is better cut along K (a few hundred tokens), another head size or rotation,
// pairs that cannot be scheduled - and nothing was launched: the caller then runs the product and
// the prepare kernel.
KESTREL_API int kestrel_gemm_tc_qkv_prepare(const void *x, const void *w, int T, int K, long long ldx, long long ldw, const float *bias,
                                            const float *q_norm_w, const float *k_norm_w, float norm_eps, const float *inv_freq, int rot,
                                            int rot_mode, float rot_scale, const int *positions, const int *seq_of_token,
                                            const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache,
                                            void *q_out, int nq, int nkv, int hd, int write_kv, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!g_qkv_fused || hd != TC_BM || rot != TC_BM || rot_mode != 0 || !inv_freq || nq <= 0 || nkv <= 0 || page_size <= 0) return 1;
    const int N = (nq + 2 * nkv) * TC_BM;
    if (T <= g_pair_min_tokens || !g_persistent || !g_pairs || !kestrel_gemm_tc_supported(x, w, T, N, K, ldx, ldw)) return 1;
    if (g_qkv_fused < 2) {
        // uncut where cutting along K gains nothing, or little while the tiles come in three rounds
        // or more, so that all but the last epilogue run under the next tile's products (measured:
        // 1,792 tokens 98 us uncut and fused against 117 us in two slices with the prepare kernel;
        // 512 tokens, one round, 44 against 36)
        const int S = kestrel_gemm_tc_splits(T, N, K);
        long long waves = 0;
        const long long whole = pair_cost(T, N, K, 1, &waves);
        if (S > 1 && !(waves >= 3 && whole * 10 <= pair_cost(T, N, K, S) * 11)) return 1;
    }
    if ((((uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) != 0) return 1;
    CUtensorMap mw, mx;
    int rc = kestrel_tensor_map_bf16(&mw, w, N, K, ldw, TC_BM);
    if (rc) return rc;
    rc = kestrel_tensor_map_bf16(&mx, x, T, K, ldx, TCP_BN / 2);
    if (rc) return rc;
    QkvPrepParams prep;
    prep.bias = bias; prep.q_norm_w = q_norm_w; prep.k_norm_w = k_norm_w; prep.inv_freq = inv_freq;
    prep.norm_eps = norm_eps; prep.rot_scale = rot_scale; prep.positions = positions; prep.seq_of_token = seq_of_token;
    prep.block_table = block_table; prep.table_stride = table_stride; prep.page_size = page_size;
    prep.k_cache = (__nv_bfloat16 *)k_cache; prep.v_cache = (__nv_bfloat16 *)v_cache; prep.q_out = (__nv_bfloat16 *)q_out;
    prep.nq = nq; prep.nkv = nkv; prep.write_kv = write_kv ? 1 : 0;
    return launch_tc_pair<TC_QKV_PREP>(mw, mx, nullptr, T, N, K, 0, 0, 0, 1, 0, stream, prep);
}

KESTREL_API void kestrel_gemm_tc_set_qkv_fused(int mode) { g_qkv_fused = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }

// out bf16 [T, ff] = silu(x Wg^T) * (x Wu^T), w bf16 [2 ff, K] with the gate rows first;
// weights_static as in kestrel_gemm_tc_w
KESTREL_API int kestrel_gemm_tc_swiglu_w(const void *x, const void *w, void *out, int T, int ff, int K, long long ldx,
                                         long long ldw, long long ldo, int weights_static, cudaStream_t stream) {
    if (T == 0) return 0;
    KESTREL_REQUIRE(kestrel_gemm_tc_supported(x, w, T, ff, K, ldx, ldw), "gemm_tc_swiglu: sizes T=%d ff=%d K=%d do not fit the TMA rules", T, ff, K);
    return dispatch_tc<TC_SWIGLU>(x, w, out, T, ff, 2 * ff, K, ldx, ldw, ldo, 1, 0, ff, weights_static ? 1 : 0, stream);
}

KESTREL_API int kestrel_gemm_tc_swiglu(const void *x, const void *w, void *out, int T, int ff, int K, long long ldx,
                                       long long ldw, long long ldo, cudaStream_t stream) {
    return kestrel_gemm_tc_swiglu_w(x, w, out, T, ff, K, ldx, ldw, ldo, 0, stream);
}

// Reads (and clears) the error word that a bounded wait sets when it runs out: 0 = none,
// 1 = the loader waited for a free stage, 2 = the MMA thread waited for data, 3 = the epilogue
// waited for the accumulator, 4 = the MMA thread waited for a drained accumulator.  Synchronises the device.
KESTREL_API int kestrel_gemm_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    return v;
}
