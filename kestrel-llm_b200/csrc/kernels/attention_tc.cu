// Causal attention of prompt portions on the 5th-generation tensor cores, head size 128.
//
// A CTA owns 128 rows - (token, query head of one kv group) pairs, token-major, as in
// attention_mma.cu - and walks the keys its rows may see in tiles of 128, anchored at
// multiples of 128 of the absolute position:
//   S = Q K^T    tcgen05.mma M=128 N=128, 8 steps of K=16 over the head size; Q and the K tile
//                sit in shared memory as K-major operands (two panels of 64 dims, rows of 128
//                bytes, 128-byte swizzle); S goes to TMEM columns 0..127;
//   softmax      thread r owns row r: two passes of tcgen05.ld over S (row maximum, then
//                exp2 and sum in float32), P written as bfloat16 into the K tile's shared
//                memory (K is no longer needed), again as a K-major operand;
//   PV           tcgen05.mma with P as A and the V tile as an MN-major B operand (V rows are
//                keys, 128 bytes of 64 dims each, which is MN-major for a [dim, key] product);
//                the tile's product goes to TMEM columns 128..255 and is added to the row's
//                float32 output registers after rescaling by 2^(m_old - m_new).
// The tiles come from the paged cache through the block table with cp.async, written at the
// swizzled addresses the operand descriptors expect.  Shared memory per CTA is 96 KB (Q, K/P,
// V), so two CTAs share an SM and one computes while the other loads.  Every mbarrier wait is
// bounded; the error word is read by kestrel_attention_tc_error.  Formulas as in
// attention_plain.cu (reference: st.c:10779-10911, st.c:9762-9859).
#include "attention_params.cuh"
#include "tcgen05.cuh"
#include <math.h>

#define AT_THREADS 128
#define AT_BM 128
#define AT_BN 128
#define AT_HD 128
#define AT_PANEL (128 * 128)            // bytes of one panel: 128 rows of 128 bytes

__device__ int g_at_error = 0;

__device__ __forceinline__ void at_cp_async16(uint32_t dst, const void *src, bool valid) {
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float *v) {
    tc_ld16(taddr, v);
    tc_ld16(taddr + 16, v + 16);
}

__global__ void __launch_bounds__(AT_THREADS)
attention_tc_kernel(const AttnParams p) {
    pdl_launch_dependents();
    // M = 128, N = 128, bf16 x bf16 -> f32; both operands K-major for S, B MN-major for PV
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BN >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
    constexpr uint32_t IDESC_PV = IDESC_S | (1u << 16);
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base, kp_s = base + 2 * AT_PANEL, v_s = base + 4 * AT_PANEL;
    const uint32_t bar = base + 6 * AT_PANEL, tmem_slot = bar + 8;
    volatile uint32_t *tmem_slot_ptr = (volatile uint32_t *)(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    uint8_t *kp_ptr = smem_raw + (kp_s - smem_u32(smem_raw));

    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;
    pdl_wait();

    const int tile = blockIdx.x, kvh = blockIdx.y;
    const int seq = p.tile_seq[tile], row0 = p.tile_row0[tile];
    const int G = p.nq / p.nkv;
    const int tok_begin = p.cu_seqlens[seq], n_tok = p.cu_seqlens[seq + 1] - tok_begin;
    const int kv_len = p.kv_lens[seq];
    const int pos_begin = kv_len - n_tok;
    const int rows_here = min(AT_BM, n_tok * G - row0);
    const int *table = p.block_table + (size_t)seq * p.table_stride;
    const int first_tok = row0 / G, last_tok = (row0 + rows_here - 1) / G;
    const int k_hi = pos_begin + last_tok + 1;
    const int k_first = p.window > 0 ? max(0, pos_begin + first_tok - p.window + 1) : 0;
    const int k_lo = (k_first / AT_BN) * AT_BN;
    const int n_tiles = (k_hi - k_lo + AT_BN - 1) / AT_BN;

    // this thread's row
    const bool row_ok = tid < rows_here;
    const int my_pos = row_ok ? pos_begin + (row0 + tid) / G : -1;
    const int my_lo = p.window > 0 ? max(0, my_pos - p.window + 1) : 0;

    // Q: row r of the tile, 16 chunks of 8 dims; thread t copies chunk t % 16 of rows t / 16 + 8 j
    {
        int c = tid & 15;
        for (int r = tid >> 4; r < AT_BM; r += 8) {
            bool valid = r < rows_here;
            size_t off = 0;
            if (valid) {
                int row = row0 + r;
                off = ((size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G) * AT_HD + c * 8;
            }
            at_cp_async16(q_s + (c >> 3) * AT_PANEL + swizzle128(r, c & 7), p.q + off, valid);
        }
    }
    // K and V tile: thread t copies chunk t % 16 of keys (t / 16) * 16 .. + 15
    auto load_kv = [&](int t) {
        int c = tid & 15, r0 = (tid >> 4) * 16;
        int s0 = k_lo + t * AT_BN + r0;
        bool one_page = p.page_size % 16 == 0;
        size_t page_off = 0;
        if (one_page && s0 + 16 > k_first && s0 < k_hi) {
            int page = table[s0 / p.page_size];
            page_off = (((size_t)page * p.nkv + kvh) * p.page_size + (s0 % p.page_size)) * AT_HD + c * 8;
        }
#pragma unroll 4
        for (int j = 0; j < 16; ++j) {
            int s = s0 + j, r = r0 + j;
            bool valid = s >= k_first && s < k_hi;
            size_t off = 0;
            if (valid) {
                if (one_page) {
                    off = page_off + (size_t)j * AT_HD;
                } else {
                    int page = table[s / p.page_size];
                    off = (((size_t)page * p.nkv + kvh) * p.page_size + (s % p.page_size)) * AT_HD + c * 8;
                }
            }
            uint32_t sw = (c >> 3) * AT_PANEL + swizzle128(r, c & 7);
            at_cp_async16(kp_s + sw, p.k_cache + off, valid);
            at_cp_async16(v_s + sw, p.v_cache + off, valid);
        }
    };

    float o[AT_HD];
#pragma unroll
    for (int i = 0; i < AT_HD; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    uint32_t phase = 0;
    bool ok = true;
    const uint32_t lane_base = ((uint32_t)(32 * warp)) << 16;

    for (int t = 0; t < n_tiles && ok; ++t) {
        const int kbase = k_lo + t * AT_BN;
        load_kv(t);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // cp.async writes -> tensor-core reads
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < AT_HD / 16; ++ks) {
                uint32_t off = (ks >> 2) * AT_PANEL + (ks & 3) * 32;
                tc_mma(tmem, smem_desc(q_s + off), smem_desc(kp_s + off), IDESC_S, ks > 0 ? 1u : 0u);
            }
            tc_commit(bar);
        }
        if (!mbar_wait(bar, phase)) { atomicExch(&g_at_error, 1); ok = false; }
        phase ^= 1;
        tc_fence_after();

        // softmax of this thread's row: pass 1, the maximum
        const bool whole = kbase >= k_first && kbase + AT_BN <= k_hi && kbase + AT_BN - 1 <= my_pos && kbase >= my_lo;
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < AT_BN; c += 32) {
            float s[32];
            tc_ld32(tmem + lane_base + c, s);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                int key = kbase + c + j;
                bool vis = whole || (key <= my_pos && key >= my_lo && key < k_hi && key >= k_first);
                mx = fmaxf(mx, vis ? s[j] * p.scale_log2 : -INFINITY);
            }
        }
        float m_new = fmaxf(m_run, mx);
        float m_use = m_new == -INFINITY ? 0.f : m_new;
        float alpha = at_exp2(m_run - m_use);
        m_run = m_new;
        // pass 2: p = 2^(s - m), row sum, P as bfloat16 into the K tile's memory
        float l_add = 0.f;
#pragma unroll 1
        for (int c = 0; c < AT_BN; c += 32) {
            float s[32];
            tc_ld32(tmem + lane_base + c, s);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                int key = kbase + c + j;
                bool vis = whole || (key <= my_pos && key >= my_lo && key < k_hi && key >= k_first);
                float pv = vis ? at_exp2(s[j] * p.scale_log2 - m_use) : 0.f;
                s[j] = pv;
                l_add += pv;
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {        // four chunks of 8 keys
                int chunk = (c >> 3) + g;        // 0..15 over the 128 keys
                uint4 u;
                __nv_bfloat162 b0 = __floats2bfloat162_rn(s[8 * g + 0], s[8 * g + 1]);
                __nv_bfloat162 b1 = __floats2bfloat162_rn(s[8 * g + 2], s[8 * g + 3]);
                __nv_bfloat162 b2 = __floats2bfloat162_rn(s[8 * g + 4], s[8 * g + 5]);
                __nv_bfloat162 b3 = __floats2bfloat162_rn(s[8 * g + 6], s[8 * g + 7]);
                u.x = *reinterpret_cast<uint32_t *>(&b0);
                u.y = *reinterpret_cast<uint32_t *>(&b1);
                u.z = *reinterpret_cast<uint32_t *>(&b2);
                u.w = *reinterpret_cast<uint32_t *>(&b3);
                *reinterpret_cast<uint4 *>(kp_ptr + (chunk >> 3) * AT_PANEL + swizzle128(tid, chunk & 7)) = u;
            }
        }
        l_run = l_run * alpha + l_add;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // P written by threads -> tensor-core reads
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < AT_BN / 16; ++ks) {
                // A = P: keys 16 ks.. in panel ks / 4; B = V: 16 keys down = 2 groups of 8 rows
                uint64_t da = smem_desc(kp_s + (ks >> 2) * AT_PANEL + (ks & 3) * 32);
                uint64_t db = smem_desc_mn_major(v_s + ks * 2048, AT_PANEL);
                tc_mma(tmem + 128, da, db, IDESC_PV, ks > 0 ? 1u : 0u);
            }
            tc_commit(bar);
        }
        if (!mbar_wait(bar, phase)) { atomicExch(&g_at_error, 2); ok = false; }
        phase ^= 1;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < AT_HD; c += 32) {
            float pvv[32];
            tc_ld32(tmem + lane_base + 128 + c, pvv);
#pragma unroll
            for (int j = 0; j < 32; ++j) o[c + j] = o[c + j] * alpha + pvv[j];
        }
        tc_fence_before();
        __syncthreads();          // K/P and V may be overwritten, S and PV columns rewritten
    }

    if (row_ok && ok) {
        int row = row0 + tid;
        size_t qrow = (size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G;
        float inv = 1.0f / l_run;
        __nv_bfloat16 *po = p.out + qrow * AT_HD;
#pragma unroll
        for (int c = 0; c < AT_HD; c += 8) {
            uint4 u;
            __nv_bfloat162 b0 = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv);
            __nv_bfloat162 b1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
            __nv_bfloat162 b2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv);
            __nv_bfloat162 b3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
            u.x = *reinterpret_cast<uint32_t *>(&b0);
            u.y = *reinterpret_cast<uint32_t *>(&b1);
            u.z = *reinterpret_cast<uint32_t *>(&b2);
            u.w = *reinterpret_cast<uint32_t *>(&b3);
            *reinterpret_cast<uint4 *>(po + c) = u;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}

// Tiles of 128 rows (tile_seq / tile_row0), head size 128, no slices.
KESTREL_API int kestrel_attention_tc(const void *q, const void *k_cache, const void *v_cache, void *out,
                                     const int *tile_seq, const int *tile_row0, int tiles, const int *cu_seqlens,
                                     const int *kv_lens, const int *block_table, int table_stride, int page_size,
                                     int T, int nq, int nkv, int hd, int window, float scale, cudaStream_t stream) {
    if (T == 0 || tiles == 0) return 0;
    KESTREL_REQUIRE(hd == AT_HD, "attention_tc: head size %d; this kernel is built for %d", hd, AT_HD);
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_tc: %d query heads over %d kv heads", nq, nkv);
    KESTREL_REQUIRE(nkv <= 65535, "attention_tc: grid too large");
    AttnParams p = {};
    p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out; p.tile_seq = tile_seq; p.tile_row0 = tile_row0; p.cu_seqlens = cu_seqlens;
    p.kv_lens = kv_lens; p.block_table = block_table; p.table_stride = table_stride; p.page_size = page_size;
    p.nq = nq; p.nkv = nkv; p.hd = hd; p.window = window; p.slices = 1; p.slice_len = 1 << 30;
    p.scale_log2 = scale * 1.4426950408889634f;
    size_t smem = 6 * AT_PANEL + 64 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return kestrel_fail(-3, "attention_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    kestrel_launch(attention_tc_kernel, dim3(tiles, nkv), dim3(AT_THREADS), smem, stream, p);
    return kestrel_check_launch("attention_tc");
}

// Error word of the kernel's bounded waits: 0 = none, 1 = waited for S, 2 = waited for PV.
// Synchronises the device and clears the word.
KESTREL_API int kestrel_attention_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_at_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_at_error, &zero, sizeof(int));
    return v;
}
