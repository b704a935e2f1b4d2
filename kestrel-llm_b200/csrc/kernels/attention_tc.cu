// Causal attention of prompt portions on the 5th-generation tensor cores, head size 128.
//
// A CTA owns 128 rows - (token, query head of one kv group) pairs, token-major, as in
// attention_mma.cu - and walks the keys its rows may see in tiles of 128, anchored at
// multiples of 128 of the absolute position:
//   S = Q K^T    tcgen05.mma M=128 N=128, 8 steps of K=16 over the head size; Q and the K tile
//                sit in shared memory as K-major operands (two panels of 64 dims, rows of 128
//                bytes, 128-byte swizzle); S goes to TMEM columns 0..127;
//   softmax      two threads own a row, 64 keys each: one tcgen05.ld of S, row maximum (the
//                halves exchange it), exp2 and sum in float32, P written as bfloat16 into the
//                K tile's shared memory (K is no longer needed), again as a K-major operand;
//   PV           tcgen05.mma with P as A and the V tile as an MN-major B operand (V rows are
//                keys, 128 bytes of 64 dims each, which is MN-major for a [dim, key] product);
//                the tile's product goes to TMEM columns 128..255 and is added to the row's
//                float32 output registers after rescaling by 2^(m_old - m_new).
// The tiles come from the paged cache through the block table with cp.async, written at the
// swizzled addresses the operand descriptors expect: V(t) lands while S(t) is computed and
// softmaxed, K(t+1) while the output is updated.  Shared memory per CTA is 97 KB (Q, K/P, V),
// so two CTAs share an SM.  Every mbarrier wait is
// bounded; the error word is read by kestrel_attention_tc_error.  Formulas as in
// attention_plain.cu (reference: st.c:10779-10911, st.c:9762-9859).
#include "attention_params.cuh"
#include "tcgen05.cuh"
#include <math.h>

#define AT_THREADS 256
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
// 64 consecutive TMEM columns of this thread's lane: four loads in flight, one wait
__device__ __forceinline__ void tc_ld64(uint32_t taddr, float *v) {
    uint32_t r[64];
#pragma unroll
    for (int q = 0; q < 4; ++q)
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[16 * q + 0]), "=r"(r[16 * q + 1]), "=r"(r[16 * q + 2]), "=r"(r[16 * q + 3]), "=r"(r[16 * q + 4]),
              "=r"(r[16 * q + 5]), "=r"(r[16 * q + 6]), "=r"(r[16 * q + 7]), "=r"(r[16 * q + 8]), "=r"(r[16 * q + 9]),
              "=r"(r[16 * q + 10]), "=r"(r[16 * q + 11]), "=r"(r[16 * q + 12]), "=r"(r[16 * q + 13]), "=r"(r[16 * q + 14]),
              "=r"(r[16 * q + 15])
            : "r"(taddr + 16 * q));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// 256 threads: thread (r, h) = (tid % 128, tid / 128) owns row r and half h of it: 64 of the
// tile's 128 keys in the softmax, 64 of the 128 output dims.  Warps w and w + 4 share TMEM
// lanes 32 (w % 4)...; the two halves of a row exchange their maxima through shared memory.
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
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_ptr = (volatile uint32_t *)(aligned + 6 * AT_PANEL + 8);
    float *xchg = (float *)(aligned + 6 * AT_PANEL + 16);           // [2][128] row maxima of the halves
    uint8_t *kp_ptr = aligned + 2 * AT_PANEL;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int r = tid & 127, h = tid >> 7;
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

    const int tile = blockIdx.x, kvh = blockIdx.y, slice = blockIdx.z;
    const int slice_len = p.slice_len_ptr ? *p.slice_len_ptr : p.slice_len;
    const int seq = p.tile_seq[tile], row0 = p.tile_row0[tile];
    const int G = p.nq / p.nkv;
    const int tok_begin = p.cu_seqlens[seq], n_tok = p.cu_seqlens[seq + 1] - tok_begin;
    const int kv_len = p.kv_lens[seq];
    const int pos_begin = kv_len - n_tok;
    const int rows_here = min(AT_BM, n_tok * G - row0);
    const int *table = p.block_table + (size_t)seq * p.table_stride;
    const int first_tok = row0 / G, last_tok = (row0 + rows_here - 1) / G;
    // keys this CTA's rows may see, cut to its slice of the key range (slices are multiples of 128)
    const int k_hi = min(pos_begin + last_tok + 1, (slice + 1) * slice_len);
    const int k_first = max(p.window > 0 ? max(0, pos_begin + first_tok - p.window + 1) : 0, slice * slice_len);
    const int k_lo = (k_first / AT_BN) * AT_BN;
    const int n_tiles = k_hi > k_lo ? (k_hi - k_lo + AT_BN - 1) / AT_BN : 0;
    // warps none of whose 32 rows exist (decode: a few rows per request) skip the softmax arithmetic
    const bool warp_has_rows = 32 * (warp & 3) < rows_here;

    const bool row_ok = r < rows_here;
    const int my_pos = row_ok ? pos_begin + (row0 + r) / G : -1;
    const int my_lo = p.window > 0 ? max(0, my_pos - p.window + 1) : 0;

    // copies: thread t moves 16-byte chunk t % 16 of rows (t / 16) * 8 .. + 7
    const int ld_c = tid & 15, ld_r0 = (tid >> 4) * 8;
    const uint32_t ld_panel = (uint32_t)(ld_c >> 3) * AT_PANEL;
    {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int rr = ld_r0 + j;
            bool valid = rr < rows_here;
            size_t off = 0;
            if (valid) {
                int row = row0 + rr;
                off = ((size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G) * AT_HD + ld_c * 8;
            }
            at_cp_async16(q_s + ld_panel + swizzle128(rr, ld_c & 7), p.q + off, valid);
        }
    }
    const bool one_page = p.page_size % 8 == 0;
    auto load_tile = [&](int t, uint32_t dst, const __nv_bfloat16 *cache) {
        int s0 = k_lo + t * AT_BN + ld_r0;
        size_t page_off = 0;
        if (one_page && s0 + 8 > k_first && s0 < k_hi) {
            int page = table[s0 / p.page_size];
            page_off = (((size_t)page * p.nkv + kvh) * p.page_size + (s0 % p.page_size)) * AT_HD + ld_c * 8;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int s = s0 + j;
            bool valid = s >= k_first && s < k_hi;
            size_t off = 0;
            if (valid) {
                if (one_page) {
                    off = page_off + (size_t)j * AT_HD;
                } else {
                    int page = table[s / p.page_size];
                    off = (((size_t)page * p.nkv + kvh) * p.page_size + (s % p.page_size)) * AT_HD + ld_c * 8;
                }
            }
            at_cp_async16(dst + ld_panel + swizzle128(ld_r0 + j, ld_c & 7), cache + off, valid);
        }
    };
    if (n_tiles > 0) load_tile(0, kp_s, p.k_cache);
    asm volatile("cp.async.commit_group;" ::: "memory");             // group: Q and K(0)

    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    uint32_t phase = 0;
    bool ok = true;
    const uint32_t lane_base = ((uint32_t)(32 * (warp & 3))) << 16;
    const int col0 = 64 * h;

    for (int t = 0; t < n_tiles && ok; ++t) {
        const int kbase = k_lo + t * AT_BN;
        load_tile(t, v_s, p.v_cache);                                 // V(t) lands while S is computed and softmaxed
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");          // K(t) (and Q) have landed
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // cp.async writes -> tensor-core reads
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

        // softmax of this thread's half row
        float alpha = 1.f;
        if (warp_has_rows) {
            float s[64];
            tc_ld64(tmem + lane_base + col0, s);
            const bool whole = kbase >= k_first && kbase + AT_BN <= k_hi && kbase + AT_BN - 1 <= my_pos && kbase >= my_lo;
            float mx = -INFINITY;
            if (whole) {
#pragma unroll
                for (int j = 0; j < 64; ++j) { s[j] *= p.scale_log2; mx = fmaxf(mx, s[j]); }
            } else {
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    int key = kbase + col0 + j;
                    bool vis = key <= my_pos && key >= my_lo && key < k_hi && key >= k_first;
                    s[j] = vis ? s[j] * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, s[j]);
                }
            }
            xchg[h * 128 + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");   // the two warps that share these rows
            mx = fmaxf(mx, xchg[(h ^ 1) * 128 + r]);
            float m_new = fmaxf(m_run, mx);
            float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha = at_exp2(m_run - m_use);
            m_run = m_new;
            float l_add = 0.f;
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                s[j] = at_exp2(s[j] - m_use);
                l_add += s[j];
            }
            l_run = l_run * alpha + l_add;
            // P as bfloat16 into the K tile's memory: keys 64 h .. + 63 are panel h of row r
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                uint4 u;
                __nv_bfloat162 b0 = __floats2bfloat162_rn(s[8 * g + 0], s[8 * g + 1]);
                __nv_bfloat162 b1 = __floats2bfloat162_rn(s[8 * g + 2], s[8 * g + 3]);
                __nv_bfloat162 b2 = __floats2bfloat162_rn(s[8 * g + 4], s[8 * g + 5]);
                __nv_bfloat162 b3 = __floats2bfloat162_rn(s[8 * g + 6], s[8 * g + 7]);
                u.x = *reinterpret_cast<uint32_t *>(&b0);
                u.y = *reinterpret_cast<uint32_t *>(&b1);
                u.z = *reinterpret_cast<uint32_t *>(&b2);
                u.w = *reinterpret_cast<uint32_t *>(&b3);
                *reinterpret_cast<uint4 *>(kp_ptr + h * AT_PANEL + swizzle128(r, g)) = u;
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");          // V(t) has landed
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P and V -> tensor-core reads
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
        if (t + 1 < n_tiles) load_tile(t + 1, kp_s, p.k_cache);       // P is consumed: K(t+1) may overwrite it
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (warp_has_rows) {
            float pvv[64];
            tc_ld64(tmem + lane_base + 128 + col0, pvv);
#pragma unroll
            for (int j = 0; j < 64; ++j) o[j] = o[j] * alpha + pvv[j];
        }
        tc_fence_before();
        __syncthreads();          // S and PV columns may be rewritten, V overwritten
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // the row's sum is the sum of its halves
    __syncthreads();
    xchg[h * 128 + r] = l_run;
    __syncthreads();
    float l_tot = l_run + xchg[(h ^ 1) * 128 + r];
    if (row_ok && ok) {
        int row = row0 + r;
        size_t qrow = (size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G;
        if (p.slices > 1) {
            // this slice's unnormalised out, maximum and sum; attention_merge_kernel combines the slices
            float *po = p.part_o + (qrow * p.slices + slice) * AT_HD + col0;
#pragma unroll
            for (int c = 0; c < 64; c += 4) *reinterpret_cast<float4 *>(po + c) = make_float4(o[c], o[c + 1], o[c + 2], o[c + 3]);
            if (h == 0) {
                p.part_ml[(qrow * p.slices + slice) * 2] = m_run;
                p.part_ml[(qrow * p.slices + slice) * 2 + 1] = l_tot;
            }
        } else {
            float inv = 1.0f / l_tot;
            __nv_bfloat16 *po = p.out + qrow * AT_HD + col0;
#pragma unroll
            for (int c = 0; c < 64; c += 8) {
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
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}

extern "C" int kestrel_attention_merge(const float *part_o, const float *part_ml, void *out, const int *tile_seq,
                                       const int *tile_row0, int tiles, const int *cu_seqlens, int slices, int hd,
                                       int nq, int nkv, cudaStream_t stream);

// Tiles of up to 128 rows (tile_seq / tile_row0), head size 128.  With slices > 1 (tiles of at
// most 16 rows: decode tokens) every CTA takes a slice of slice_len keys, a multiple of 128 -
// or the value at slice_len_ptr on the device - and the slices are merged in ascending order;
// part_o / part_ml are scratch of T * nq * slices * 128 and T * nq * slices * 2 floats.
KESTREL_API int kestrel_attention_tc(const void *q, const void *k_cache, const void *v_cache, void *out,
                                     float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0,
                                     int tiles, const int *cu_seqlens, const int *kv_lens, const int *block_table,
                                     int table_stride, int page_size, int T, int nq, int nkv, int hd, int window,
                                     int slices, int slice_len, const int *slice_len_ptr, float scale,
                                     cudaStream_t stream) {
    if (T == 0 || tiles == 0) return 0;
    KESTREL_REQUIRE(hd == AT_HD, "attention_tc: head size %d; this kernel is built for %d", hd, AT_HD);
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_tc: %d query heads over %d kv heads", nq, nkv);
    KESTREL_REQUIRE(slices >= 1 && slice_len > 0 && slice_len % AT_BN == 0, "attention_tc: slice length %d must be a positive multiple of %d", slice_len, AT_BN);
    KESTREL_REQUIRE(slices == 1 || (part_o && part_ml), "attention_tc: %d slices without scratch", slices);
    KESTREL_REQUIRE(nkv <= 65535 && slices <= 65535, "attention_tc: grid too large");
    AttnParams p = {};
    p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out; p.part_o = part_o; p.part_ml = part_ml; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
    p.cu_seqlens = cu_seqlens; p.kv_lens = kv_lens; p.block_table = block_table; p.table_stride = table_stride;
    p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.hd = hd; p.window = window; p.slices = slices; p.slice_len = slice_len;
    p.slice_len_ptr = slice_len_ptr;
    p.scale_log2 = scale * 1.4426950408889634f;
    size_t smem = 6 * AT_PANEL + 16 + 2 * 128 * 4 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return kestrel_fail(-3, "attention_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    kestrel_launch(attention_tc_kernel, dim3(tiles, nkv, slices), dim3(AT_THREADS), smem, stream, p);
    int rc = kestrel_check_launch("attention_tc");
    if (rc || slices == 1) return rc;
    return kestrel_attention_merge(part_o, part_ml, out, tile_seq, tile_row0, tiles, cu_seqlens, slices, hd, nq, nkv, stream);
}

// Error word of the kernel's bounded waits: 0 = none, 1 = waited for S, 2 = waited for PV.
// Synchronises the device and clears the word.
KESTREL_API int kestrel_attention_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_at_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_at_error, &zero, sizeof(int));
    return v;
}
