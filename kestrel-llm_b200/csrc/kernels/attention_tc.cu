// Causal attention of prompt portions on the 5th-generation tensor cores, head size 128.
//
// A CTA owns up to 256 rows - (token, query head of one kv group) pairs, token-major, as in
// attention_mma.cu - as two row tiles A and B of 128, and walks the keys its rows may see in
// tiles of 128, anchored at multiples of 128 of the absolute position.  Both row tiles use the
// same K and V tiles, so a key tile is fetched once per 256 rows.  Eleven warps in three roles,
// coupled by mbarriers:
//   loaders  (warp 8 for K, warp 10 for V)  look the tile's pages up in the block table and
//            fetch K(t) or V(t) with TMA (boxes of one page, or of 128 keys of a larger page, by
//            64 dims; 128-byte swizzle) into two-stage rings, each as far ahead as its ring allows;
//   issuer   (warp 9, one thread)  S_X(t) = Q_X K(t)^T and O_X += P_X(t) V(t) for X = A, B in the
//            order S_A S_B | PV_A S_A' PV_B S_B' | ..., so that the tensor cores work on one row
//            tile while the other is softmaxed: tcgen05.mma M=128 N=128, 8 steps of K=16.  Q and K
//            are K-major operands in shared memory (two panels of 64 elements, rows of 128
//            bytes), V an MN-major one (its rows are keys); P is read from TMEM;
//   softmax  (warps 0-3 for A, 4-7 for B)  a thread owns a row: its 128 scores come out of TMEM
//            once, into registers; row maximum, exp2 and sum in float32, P written as packed
//            bfloat16 over the first 64 columns of S in TMEM.  Nothing is exchanged between
//            threads and no barrier stands between S and P (with two threads a row and the
//            scores read twice, once for the maximum and once for the exponentials, the two
//            hand-overs between the halves were on every tile's critical path).
// TMEM (512 columns): S_A, S_B, O_A, O_B.  The output accumulates in TMEM; it is rescaled by
// 2^(m_old - m_new) only when a row's maximum has grown by more than 8 (in log2 units) since the
// reference it was accumulated against - P then stays below 2^8, which costs bfloat16 and the
// float32 sum no precision - and the normalisation at the end uses the same reference.
// Keys outside [first key, last key] of a row tile are masked in S; V rows outside the CTA's
// range are zeroed in shared memory (a page may hold another request's stale values there, and
// 0 x NaN would not be 0).  Shared memory per CTA is 193 KB: one CTA per SM; CTAs with the most
// keys are launched first.  Every mbarrier wait is bounded; the error word is read by
// kestrel_attention_tc_error.  Formulas as in attention_plain.cu (reference: st.c:10779-10911,
// st.c:9762-9859).
#include "attention_params.cuh"
#include "tcgen05.cuh"
#include <math.h>

#define AT_THREADS 352           // 8 softmax warps, two loaders, the issuer
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
// 32 consecutive TMEM columns of this thread's lane into registers; at_ld_wait() before they are used
__device__ __forceinline__ void at_ld32(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void at_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// two float32 lanes in one instruction (fma.rn.f32x2, add.rn.f32x2): half the issue slots of the
// softmax's multiply-adds and sums
__device__ __forceinline__ uint64_t at_pack2(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void at_unpack2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t at_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t at_add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 16 packed words into 16 consecutive TMEM columns of this thread's lane
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D (TMEM) = or += A (TMEM, M x 16 bfloat16 packed two to a column) x B (shared memory)
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

enum {
    B_Q_FULL = 0, B_K_FULL = 1, B_K_EMPTY = 3, B_V_FULL = 5, B_V_EMPTY = 7, B_S_FULL = 9, B_P_FULL = 11, B_PV_DONE = 13,
    B_COUNT = 15
};
#define AT_RESCALE_STEP 8.0f            // log2 units by which a row's maximum may outgrow its reference

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const AttnParams p, int cache_pages, int rows_per_tile) {
    pdl_launch_dependents();
    // M = 128, N = 128, bf16 x bf16 -> f32; both operands K-major for S, B MN-major for PV
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(AT_BN >> 3) << 17) | ((uint32_t)(AT_BM >> 4) << 24);
    constexpr uint32_t IDESC_PV = IDESC_S | (1u << 16);
    constexpr uint32_t TILE_BYTES = 2 * AT_PANEL;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t q_s = base, k_s = base + 2 * TILE_BYTES, v_s = base + 4 * TILE_BYTES;       // Q_A Q_B | K ring | V ring
    const uint32_t bars = base + 6 * TILE_BYTES, tmem_slot = bars + 8 * B_COUNT;
    volatile uint32_t *tmem_slot_ptr = (volatile uint32_t *)(aligned + 6 * TILE_BYTES + 8 * B_COUNT);
    uint8_t *v_ptr = aligned + 4 * TILE_BYTES;
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(bar(B_Q_FULL), 8);
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(B_K_FULL + b), 1);  mbar_init(bar(B_K_EMPTY + b), 1);
            mbar_init(bar(B_V_FULL + b), 1);  mbar_init(bar(B_V_EMPTY + b), 1);
            mbar_init(bar(B_S_FULL + b), 1);  mbar_init(bar(B_P_FULL + b), 4);
            mbar_init(bar(B_PV_DONE + b), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;
    pdl_wait();

    // blocks are handed out in the order of blockIdx.x: the kv heads of a tile follow each other and
    // late tiles, which see the most keys, come first - across all kv heads
    const int kvh = blockIdx.x % p.nkv, tile = (int)(gridDim.x / p.nkv) - 1 - (int)(blockIdx.x / p.nkv), slice = blockIdx.z;
    const int slice_len = attn_slice_len(p);
    const int seq = p.tile_seq[tile], row0 = p.tile_row0[tile];
    const int G = p.nq / p.nkv;
    const int tok_begin = p.cu_seqlens[seq], n_tok = p.cu_seqlens[seq + 1] - tok_begin;
    const int kv_len = p.kv_lens[seq];
    const int pos_begin = kv_len - n_tok;
    const int rows_here = min(rows_per_tile, n_tok * G - row0);         // up to 256: row tile A, then B
    const int *table = p.block_table + (size_t)seq * p.table_stride;
    const int first_tok = row0 / G, last_tok = (row0 + rows_here - 1) / G;
    // keys this CTA's rows may see, cut to its slice of the key range (slices are multiples of 128)
    const int k_hi = min(pos_begin + last_tok + 1, (slice + 1) * slice_len);
    const int k_first = max(p.window > 0 ? max(0, pos_begin + first_tok - p.window + 1) : 0, slice * slice_len);
    const int k_lo = (k_first / AT_BN) * AT_BN;
    const int n_tiles = k_hi > k_lo ? (k_hi - k_lo + AT_BN - 1) / AT_BN : 0;
    // row tile A ends earlier: it skips the key tiles beyond its last row
    const int rows_a = min(rows_here, AT_BM);
    const bool has_b = rows_here > AT_BM;
    const int k_hi_a = min(pos_begin + (row0 + rows_a - 1) / G + 1, (slice + 1) * slice_len);
    const int n_tiles_a = has_b ? (k_hi_a > k_lo ? (k_hi_a - k_lo + AT_BN - 1) / AT_BN : 0) : n_tiles;

    if (warp == 8 || warp == 10) {
        // ------------------------------------------------------------------ loaders
        // warp 8 fetches the K tiles, warp 10 the V tiles, each as far ahead as its ring allows;
        // lane l fetches the l-th page of a tile (both panels)
        const bool is_v = warp == 10;
        const CUtensorMap *map = is_v ? &map_v : &map_k;
        const int full0 = is_v ? B_V_FULL : B_K_FULL, empty0 = is_v ? B_V_EMPTY : B_K_EMPTY;
        const uint32_t ring = is_v ? v_s : k_s;
        const int box_rows = min(p.page_size, AT_BN);
        const int boxes = AT_BN / box_rows;
        for (int t = 0; t < n_tiles; ++t) {
            const int b = t & 1;
            const uint32_t par = (uint32_t)(t >> 1) & 1u;
            int row = 0;
            if (lane < boxes) {
                int s0 = k_lo + t * AT_BN + lane * box_rows;
                int idx = s0 / p.page_size;
                int page = idx < p.table_width ? table[idx] : 0;
                if (page < 0 || page >= cache_pages) page = 0;      // a released or absent page: its keys are masked, its values zeroed
                row = (page * p.nkv + kvh) * p.page_size + s0 % p.page_size;
            }
            if (!mbar_wait(bar(empty0 + b), par ^ 1u)) { atomicExch(&g_at_error, is_v ? 4 : 3); break; }
            if (lane == 0) mbar_expect_tx(bar(full0 + b), TILE_BYTES);
            __syncwarp();
            if (lane < boxes) {
                uint32_t dst = ring + b * TILE_BYTES + lane * box_rows * 128;
                tma_load_2d(dst, map, bar(full0 + b), 0, row);
                tma_load_2d(dst + AT_PANEL, map, bar(full0 + b), 64, row);
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ issuer
        if (lane == 0 && n_tiles > 0) {
            bool ok = mbar_wait(bar(B_Q_FULL), 0);
            if (!ok) atomicExch(&g_at_error, 5);
            // S_X(t) = Q_X K(t)^T into S_X; the K stage is free once the last S product of the tile is done
            auto issue_s = [&](int x, int t) {
                const int b = t & 1;
#pragma unroll
                for (int ks = 0; ks < AT_HD / 16; ++ks) {
                    uint32_t off = (ks >> 2) * AT_PANEL + (ks & 3) * 32;
                    tc_mma(tmem + x * 128, smem_desc(q_s + x * TILE_BYTES + off), smem_desc(k_s + b * TILE_BYTES + off), IDESC_S, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar(B_S_FULL + x));
            };
            // O_X (+)= P_X(t) V(t): P is read from the first 64 columns of S_X
            auto issue_pv = [&](int x, int t) {
                const int b = t & 1;
                if (!mbar_wait(bar(B_P_FULL + x), (uint32_t)t & 1u)) { atomicExch(&g_at_error, 2); return false; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < AT_BN / 16; ++ks) {
                    // A = P: keys 16 ks.. are columns 8 ks..; B = V: 16 keys down = 2 groups of 8 rows
                    uint64_t db = smem_desc_mn_major(v_s + b * TILE_BYTES + ks * 2048, AT_PANEL);
                    tc_mma_ts(tmem + 256 + x * 128, tmem + x * 128 + ks * 8, db, IDESC_PV, (t > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(bar(B_PV_DONE + x));
                return true;
            };
            auto wait_k = [&](int t) {
                if (mbar_wait(bar(B_K_FULL + (t & 1)), (uint32_t)(t >> 1) & 1u)) { tc_fence_after(); return true; }
                atomicExch(&g_at_error, 1);
                return false;
            };
            if (ok) ok = wait_k(0);
            if (ok) {
                if (n_tiles_a > 0) issue_s(0, 0);
                if (has_b) issue_s(1, 0);
                tc_commit(bar(B_K_EMPTY + 0));
            }
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int b = t & 1;
                const bool next = t + 1 < n_tiles;
                if (!mbar_wait(bar(B_V_FULL + b), (uint32_t)(t >> 1) & 1u)) { atomicExch(&g_at_error, 6); ok = false; break; }
                if (next && !(ok = wait_k(t + 1))) break;
                // PV_A(t), S_A(t+1), PV_B(t), S_B(t+1): the products of one row tile fill the time the other's softmax takes
                if (t < n_tiles_a && !(ok = issue_pv(0, t))) break;
                if (next && t + 1 < n_tiles_a) issue_s(0, t + 1);
                if (has_b && !(ok = issue_pv(1, t))) break;
                if (next && has_b) issue_s(1, t + 1);
                if (next) tc_commit(bar(B_K_EMPTY + ((t + 1) & 1)));
                tc_commit(bar(B_V_EMPTY + b));
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax
        // warps 0-3: row tile A, warps 4-7: row tile B; thread r of a tile owns row r (TMEM lane r)
        const int x = warp >> 2, r = tid & 127;
        {
            // Q: thread t moves 16-byte chunk t % 16 of rows (t / 16) * 8 .. + 7 of both row tiles
            const int ld_c = tid & 15, ld_r0 = (tid >> 4) * 8;
            const uint32_t ld_panel = (uint32_t)(ld_c >> 3) * AT_PANEL;
#pragma unroll
            for (int xt = 0; xt < 2; ++xt) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int rr = ld_r0 + j;
                    bool valid = xt * AT_BM + rr < rows_here;
                    size_t off = 0;
                    if (valid) {
                        int row = row0 + xt * AT_BM + rr;
                        off = ((size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G) * AT_HD + ld_c * 8;
                    }
                    at_cp_async16(q_s + xt * TILE_BYTES + ld_panel + swizzle128(rr, ld_c & 7), p.q + off, valid);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // cp.async writes -> tensor-core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_Q_FULL));
        }
        const int rows_x = x == 0 ? rows_a : rows_here - AT_BM;          // rows of this row tile (<= 0: none)
        const int n_tiles_x = x == 0 ? n_tiles_a : (has_b ? n_tiles : 0);
        const int k_hi_x = x == 0 ? k_hi_a : k_hi;
        const bool row_ok = r < rows_x;
        const int my_pos = row_ok ? pos_begin + (row0 + x * AT_BM + r) / G : -1;
        const int my_lo = p.window > 0 ? max(0, my_pos - p.window + 1) : 0;
        // warps none of whose 32 rows exist (decode: a few rows per request) skip the arithmetic
        const bool warp_has_rows = 32 * (warp & 3) < rows_x;
        const uint32_t lane_base = ((uint32_t)(32 * (warp & 3))) << 16;
        const uint32_t s_addr = tmem + lane_base + x * 128, o_addr = tmem + lane_base + 256 + x * 128;
        float m_ref = -INFINITY, l_run = 0.f;       // the reference the output is accumulated against, and the row's sum
        bool ok = true;             // after a wait gave up the loop runs on without waiting, so that the warps still meet

        for (int t = 0; t < n_tiles_x; ++t) {
            const int b = t & 1;
            const int kbase = k_lo + t * AT_BN;
            // S_X(t) is done - and with it, in the issuer's order, O_X += P_X(t-1) V(t-1)
            if (ok && !mbar_wait(bar(B_S_FULL + x), (uint32_t)t & 1u)) { atomicExch(&g_at_error, 7); ok = false; }
            tc_fence_after();
            if (warp_has_rows) {
                uint32_t sr[128];
#pragma unroll
                for (int c = 0; c < 128; c += 32) at_ld32(s_addr + c, sr + c);
                at_ld_wait();
                const bool whole = kbase >= k_first && kbase + AT_BN <= k_hi_x && kbase + AT_BN - 1 <= my_pos && kbase >= my_lo;
                if (!__all_sync(0xffffffffu, whole)) {
                    // keys this row may not see count as minus infinity: no maximum, a weight of zero
#pragma unroll
                    for (int j = 0; j < 128; ++j) {
                        int key = kbase + j;
                        bool vis = key <= my_pos && key >= my_lo && key < k_hi_x && key >= k_first;
                        if (!vis) sr[j] = 0xff800000u;
                    }
                }
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 128; j += 8) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        m4[k] = at_max3(m4[k], __uint_as_float(sr[j + 2 * k]), __uint_as_float(sr[j + 2 * k + 1]));
                }
                const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * p.scale_log2;   // the scale is positive
                // the reference moves only when the maximum has outgrown it by more than the step
                const bool grow = mx > m_ref + AT_RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY);
                float alpha = 1.f;
                if (grow) {
                    if (m_ref != -INFINITY) alpha = at_exp2(m_ref - mx);
                    m_ref = mx;
                }
                l_run *= alpha;
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                const uint64_t scale2 = at_pack2(p.scale_log2, p.scale_log2), shift2 = at_pack2(-m_use, -m_use);
                uint64_t l2[4] = {0ull, 0ull, 0ull, 0ull};          // four pairs of partial sums
                // P over this row's own scores, which are all in registers; sixteen columns are stored
                // while the next sixteen are computed
#pragma unroll
                for (int c = 0; c < 64; c += 16) {
                    uint32_t w[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float x0, x1;
                        at_unpack2(at_fma2(at_pack2(__uint_as_float(sr[2 * (c + j)]), __uint_as_float(sr[2 * (c + j) + 1])), scale2, shift2), x0, x1);
                        const float e0 = at_exp2(x0), e1 = at_exp2(x1);
                        l2[j & 3] = at_add2(l2[j & 3], at_pack2(e0, e1));
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
                        w[j] = *reinterpret_cast<uint32_t *>(&b2);
                    }
                    tc_st16(s_addr + c, w);
                }
                {
                    float a0, a1;
                    at_unpack2(at_add2(at_add2(l2[0], l2[1]), at_add2(l2[2], l2[3])), a0, a1);
                    l_run += a0 + a1;
                }
                if (__any_sync(0xffffffffu, alpha != 1.f)) {
                    // the whole warp walks its rows' outputs (tcgen05.ld / st are warp-wide); rows whose
                    // reference stays are multiplied by one.  O_X is idle: its last product is done.
#pragma unroll
                    for (int c = 0; c < 128; c += 32) {
                        uint32_t o[32];
                        at_ld32(o_addr + c, o);
                        at_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                        tc_st16(o_addr + c, o);
                        tc_st16(o_addr + c + 16, o + 16);
                    }
                }
                tc_wait_st();
            }
            if (kbase < k_first || kbase + AT_BN > k_hi) {
                // V rows of keys outside the CTA's range become zero before this row tile's product
                // reads them (both row tiles write the same zeros: either may be the only one at a tile)
                if (ok && !mbar_wait(bar(B_V_FULL + b), (uint32_t)(t >> 1) & 1u)) { atomicExch(&g_at_error, 8); ok = false; }
                const int lo_rows = max(0, k_first - kbase), hi_row = min(AT_BN, k_hi - kbase);
                for (int idx = r; idx < AT_BN * 16; idx += 128) {
                    int row = idx >> 4, c = idx & 15;
                    if (row < lo_rows || row >= hi_row)
                        *reinterpret_cast<uint4 *>(v_ptr + b * TILE_BYTES + (c >> 3) * AT_PANEL + row * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // zeroed V rows -> tensor-core reads
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_P_FULL + x));
        }

        // the last product of this row tile
        if (n_tiles_x > 0 && ok && !mbar_wait(bar(B_PV_DONE + x), (uint32_t)(n_tiles_x - 1) & 1u)) { atomicExch(&g_at_error, 9); ok = false; }
        tc_fence_after();
        if (warp_has_rows) {
            const bool write = row_ok && ok;
            int row = row0 + x * AT_BM + r;
            size_t qrow = write ? (size_t)(tok_begin + row / G) * p.nq + kvh * G + row % G : 0;
            const float inv = p.slices > 1 ? 1.f : 1.0f / l_run;
#pragma unroll
            for (int c = 0; c < 128; c += 32) {
                uint32_t o[32];
                if (n_tiles_x > 0) {
                    at_ld32(o_addr + c, o);             // warp-wide, whatever rows exist
                    at_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = 0u;
                }
                if (!write) continue;
                if (p.slices > 1) {
                    // this slice's unnormalised out; attention_merge_kernel combines the slices
                    float *po = p.part_o + (qrow * p.slices + slice) * AT_HD + c;
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<uint4 *>(po + j) = make_uint4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                } else {
                    __nv_bfloat16 *po = p.out + qrow * AT_HD + c;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 u;
                        __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(o[j]) * inv, __uint_as_float(o[j + 1]) * inv);
                        __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(o[j + 2]) * inv, __uint_as_float(o[j + 3]) * inv);
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[j + 4]) * inv, __uint_as_float(o[j + 5]) * inv);
                        __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(o[j + 6]) * inv, __uint_as_float(o[j + 7]) * inv);
                        u.x = *reinterpret_cast<uint32_t *>(&b0);
                        u.y = *reinterpret_cast<uint32_t *>(&b1);
                        u.z = *reinterpret_cast<uint32_t *>(&b2);
                        u.w = *reinterpret_cast<uint32_t *>(&b3);
                        *reinterpret_cast<uint4 *>(po + j) = u;
                    }
                }
            }
            if (write && p.slices > 1) {
                p.part_ml[(qrow * p.slices + slice) * 2] = m_ref;
                p.part_ml[(qrow * p.slices + slice) * 2 + 1] = l_run;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// Whether the kernel takes this head size and page size.
KESTREL_API int kestrel_attention_tc_supported(int hd, int page_size) {
    return hd == AT_HD && page_size > 0 && page_size % 8 == 0 && (AT_BN % page_size == 0 || page_size % AT_BN == 0);
}

// CTAs of this kernel that run at once: one per SM (shared memory and the 512 TMEM columns)
KESTREL_API int kestrel_attention_tc_slots(void) { return kestrel_sms(); }

// Tiles of rows_per_tile rows, up to 256 (tile_seq / tile_row0 list them), head size 128;
// cache_pages is the number of pages the cache tensors hold.  With slices > 1 (few tiles far
// into a long context) every CTA takes a slice of slice_len keys, a multiple of 128 - or of a
// length that follows the longest request at max_kv_ptr on the device - and the slices are merged in ascending order;
// part_o / part_ml are scratch of T * nq * slices * 128 and T * nq * slices * 2 floats.
KESTREL_API int kestrel_attention_tc(const void *q, const void *k_cache, const void *v_cache, void *out,
                                     float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0,
                                     int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens, const int *block_table,
                                     int table_width, int table_stride, int page_size, int cache_pages, int T, int nq, int nkv, int hd,
                                     int window, int slices, int slice_len, const int *max_kv_ptr, float scale,
                                     cudaStream_t stream) {
    if (T == 0 || tiles == 0) return 0;
    KESTREL_REQUIRE(hd == AT_HD, "attention_tc: head size %d; this kernel is built for %d", hd, AT_HD);
    KESTREL_REQUIRE(rows_per_tile >= 1 && rows_per_tile <= 2 * AT_BM, "attention_tc: tiles of %d rows; a CTA takes up to %d", rows_per_tile, 2 * AT_BM);
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_tc: %d query heads over %d kv heads", nq, nkv);
    KESTREL_REQUIRE(slices >= 1 && slice_len > 0 && slice_len % AT_BN == 0, "attention_tc: slice length %d must be a positive multiple of %d", slice_len, AT_BN);
    KESTREL_REQUIRE(slices == 1 || (part_o && part_ml), "attention_tc: %d slices without scratch", slices);
    KESTREL_REQUIRE((long long)tiles * nkv < (1ll << 31) && slices <= 65535, "attention_tc: grid too large");
    KESTREL_REQUIRE(kestrel_attention_tc_supported(hd, page_size), "attention_tc: pages of %d keys; the page size must be a multiple of 8 that divides 128 or is a multiple of it", page_size);
    KESTREL_REQUIRE(cache_pages > 0 && (long long)cache_pages * nkv * page_size < (1ll << 31), "attention_tc: a cache of %d pages is beyond the 32-bit row coordinate", cache_pages);
    CUtensorMap map_k, map_v;
    const long long cache_rows = (long long)cache_pages * nkv * page_size;
    int rc = kestrel_tensor_map_bf16(&map_k, k_cache, cache_rows, AT_HD, AT_HD, page_size < AT_BN ? page_size : AT_BN);
    if (rc) return rc;
    rc = kestrel_tensor_map_bf16(&map_v, v_cache, cache_rows, AT_HD, AT_HD, page_size < AT_BN ? page_size : AT_BN);
    if (rc) return rc;
    AttnParams p = {};
    p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out; p.part_o = part_o; p.part_ml = part_ml; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
    p.cu_seqlens = cu_seqlens; p.kv_lens = kv_lens; p.block_table = block_table; p.table_width = table_width; p.table_stride = table_stride;
    p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.hd = hd; p.window = window; p.slices = slices; p.slice_len = slice_len;
    p.max_kv_ptr = max_kv_ptr;
    p.scale_log2 = scale * 1.4426950408889634f;
    size_t smem = 12 * AT_PANEL + 8 * B_COUNT + 16 + 1024;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return kestrel_fail(-3, "attention_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    kestrel_launch(attention_tc_kernel, dim3((unsigned)((long long)tiles * nkv), 1, slices), dim3(AT_THREADS), smem, stream, map_k, map_v, p, cache_pages, rows_per_tile);
    rc = kestrel_check_launch("attention_tc");
    if (rc || slices == 1) return rc;
    return kestrel_attention_merge(part_o, part_ml, out, tile_seq, tile_row0, tiles, rows_per_tile, cu_seqlens, slices, hd, nq, nkv, stream);
}

// Error word of the kernel's bounded waits: 0 = none, else the number of the wait that gave up
// (1, 2, 5, 6: issuer; 3, 4: loaders; 7, 8, 9: softmax).
// Synchronises the device and clears the word.
KESTREL_API int kestrel_attention_tc_error(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_at_error, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_at_error, &zero, sizeof(int));
    return v;
}
