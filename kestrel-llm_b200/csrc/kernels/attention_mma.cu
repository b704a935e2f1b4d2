// Causal attention of bfloat16 queries over the paged cache on the tensor cores
// (mma.sync.m16n8k16, float32 softmax statistics and accumulators), for prompt portions and
// for decode tokens, with the key range optionally split over CTAs.
//
// Rows of work are (token, query head of one kv group) pairs of one request's tokens in this
// step, flattened token-major: row r is token r / G, head r % G (G = query heads per kv head),
// so the G heads that share a kv head read its keys and values once.  A CTA takes a tile of
// rows of one (request, kv head) and a slice of the key range:
//   * ROWS mode (tile of 128 rows, 64 for head sizes above 128): each of the 4 warps owns 32
//     (16) rows and walks all keys of the slice in tiles of 64 - prompt portions;
//   * KEYS mode (tile of 16 rows): all warps share the 16 rows, each takes 16 keys of every
//     64-key tile, and the four running (max, sum, out) states are merged in warp order at
//     the end - decode tokens, where rows are few and keys many.
// K and V tiles go from the cache pages (through the block table) to shared memory with
// cp.async, double buffered; fragments come from ldmatrix.  Key tiles are anchored at
// multiples of 64 of the absolute position, so the order of sums for a row depends on its
// position and on the slice length only.  With more than one slice each CTA writes its
// unnormalised out, max and sum to scratch and attention_merge_kernel combines the slices in
// ascending order.  Formulas as in attention_plain.cu (reference: st.c:10779-10911,
// st.c:9762-9859); exp is taken as exp2 of the score scaled by log2(e).
//
// Head sizes up to 256 in any multiple of 8; the kernel is instantiated for 32, 64, 128 and 256
// and a smaller head is padded with zero columns in shared memory.
#include "common.cuh"
#include <math.h>

#define AM_THREADS 128
#define AM_BN 64            // keys per tile
#ifndef AM_KEYS_STAGES
#define AM_KEYS_STAGES 3     // cp.async stages of the KEYS (decode) mode
#endif
#define AM_ROWS_MT 2        // 16-row tiles per warp in ROWS mode (head sizes up to 128): a tile of 128 rows per CTA

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

#include "attention_params.cuh"
#include "mma_sync.cuh"

template <int HD, bool KEYS_MODE, int MT>
__global__ void __launch_bounds__(AM_THREADS)
attention_mma_kernel(const AttnParams p) {
    pdl_launch_dependents();
    pdl_wait();
    static_assert(!KEYS_MODE || MT == 1, "KEYS mode has one 16-row tile");
    constexpr int BM = KEYS_MODE ? 16 : 64 * MT;       // ROWS mode: each warp owns MT tiles of 16 rows
    constexpr int LDS = HD + 8;                       // padded row, in elements: ldmatrix without bank conflicts
    constexpr int KS = HD / 16;                       // k-steps of the QK product
    constexpr int NT_S = KEYS_MODE ? 2 : 8;           // 8-key tiles of a warp's score block
    constexpr int NT_O = HD / 8;                      // 8-dim tiles of the output
    constexpr int STAGES = KEYS_MODE ? AM_KEYS_STAGES : 2;   // decode is bound by HBM latency: more tiles in flight
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16 *Qs = reinterpret_cast<__nv_bfloat16 *>(smem_raw);
    __nv_bfloat16 *Ks = Qs + BM * LDS;                // [STAGES][AM_BN][LDS]
    __nv_bfloat16 *Vs = Ks + STAGES * AM_BN * LDS;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, kvh = blockIdx.y, slice = blockIdx.z;
    const int seq = p.tile_seq[tile], row0 = p.tile_row0[tile];
    const int G = p.nq / p.nkv, hd = p.hd;
    const int tok_begin = p.cu_seqlens[seq], n_tok = p.cu_seqlens[seq + 1] - tok_begin;
    const int kv_len = p.kv_lens[seq];
    const int pos_begin = kv_len - n_tok;             // position of the request's first token of this step
    const int n_rows = n_tok * G;
    const int rows_here = min(BM, n_rows - row0);
    const int *table = p.block_table + (size_t)seq * p.table_stride;
    const int slice_len = attn_slice_len(p);

    // key range of this CTA: what its rows may see, cut to the slice, on 64-key tile boundaries
    const int first_tok = row0 / G, last_tok = (row0 + rows_here - 1) / G;
    int k_hi = pos_begin + last_tok + 1;              // exclusive
    int k_lo = p.window > 0 ? max(0, pos_begin + first_tok - p.window + 1) : 0;
    k_lo = max(k_lo, slice * slice_len);
    k_hi = min(k_hi, (slice + 1) * slice_len);
    const int k_first = k_lo;                         // keys before it are never read: their page may be gone
    k_lo = (k_lo / AM_BN) * AM_BN;
    const int n_tiles = k_hi > k_lo ? (k_hi - k_lo + AM_BN - 1) / AM_BN : 0;

    // ---- loads -------------------------------------------------------------------------
    constexpr int CHUNKS = HD / 8;                    // 16-byte chunks of a padded row
    constexpr int RPT = AM_BN * CHUNKS / AM_THREADS;  // a thread copies chunk ld_c of RPT consecutive keys
    const int ld_c = tid % CHUNKS, ld_r0 = (tid / CHUNKS) * RPT;
    const bool one_page = p.page_size % RPT == 0;     // the RPT keys then lie in one page: one table lookup
    // The page of a tile's keys is looked up one iteration before the copies that need it are
    // issued, so that the latency of that (dependent) load is not on the loop's critical path.
    auto lookup_page = [&](int t) -> int {
        int s0 = k_lo + t * AM_BN + ld_r0;
        if (one_page && t < n_tiles && s0 + RPT > k_first && s0 < k_hi) return table[s0 / p.page_size];
        return 0;
    };
    auto load_kv_tile = [&](int t, int stage, int page) {
        int s0 = k_lo + t * AM_BN + ld_r0;
        __nv_bfloat16 *dk = Ks + ((size_t)stage * AM_BN + ld_r0) * LDS + ld_c * 8;
        __nv_bfloat16 *dv = Vs + ((size_t)stage * AM_BN + ld_r0) * LDS + ld_c * 8;
        bool col_ok = ld_c * 8 < hd;
        size_t page_off = (((size_t)page * p.nkv + kvh) * p.page_size + (s0 % p.page_size)) * hd + ld_c * 8;
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
            int s = s0 + j;
            bool valid = col_ok && s >= k_first && s < k_hi;
            size_t off = 0;
            if (valid) {
                if (one_page) {
                    off = page_off + (size_t)j * hd;
                } else {
                    int page = table[s / p.page_size];
                    off = (((size_t)page * p.nkv + kvh) * p.page_size + (s % p.page_size)) * hd + ld_c * 8;
                }
            }
            cp_async16((uint32_t)__cvta_generic_to_shared(dk + j * LDS), p.k_cache + off, valid);
            cp_async16((uint32_t)__cvta_generic_to_shared(dv + j * LDS), p.v_cache + off, valid);
        }
    };
    for (int idx = tid; idx < BM * CHUNKS; idx += AM_THREADS) {
        int r = idx / CHUNKS, c = idx % CHUNKS;
        bool valid = r < rows_here && c * 8 < hd;
        size_t off = 0;
        if (valid) {
            int row = row0 + r;
            int tok = tok_begin + row / G, head = kvh * G + row % G;
            off = ((size_t)tok * p.nq + head) * hd + c * 8;
        }
        cp_async16((uint32_t)__cvta_generic_to_shared(Qs + r * LDS + c * 8), p.q + off, valid);
    }
    for (int st = 0; st < STAGES - 1; ++st) {          // Q travels with the first group
        if (st < n_tiles) load_kv_tile(st, st, lookup_page(st));
        cp_async_commit();
    }
    int next_page = lookup_page(STAGES - 1);

    // ---- per-thread state ----------------------------------------------------------------
    // a warp's rows: ROWS mode rows 16*MT*warp.. (MT tiles of 16), KEYS mode rows 0..15 for every warp
    const int wrow0 = KEYS_MODE ? 0 : 16 * MT * warp;
    int pos_r[MT][2], lo_r[MT][2];
    int min_pos = 0x7fffffff, max_lo = 0;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            int r = wrow0 + 16 * mt + (lane >> 2) + 8 * i;     // the rows this thread holds
            bool ok = r < rows_here;
            int ps = pos_begin + (row0 + r) / G;
            pos_r[mt][i] = ok ? ps : -1;                       // an absent row sees no key
            lo_r[mt][i] = p.window > 0 ? max(0, ps - p.window + 1) : 0;
            min_pos = min(min_pos, pos_r[mt][i]);
            max_lo = max(max_lo, lo_r[mt][i]);
        }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {                   // over the warp: tiles every row sees whole need no mask
        min_pos = min(min_pos, __shfl_xor_sync(0xffffffffu, min_pos, off));
        max_lo = max(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, off));
    }
    float o[MT][NT_O][4];
    float m_r[MT][2], l_r[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int i = 0; i < NT_O; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
        m_r[mt][0] = m_r[mt][1] = -INFINITY;
        l_r[mt][0] = l_r[mt][1] = 0.f;
    }
    const bool warp_active = KEYS_MODE ? true : (wrow0 < rows_here);

    for (int t = 0; t < n_tiles; ++t) {
        int stage = t % STAGES;
        cp_async_wait<STAGES - 2>();                   // tile t has landed
        __syncthreads();                               // ... for everyone, and tile t-1 is no longer read
        if (t + STAGES - 1 < n_tiles) load_kv_tile(t + STAGES - 1, (t + STAGES - 1) % STAGES, next_page);
        cp_async_commit();
        next_page = lookup_page(t + STAGES);
        if (warp_active) {
            const int kbase = k_lo + t * AM_BN + (KEYS_MODE ? 16 * warp : 0);
            const __nv_bfloat16 *Kt = Ks + ((size_t)stage * AM_BN + (KEYS_MODE ? 16 * warp : 0)) * LDS;
            const __nv_bfloat16 *Vt = Vs + ((size_t)stage * AM_BN + (KEYS_MODE ? 16 * warp : 0)) * LDS;
            if (kbase < k_hi && kbase <= pos_begin + last_tok) {
                float s[MT][NT_S][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int i = 0; i < NT_S; ++i) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t a[MT][4];
                    // A fragments of Q: rows wrow0 + 16 mt + (lane % 16), columns 16 ks + 8 (lane / 16)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Qs + (wrow0 + 16 * mt + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8),
                                    a[mt][0], a[mt][1], a[mt][2], a[mt][3]);
#pragma unroll
                    for (int np = 0; np < NT_S / 2; ++np) {
                        uint32_t b0, b1, b2, b3;
                        // keys 16 np + (lane % 8) + 8 (lane / 16), dims 16 ks + 8 ((lane / 8) % 2)
                        ldmatrix_x4((uint32_t)__cvta_generic_to_shared(Kt + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * LDS + ks * 16 + ((lane >> 3) & 1) * 8),
                                    b0, b1, b2, b3);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            mma_bf16(s[mt][2 * np], a[mt], b0, b1);
                            mma_bf16(s[mt][2 * np + 1], a[mt], b2, b3);
                        }
                    }
                }
                // scale, mask (only on tiles that some row of the warp does not see whole), running maximum
                const bool whole = kbase >= k_first && kbase + 8 * NT_S <= k_hi && kbase + 8 * NT_S - 1 <= min_pos && kbase >= max_lo;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    float mx[2] = {-INFINITY, -INFINITY};
                    if (whole) {
#pragma unroll
                        for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float v = s[mt][nt][e] * p.scale_log2;
                                s[mt][nt][e] = v;
                                mx[e >> 1] = fmaxf(mx[e >> 1], v);
                            }
                    } else {
#pragma unroll
                        for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                int i = e >> 1;
                                int key = kbase + nt * 8 + 2 * (lane & 3) + (e & 1);
                                float v = s[mt][nt][e] * p.scale_log2;
                                bool ok = key <= pos_r[mt][i] && key >= lo_r[mt][i] && key < k_hi && key >= k_first;
                                v = ok ? v : -INFINITY;
                                s[mt][nt][e] = v;
                                mx[i] = fmaxf(mx[i], v);
                            }
                    }
                    float alpha[2], m_use[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                        float mn = fmaxf(m_r[mt][i], mx[i]);
                        m_use[i] = mn == -INFINITY ? 0.f : mn;             // a row that has seen no key yet
                        alpha[i] = fast_exp2(m_r[mt][i] - m_use[i]);       // exp2(-inf) = 0 on the first keys
                        m_r[mt][i] = mn;
                        l_r[mt][i] *= alpha[i];
                    }
#pragma unroll
                    for (int nt = 0; nt < NT_O; ++nt) {
                        o[mt][nt][0] *= alpha[0]; o[mt][nt][1] *= alpha[0];
                        o[mt][nt][2] *= alpha[1]; o[mt][nt][3] *= alpha[1];
                    }
#pragma unroll
                    for (int nt = 0; nt < NT_S; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float pv = fast_exp2(s[mt][nt][e] - m_use[e >> 1]);
                            s[mt][nt][e] = pv;
                            l_r[mt][e >> 1] += pv;
                        }
                }
                // out += P V
#pragma unroll
                for (int kk = 0; kk < NT_S / 2; ++kk) {
                    uint32_t a[MT][4];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        a[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
                        a[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
                        a[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
                        a[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
                    }
#pragma unroll
                    for (int dp = 0; dp < NT_O / 2; ++dp) {
                        uint32_t b0, b1, b2, b3;
                        // keys 16 kk + (lane % 8) + 8 ((lane / 8) % 2), dims 16 dp + 8 (lane / 16), transposed
                        ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(Vt + (kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * LDS + dp * 16 + (lane >> 4) * 8),
                                          b0, b1, b2, b3);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            mma_bf16(o[mt][2 * dp], a[mt], b0, b1);
                            mma_bf16(o[mt][2 * dp + 1], a[mt], b2, b3);
                        }
                    }
                }
            }
        }
    }
    cp_async_wait<0>();

    // row sums across the four threads of a row
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            l_r[mt][i] += __shfl_xor_sync(0xffffffffu, l_r[mt][i], 1);
            l_r[mt][i] += __shfl_xor_sync(0xffffffffu, l_r[mt][i], 2);
        }

    if (KEYS_MODE) {
        // merge the four warps' states in warp order through shared memory (reuses the K stages)
        __syncthreads();
        float *mo = reinterpret_cast<float *>(Ks);                 // [4][16][HD]
        float *mml = mo + 4 * 16 * HD;                             // [4][16][2]
#pragma unroll
        for (int nt = 0; nt < NT_O; ++nt) {
            int d = nt * 8 + 2 * (lane & 3);
            *reinterpret_cast<float2 *>(mo + ((size_t)warp * 16 + (lane >> 2)) * HD + d) = make_float2(o[0][nt][0], o[0][nt][1]);
            *reinterpret_cast<float2 *>(mo + ((size_t)warp * 16 + (lane >> 2) + 8) * HD + d) = make_float2(o[0][nt][2], o[0][nt][3]);
        }
        if ((lane & 3) == 0) {
            mml[(warp * 16 + (lane >> 2)) * 2] = m_r[0][0];
            mml[(warp * 16 + (lane >> 2)) * 2 + 1] = l_r[0][0];
            mml[(warp * 16 + (lane >> 2) + 8) * 2] = m_r[0][1];
            mml[(warp * 16 + (lane >> 2) + 8) * 2 + 1] = l_r[0][1];
        }
        __syncthreads();
        // thread -> (row, 8-dim group): 16 rows x HD/8 groups
        for (int idx = tid; idx < 16 * (HD / 8); idx += AM_THREADS) {
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
            int tok = tok_begin + row / G, head = kvh * G + row % G;
            size_t qrow = (size_t)tok * p.nq + head;
            if (p.slices > 1) {
                float *po = p.part_o + (qrow * p.slices + slice) * hd;
#pragma unroll
                for (int j = 0; j < 8; ++j) if (d0 + j < hd) po[d0 + j] = acc[j];
                if (d0 == 0) { p.part_ml[(qrow * p.slices + slice) * 2] = M; p.part_ml[(qrow * p.slices + slice) * 2 + 1] = L; }
            } else {
                float inv = 1.0f / L;
                __nv_bfloat16 *po = p.out + qrow * hd;
#pragma unroll
                for (int j = 0; j < 8; ++j) if (d0 + j < hd) po[d0 + j] = __float2bfloat16_rn(acc[j] * inv);
            }
        }
    } else {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                int r = wrow0 + 16 * mt + (lane >> 2) + 8 * i;
                if (r >= rows_here) continue;
                int row = row0 + r;
                int tok = tok_begin + row / G, head = kvh * G + row % G;
                size_t qrow = (size_t)tok * p.nq + head;
                if (p.slices > 1) {
                    float *po = p.part_o + (qrow * p.slices + slice) * hd;
#pragma unroll
                    for (int nt = 0; nt < NT_O; ++nt) {
                        int d = nt * 8 + 2 * (lane & 3);
                        if (d < hd) { po[d] = o[mt][nt][2 * i]; po[d + 1] = o[mt][nt][2 * i + 1]; }
                    }
                    if ((lane & 3) == 0) { p.part_ml[(qrow * p.slices + slice) * 2] = m_r[mt][i]; p.part_ml[(qrow * p.slices + slice) * 2 + 1] = l_r[mt][i]; }
                } else {
                    float inv = 1.0f / l_r[mt][i];
                    __nv_bfloat16 *po = p.out + qrow * hd;
#pragma unroll
                    for (int nt = 0; nt < NT_O; ++nt) {
                        int d = nt * 8 + 2 * (lane & 3);
                        if (d < hd) *reinterpret_cast<__nv_bfloat162 *>(po + d) = __floats2bfloat162_rn(o[mt][nt][2 * i] * inv, o[mt][nt][2 * i + 1] * inv);
                    }
                }
            }
    }
}

// out[row] = sum over slices of part_o * 2^(m - M) / sum of l * 2^(m - M), slices in ascending
// order, for the rows of the listed tiles (rows_per_tile = gridDim.z rows each at most); one
// block per (tile, kv head, row of the tile).  The slices' weights are worked out once per row into shared memory; then
// every thread adds its dims over the slices with AMG_UNROLL loads in flight (a row's slices
// are few and far apart in memory: a loop of dependent loads would cost a memory latency each).
#define AMG_THREADS 128
#define AMG_MAX_SLICES 1024
#define AMG_UNROLL 16
__global__ void __launch_bounds__(AMG_THREADS)
attention_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml,
                       __nv_bfloat16 *__restrict__ out, const int *__restrict__ tile_seq,
                       const int *__restrict__ tile_row0, const int *__restrict__ cu_seqlens,
                       int slices, int hd, int nq, int nkv) {
    pdl_launch_dependents();
    __shared__ float f_s[AMG_MAX_SLICES], lf_s[AMG_MAX_SLICES];
    __shared__ float red[AMG_THREADS / 32];
    __shared__ float inv_l;
    const int tile = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
    const int tid = threadIdx.x;
    const int seq = tile_seq[tile], row0 = tile_row0[tile];
    const int G = nq / nkv;
    const int tok_begin = cu_seqlens[seq];
    const int n_rows = (cu_seqlens[seq + 1] - tok_begin) * G;
    if (r >= min((int)gridDim.z, n_rows - row0)) return;
    const int row = row0 + r;
    const size_t qrow = (size_t)(tok_begin + row / G) * nq + kvh * G + row % G;
    const float *ml = part_ml + qrow * slices * 2;
    pdl_wait();
    float mx = -INFINITY;
    for (int s = tid; s < slices; s += AMG_THREADS) mx = fmaxf(mx, ml[2 * s]);
    mx = warp_max(mx);
    if ((tid & 31) == 0) red[tid >> 5] = mx;
    __syncthreads();
    float M = red[0];
#pragma unroll
    for (int w = 1; w < AMG_THREADS / 32; ++w) M = fmaxf(M, red[w]);
    for (int s = tid; s < slices; s += AMG_THREADS) {
        float2 v = *reinterpret_cast<const float2 *>(ml + 2 * s);
        float f = v.x == -INFINITY ? 0.f : exp2f(v.x - M);
        f_s[s] = f;
        lf_s[s] = f != 0.f ? v.y * f : 0.f;
    }
    __syncthreads();
    if (tid == 0) {             // the sum of the weights in ascending order, as the rows' own sums
        float L = 0.f;
        for (int s = 0; s < slices; ++s) L += lf_s[s];
        inv_l = L;
    }
    __syncthreads();
    const float L = inv_l;
    const float *po = part_o + qrow * slices * hd;
    for (int d = tid; d < hd; d += AMG_THREADS) {
        float acc = 0.f;
        int s = 0;
        for (; s + AMG_UNROLL <= slices; s += AMG_UNROLL) {
            float v[AMG_UNROLL];
#pragma unroll
            for (int u = 0; u < AMG_UNROLL; ++u) v[u] = po[(size_t)(s + u) * hd + d];
#pragma unroll
            for (int u = 0; u < AMG_UNROLL; ++u)
                if (f_s[s + u] != 0.f) acc += v[u] * f_s[s + u];
        }
        for (; s < slices; ++s)
            if (f_s[s] != 0.f) acc += po[(size_t)s * hd + d] * f_s[s];
        out[qrow * hd + d] = __float2bfloat16_rn(acc / L);
    }
}

// The same merge for tiles of many rows (prompt portions cut into key-range slices) and up to 32
// slices: one WARP per row, a lane per slice for the weights and four output dims a lane, every
// slice's values in flight at once; eight rows a block.  One block per row, with its three block
// barriers, took some 25 us for the 16,384 rows of a 512-token portion - more than the slices
// saved.  Slices are added in ascending order, as above.
#define AMW_MAX_SLICES 32
__global__ void __launch_bounds__(256)
attention_merge_rows_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml,
                            __nv_bfloat16 *__restrict__ out, const int *__restrict__ tile_seq,
                            const int *__restrict__ tile_row0, const int *__restrict__ cu_seqlens,
                            int slices, int hd, int nq, int nkv, int rows_per_tile) {
    pdl_launch_dependents();
    const int tile = blockIdx.x, kvh = blockIdx.y, lane = threadIdx.x & 31;
    const int r = blockIdx.z * 8 + (threadIdx.x >> 5);
    const int seq = tile_seq[tile], row0 = tile_row0[tile];
    const int G = nq / nkv;
    const int tok_begin = cu_seqlens[seq];
    const int n_rows = (cu_seqlens[seq + 1] - tok_begin) * G;
    if (r >= min(rows_per_tile, n_rows - row0)) return;
    const int row = row0 + r;
    const size_t qrow = (size_t)(tok_begin + row / G) * nq + kvh * G + row % G;
    pdl_wait();
    // lane s holds slice s: its maximum and sum
    float2 ml = lane < slices ? *reinterpret_cast<const float2 *>(part_ml + (qrow * slices + lane) * 2) : make_float2(-INFINITY, 0.f);
    const float M = warp_max(ml.x);
    const float f = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
    const float lf = f != 0.f ? ml.y * f : 0.f;
    const int d = 4 * lane;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float L = 0.f;
    const float *po = part_o + qrow * slices * hd + d;
    float4 v[AMW_MAX_SLICES / 4];
    for (int s0 = 0; s0 < slices; s0 += AMW_MAX_SLICES / 4) {        // eight slices' values in flight
#pragma unroll
        for (int u = 0; u < AMW_MAX_SLICES / 4; ++u)
            if (s0 + u < slices && d < hd) v[u] = *reinterpret_cast<const float4 *>(po + (size_t)(s0 + u) * hd);
#pragma unroll
        for (int u = 0; u < AMW_MAX_SLICES / 4; ++u) {
            if (s0 + u >= slices) break;
            const float fs = __shfl_sync(0xffffffffu, f, s0 + u);
            L += __shfl_sync(0xffffffffu, lf, s0 + u);
            if (fs != 0.f && d < hd) {
                acc.x += v[u].x * fs; acc.y += v[u].y * fs; acc.z += v[u].z * fs; acc.w += v[u].w * fs;
            }
        }
    }
    if (d < hd) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x / L, acc.y / L), hi = __floats2bfloat162_rn(acc.z / L, acc.w / L);
        uint2 u2;
        u2.x = *reinterpret_cast<uint32_t *>(&lo);
        u2.y = *reinterpret_cast<uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(out + qrow * hd + d) = u2;
    }
}

template <int HD, bool KEYS_MODE, int MT>
static int launch_attention(const AttnParams &p, int tiles, cudaStream_t stream) {
    constexpr int BM = KEYS_MODE ? 16 : 64 * MT;
    constexpr int LDS = HD + 8;
    constexpr int STAGES = KEYS_MODE ? AM_KEYS_STAGES : 2;
    size_t smem = (size_t)(BM + 2 * STAGES * AM_BN) * LDS * 2;
    static bool attr_set = false;
    if (!attr_set && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<HD, KEYS_MODE, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return kestrel_fail(-3, "attention_mma: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid(tiles, p.nkv, p.slices);
    kestrel_launch(attention_mma_kernel<HD, KEYS_MODE, MT>, dim3(grid), dim3(AM_THREADS), smem, stream, p);
    return kestrel_check_launch("attention_mma");
}

// merges the slices of the listed tiles (at most rows_per_tile rows each) into out; also used by
// attention_decode.cu and attention_tc.cu
KESTREL_API int kestrel_attention_merge(const float *part_o, const float *part_ml, void *out, const int *tile_seq,
                                        const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, int slices,
                                        int hd, int nq, int nkv, cudaStream_t stream) {
    KESTREL_REQUIRE(rows_per_tile >= 1 && rows_per_tile <= 65535, "attention_merge: tiles of %d rows", rows_per_tile);
    KESTREL_REQUIRE(slices >= 1 && slices <= AMG_MAX_SLICES, "attention_merge: %d slices; the kernel merges up to %d", slices, AMG_MAX_SLICES);
    KESTREL_REQUIRE(tiles <= 0x7fffffff && nkv <= 65535, "attention_merge: grid too large");
    if (rows_per_tile > 16 && slices <= AMW_MAX_SLICES && hd % 4 == 0 && hd <= 128 && (((uintptr_t)part_o | (uintptr_t)out) & 15) == 0) {
        kestrel_launch(attention_merge_rows_kernel, dim3(tiles, nkv, (rows_per_tile + 7) / 8), dim3(256), 0, stream, part_o, part_ml,
                       (__nv_bfloat16 *)out, tile_seq, tile_row0, cu_seqlens, slices, hd, nq, nkv, rows_per_tile);
        return kestrel_check_launch("attention_merge");
    }
    kestrel_launch(attention_merge_kernel, dim3(tiles, nkv, rows_per_tile), dim3(AMG_THREADS), 0, stream, part_o, part_ml, (__nv_bfloat16 *)out,
                   tile_seq, tile_row0, cu_seqlens, slices, hd, nq, nkv);
    return kestrel_check_launch("attention_merge");
}

// rows (token, head) of a ROWS-mode tile for this head size
KESTREL_API int kestrel_attention_mma_rows_per_tile(int hd) { return hd <= 128 ? 64 * AM_ROWS_MT : 64; }

// CTAs of the KEYS-mode kernel that the GPU's SMs hold at once, by shared memory and threads
KESTREL_API int kestrel_attention_mma_slots(int hd) {
    int HD = hd <= 32 ? 32 : hd <= 64 ? 64 : hd <= 128 ? 128 : 256;
    size_t smem = (size_t)(16 + 2 * AM_KEYS_STAGES * AM_BN) * (HD + 8) * 2 + 1024;
    int per_sm = (int)((227 * 1024) / smem);
    if (per_sm > 2048 / AM_THREADS) per_sm = 2048 / AM_THREADS;
    if (per_sm < 1) per_sm = 1;
    return kestrel_sms() * per_sm;
}

// rows_per_tile must be 16 (KEYS mode) or 64 (ROWS mode); tile_seq / tile_row0 describe the
// tiles.  part_o / part_ml are scratch for slices > 1: float32 [T * nq * slices * hd] and
// [T * nq * slices * 2].  max_kv_ptr, if given, points to the longest request's length on the
// device; the slice length then follows it instead of slice_len, so that a captured launch can
// follow the context.
KESTREL_API int kestrel_attention_mma(const void *q, const void *k_cache, const void *v_cache, void *out,
                                      float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0,
                                      int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens,
                                      const int *block_table, int table_stride, int page_size, int T, int nq,
                                      int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr,
                                      float scale, cudaStream_t stream) {
    if (T == 0 || tiles == 0) return 0;
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_mma: %d query heads over %d kv heads", nq, nkv);
    KESTREL_REQUIRE(hd > 0 && hd % 8 == 0 && hd <= 256, "attention_mma: head size %d is not a multiple of 8 up to 256", hd);
    int rows_mode_tile = hd <= 128 ? 64 * AM_ROWS_MT : 64;
    KESTREL_REQUIRE(rows_per_tile == 16 || rows_per_tile == rows_mode_tile,
                    "attention_mma: tiles of %d rows; head size %d takes 16 or %d", rows_per_tile, hd, rows_mode_tile);
    KESTREL_REQUIRE(slices >= 1 && slice_len > 0 && slice_len % AM_BN == 0, "attention_mma: slice length %d must be a positive multiple of %d", slice_len, AM_BN);
    KESTREL_REQUIRE(slices == 1 || (part_o && part_ml), "attention_mma: %d slices without scratch", slices);
    KESTREL_REQUIRE(nkv <= 65535 && slices <= 65535, "attention_mma: grid too large");
    AttnParams p;
    p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
    p.out = (__nv_bfloat16 *)out; p.part_o = part_o; p.part_ml = part_ml; p.tile_seq = tile_seq; p.tile_row0 = tile_row0;
    p.cu_seqlens = cu_seqlens; p.kv_lens = kv_lens; p.block_table = block_table; p.table_stride = table_stride;
    p.page_size = page_size; p.nq = nq; p.nkv = nkv; p.hd = hd; p.window = window; p.slices = slices; p.slice_len = slice_len;
    p.max_kv_ptr = max_kv_ptr;
    p.scale_log2 = scale * 1.4426950408889634f;
    bool keys = rows_per_tile == 16;
    int rc;
    if (hd <= 32) rc = keys ? launch_attention<32, true, 1>(p, tiles, stream) : launch_attention<32, false, AM_ROWS_MT>(p, tiles, stream);
    else if (hd <= 64) rc = keys ? launch_attention<64, true, 1>(p, tiles, stream) : launch_attention<64, false, AM_ROWS_MT>(p, tiles, stream);
    else if (hd <= 128) rc = keys ? launch_attention<128, true, 1>(p, tiles, stream) : launch_attention<128, false, AM_ROWS_MT>(p, tiles, stream);
    else rc = keys ? launch_attention<256, true, 1>(p, tiles, stream) : launch_attention<256, false, 1>(p, tiles, stream);
    if (rc) return rc;
    if (slices > 1) {
        KESTREL_REQUIRE(keys, "attention_mma: slices are merged for tiles of 16 rows only");
        return kestrel_attention_merge(part_o, part_ml, out, tile_seq, tile_row0, tiles, 16, cu_seqlens, slices, hd, nq, nkv, stream);
    }
    return 0;
}
