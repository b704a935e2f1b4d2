// Attention of a whole step: which kernel takes which requests, how their rows are tiled and
// how key ranges are cut into slices.
//
// The reference has one attention routine per shape of work - one query (vllm_attn_head_worker,
// src/model/vllm_safetensors.c:10779), a block of a prompt's queries (st_attn_batched_packed,
// :18433) and one query of each of n requests (vllm_attn_batch_worker, :16968) - and its
// callers pick.  Here a step mixes those shapes, so the choice is made per request inside one
// call: float32 takes the plain kernel (one block per token and head, order of sums fixed per
// token); bfloat16 sends requests with at most 16 (token, head) rows per kv head - decode
// tokens - to the kernel with the TMA loader warp (head size 64 or 128) or to the KEYS mode of
// the mma.sync kernel, key ranges cut into slices so that the grid fills the GPU, and the
// others - prompt portions - to the tcgen05 kernel (head size 128) or to the ROWS mode of the
// mma.sync kernel.
//
// Everything here that names a tile size belongs to the attention kernels; the step's
// description that the engine packs (kbatch_pack) holds only generic facts - lengths, positions,
// tables - and this file derives the tile lists from its host copy, once per step, and copies
// them to the device in one small transfer.  Steps in which every request brings one token need
// no transfer: tile i is request i.
#include "common.cuh"

#include <algorithm>
#include <vector>

namespace {

constexpr int RING = 8;                  // tile lists of this many plans may be in flight
constexpr int NO_SPLIT = (1 << 30) / 128 * 128;

struct Plan {
    int group_size = 0, rows_large = 0, small_rows = 16;
    int ns = 0, nl = 0;                  // tiles of at most 16 rows; tiles of rows_large rows
    int small_kv = 0, large_kv = 0;      // longest request among each kind
    const int *small_seq = nullptr, *small_row0 = nullptr, *large_seq = nullptr, *large_row0 = nullptr;   // device
};

struct Planner {
    int max_tokens = 0, max_seqs = 0;
    long long serial = -1;
    std::vector<Plan> plans;             // of the step `serial`
    int *d_iota = nullptr, *d_zero = nullptr;
    int cap_ints = 0;                    // ints per ring slot
    int *h_ring[RING] = {}, *d_ring[RING] = {};
    cudaEvent_t copied[RING] = {};
    bool used[RING] = {};
    int turn = 0;
    float *scratch = nullptr;
    size_t scratch_bytes = 0;
    // Device memory that was outgrown.  A launch recorded for replay keeps the addresses it was
    // recorded with, so nothing a recorded launch may name is freed before the planner goes.
    std::vector<void *> retired;
    int last_launches = 0;
    long long h2d_bytes = 0;
};

int grow_ring(Planner &pl, int ints) {
    cudaDeviceSynchronize();
    for (int i = 0; i < RING; ++i) {
        if (pl.h_ring[i]) cudaFreeHost(pl.h_ring[i]);
        if (pl.d_ring[i]) cudaFree(pl.d_ring[i]);       // tile lists are never named by a recorded launch
        pl.h_ring[i] = pl.d_ring[i] = nullptr;
        pl.used[i] = false;
    }
    pl.cap_ints = ints;
    for (int i = 0; i < RING; ++i) {
        if (cudaMallocHost(&pl.h_ring[i], sizeof(int) * (size_t)ints) != cudaSuccess ||
            cudaMalloc(&pl.d_ring[i], sizeof(int) * (size_t)ints) != cudaSuccess)
            return kestrel_fail(-3, "attention planner: no memory for tile lists of %d entries", ints);
    }
    return 0;
}

// the lists "tile i is request i, first row 0" for up to `seqs` requests
int grow_identity(Planner &pl, int seqs, cudaStream_t stream) {
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    if (stream) cudaStreamIsCapturing(stream, &status);
    if (status != cudaStreamCaptureStatusNone)
        return kestrel_fail(-2, "attention planner: %d requests in a recorded step, made for %d; run the step once unrecorded first", seqs / 2, pl.max_seqs);
    std::vector<int> iota(seqs);
    for (int i = 0; i < seqs; ++i) iota[i] = i;
    int *d_iota = nullptr, *d_zero = nullptr;
    if (cudaMalloc(&d_iota, sizeof(int) * (size_t)seqs) != cudaSuccess || cudaMalloc(&d_zero, sizeof(int) * (size_t)seqs) != cudaSuccess ||
        cudaMemcpy(d_iota, iota.data(), sizeof(int) * (size_t)seqs, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemset(d_zero, 0, sizeof(int) * (size_t)seqs) != cudaSuccess)
        return kestrel_fail(-3, "attention planner: no memory for the lists of %d requests", seqs);
    if (pl.d_iota) pl.retired.push_back(pl.d_iota);
    if (pl.d_zero) pl.retired.push_back(pl.d_zero);
    pl.d_iota = d_iota;
    pl.d_zero = d_zero;
    pl.max_seqs = seqs;
    return 0;
}

// tile lists of this step for mixers with `gs` query heads per kv head and tiles of `rl` rows
// Requests of at most 16 rows are one small tile each.  A short portion (at most small_rows rows,
// where small_rows > 16) is cut into small tiles too while its keys are few enough: the kernel for
// decode tokens has a lower floor than the one for prompt portions, but every tile of 16 rows reads
// the request's keys again (measured inside steps of 36 layers, new tokens / keys before them:
// 16 / 0 3.78 -> 3.44 ms, 16 / 1,024 4.40 -> 3.65, 16 / 4,096 4.01 -> 3.86, 64 / 1,024 4.92 -> 4.30,
// 64 / 2,048 4.77 -> 4.61, 128 / 0 4.88 -> 4.46, 128 / 1,024 5.58 -> 5.01; the portion kernel wins at
// 32 / 4,096 4.36 against 4.50, 64 / 4,096 4.93 against 5.21, 128 / 2,048 5.47 against 5.59, and
// from 256 tokens on).  g_small_portion_scale stretches the limits (0: no short portion goes there).
int g_small_portion_scale = 100;       // per cent
inline bool small_request(long long rows, int kv, int small_rows) {
    if (rows <= 16) return true;
    if (rows > small_rows) return false;
    const long long limit = rows <= 64 ? 4352 : rows <= 256 ? 2304 : 1664;
    return (long long)kv * 100 <= limit * g_small_portion_scale;
}

}  // namespace
KESTREL_API void kestrel_attention_set_small_portions(int per_cent) { g_small_portion_scale = per_cent >= 0 ? per_cent : 100; }
namespace {
int plan_for(Planner &pl, long long serial, const int *host, const int *dev, const int *layout, int gs, int rl, int small_rows,
             bool captured, cudaStream_t stream, const Plan **out) {
    if (serial != pl.serial) {
        pl.plans.clear();
        pl.serial = serial;
    }
    for (const Plan &p : pl.plans)
        if (p.group_size == gs && p.rows_large == rl && p.small_rows == small_rows) { *out = &p; return 0; }
    const int n = layout[KB_NUM_SEQS];
    const int *cu = host + layout[KB_O_CU_SEQLENS];
    const int *kv = host + layout[KB_O_KV_LENS];
    Plan p;
    p.group_size = gs;
    p.rows_large = rl;
    p.small_rows = small_rows;
    if ((long long)layout[KB_MAX_COUNT] * gs <= 16) {
        // every request fits one tile of 16 rows: tile i is request i, first row 0
        if (n > pl.max_seqs) {
            int rc = grow_identity(pl, 2 * n, stream);
            if (rc) return rc;
        }
        p.ns = n;
        p.small_seq = pl.d_iota;
        p.small_row0 = pl.d_zero;
        p.small_kv = layout[KB_MAX_KV_LEN];
        pl.plans.push_back(p);
        *out = &pl.plans.back();
        return 0;
    }
    if (captured) return kestrel_fail(-2, "attention planner: a step recorded for replay may hold only requests of at most 16 rows per kv head");
    std::vector<int> ss, sr, ls, lr;
    for (int i = 0; i < n; ++i) {
        const long long rows = (long long)(cu[i + 1] - cu[i]) * gs;
        if (small_request(rows, kv[i], small_rows)) {
            for (long long r0 = 0; r0 < rows; r0 += 16) {
                ss.push_back(i);
                sr.push_back((int)r0);
            }
            p.small_kv = std::max(p.small_kv, kv[i]);
        } else {
            for (long long r0 = 0; r0 < rows; r0 += rl) {
                ls.push_back(i);
                lr.push_back((int)r0);
            }
            p.large_kv = std::max(p.large_kv, kv[i]);
        }
    }
    p.ns = (int)ss.size();
    p.nl = (int)ls.size();
    const int ints = 2 * (p.ns + p.nl);
    if (ints > pl.cap_ints) {
        int rc = grow_ring(pl, std::max(ints * 2, 1024));
        if (rc) return rc;
    }
    const int slot = pl.turn;
    pl.turn = (pl.turn + 1) % RING;
    if (pl.used[slot]) cudaEventSynchronize(pl.copied[slot]);      // the copy that read this staging buffer has run
    int *h = pl.h_ring[slot];
    int at = 0;
    auto put = [&](const std::vector<int> &v) { std::copy(v.begin(), v.end(), h + at); at += (int)v.size(); };
    put(ss); put(sr); put(ls); put(lr);
    int *d = pl.d_ring[slot];
    if (cudaMemcpyAsync(d, h, sizeof(int) * (size_t)ints, cudaMemcpyHostToDevice, stream) != cudaSuccess)
        return kestrel_fail(-3, "attention planner: copy of the tile lists failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaEventRecord(pl.copied[slot], stream);
    pl.used[slot] = true;
    pl.h2d_bytes += (long long)sizeof(int) * ints;
    p.small_seq = d;
    p.small_row0 = d + p.ns;
    p.large_seq = d + 2 * p.ns;
    p.large_row0 = d + 2 * p.ns + p.nl;
    pl.plans.push_back(p);
    *out = &pl.plans.back();
    return 0;
}

// scratch for `slices` slices of T * nq rows: normalised outputs, then (maximum, sum) pairs
int slice_scratch(Planner &pl, int T, int nq, int hd, int slices, cudaStream_t stream, float **part_o, float **part_ml) {
    const size_t rows = (size_t)T * nq * slices;
    const size_t need = rows * (size_t)(hd + 2) * sizeof(float);
    if (need > pl.scratch_bytes) {
        // memory cannot be had while a stream records; a step that is to be recorded runs once unrecorded first
        cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(stream, &status);
        if (status != cudaStreamCaptureStatusNone) return kestrel_fail(-2, "attention planner: %zu bytes of slice scratch are needed while a step is recorded; run the step once unrecorded first", need);
        if (pl.scratch) pl.retired.push_back(pl.scratch);
        pl.scratch = nullptr;
        pl.scratch_bytes = 0;
        const size_t want = need + need / 2;
        if (cudaMalloc(&pl.scratch, want) != cudaSuccess) return kestrel_fail(-3, "attention planner: no memory for %zu bytes of slice scratch", want);
        pl.scratch_bytes = want;
    }
    *part_o = pl.scratch;
    *part_ml = pl.scratch + rows * (size_t)hd;
    return 0;
}

int round_up(int a, int b) { return (a + b - 1) / b * b; }
int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace

KESTREL_API void *kestrel_attn_planner_create(int max_tokens, int max_seqs) {
    if (max_tokens <= 0 || max_seqs <= 0) { kestrel_fail(-2, "attention planner: bad sizes"); return nullptr; }
    Planner *pl = new Planner();
    pl->max_tokens = max_tokens;
    pl->max_seqs = max_seqs;
    bool ok = grow_identity(*pl, max_seqs, nullptr) == 0;
    for (int i = 0; ok && i < RING; ++i) ok = cudaEventCreateWithFlags(&pl->copied[i], cudaEventDisableTiming) == cudaSuccess;
    if (ok) ok = grow_ring(*pl, std::max(1024, 2 * (2 * max_seqs + max_tokens / 4))) == 0;
    if (!ok) {
        kestrel_fail(-3, "attention planner: cannot allocate its buffers: %s", cudaGetErrorString(cudaGetLastError()));
        kestrel_attn_planner_destroy(pl);
        return nullptr;
    }
    return pl;
}

KESTREL_API void kestrel_attn_planner_destroy(void *planner) {
    Planner *pl = (Planner *)planner;
    if (!pl) return;
    cudaDeviceSynchronize();
    for (int i = 0; i < RING; ++i) {
        if (pl->h_ring[i]) cudaFreeHost(pl->h_ring[i]);
        if (pl->d_ring[i]) cudaFree(pl->d_ring[i]);
        if (pl->copied[i]) cudaEventDestroy(pl->copied[i]);
    }
    if (pl->d_iota) cudaFree(pl->d_iota);
    if (pl->d_zero) cudaFree(pl->d_zero);
    if (pl->scratch) cudaFree(pl->scratch);
    for (void *p : pl->retired) cudaFree(p);
    delete pl;
}

KESTREL_API int kestrel_attn_planner_last_launches(void *planner) { return planner ? ((Planner *)planner)->last_launches : 0; }

KESTREL_API int kestrel_attention(void *planner, long long step_serial, const int *batch_host, const int *batch_dev,
                                  const int *layout, int group, int captured, const void *q, const void *k_cache,
                                  const void *v_cache, void *out, int dtype, int cache_pages, int page_size, int nq, int nkv,
                                  int hd, int window, float scale, kestrel_stream_t stream) {
    KESTREL_REQUIRE(batch_host && batch_dev && layout, "attention: no step description");
    const int T = layout[KB_NUM_TOKENS], n = layout[KB_NUM_SEQS], W = layout[KB_TABLE_WIDTH];
    KESTREL_REQUIRE(group >= 0 && group < layout[KB_NUM_GROUPS], "attention: cache group %d of %d", group, layout[KB_NUM_GROUPS]);
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention: %d query heads over %d kv heads", nq, nkv);
    const int *positions = batch_dev + layout[KB_O_POSITIONS];
    const int *seq_of_token = batch_dev + layout[KB_O_SEQ_OF_TOKEN];
    const int *cu_seqlens = batch_dev + layout[KB_O_CU_SEQLENS];
    const int *kv_lens = batch_dev + layout[KB_O_KV_LENS];
    const int *table = batch_dev + layout[KB_O_TABLES] + (size_t)group * n * W;
    const int *max_kv_dev = batch_dev + layout[KB_O_MAX_KV];
    Planner *pl = (Planner *)planner;
    if (pl) pl->last_launches = 0;
    if (T == 0) return 0;
    if (dtype != KESTREL_BF16 || hd % 8 || hd > 256) {
        if (pl) pl->last_launches = 1;
        return kestrel_attention_plain(q, k_cache, v_cache, positions, seq_of_token, table, W, page_size, out, dtype, T, nq, nkv, hd,
                                       window, scale, stream);
    }
    KESTREL_REQUIRE(pl, "attention: the tensor-core kernels need a planner");
    const int gs = nq / nkv;
    const bool use_tc = kestrel_attention_tc_supported(hd, page_size) != 0;
    // The tcgen05 kernel takes two row tiles of 128 a CTA, so that the tensor cores work on one
    // while the other is in its softmax.  Few rows leave SMs idle, one CTA per SM.  Where the keys
    // are many the key range is cut into slices instead, as many as fill the SMs once, of at least
    // 512 keys each, merged through scratch (a warp a row; measured alone, 4,096 keys of context:
    // 512 tokens 86.7 -> 61.1 us with 2 slices, 256 tokens 81.6 -> 36.2 with 4, 64 tokens 78.7 ->
    // 24.6 with 8; more CTAs than SMs lose again).  Where the keys are too few to cut, one row
    // tile a CTA and twice the CTAs is the faster form (512 tokens from position 0: 20.2 -> 15.7 us;
    // behind 1,024 keys 36.8 -> 31.2).
    int rows_large = use_tc ? 256 : kestrel_attention_mma_rows_per_tile(hd);
    int tc_slices = 1;
    const bool use_decode = kestrel_attention_decode_supported(hd, page_size) && gs <= 16;
    int small_rows = use_decode ? 512 : 16;
    if (small_rows > 16) {
        // short portions go to the kernel for decode tokens only while all its CTAs are resident at
        // once: its gain is its low floor, and thousands of 16-row CTAs lose to tiles of 128 rows
        // (sixteen portions of 128 tokens: 27.8 against 26.2 ms a step)
        const int *cu_h = batch_host + layout[KB_O_CU_SEQLENS], *kv_h = batch_host + layout[KB_O_KV_LENS];
        long long tiles16 = 0;
        for (int i = 0; i < n; ++i) {
            const long long r = (long long)(cu_h[i + 1] - cu_h[i]) * gs;
            if (small_request(r, kv_h[i], small_rows)) tiles16 += (r + 15) / 16;
        }
        if (tiles16 * nkv > kestrel_attention_decode_slots(hd)) small_rows = 16;
    }
    if (use_tc) {
        // the portions of this step that go to this kernel: their rows, their tiles of 256, their longest context
        const int *cu_h = batch_host + layout[KB_O_CU_SEQLENS], *kv_h = batch_host + layout[KB_O_KV_LENS];
        long long rows = 0, tiles256 = 0;
        int kv = 0;
        for (int i = 0; i < n; ++i) {
            const long long r = (long long)(cu_h[i + 1] - cu_h[i]) * gs;
            if (small_request(r, kv_h[i], small_rows)) continue;
            rows += r;
            tiles256 += (r + 255) / 256;
            kv = std::max(kv, kv_h[i]);
        }
        const int sms = kestrel_attention_tc_slots();
        const int cand = window > 0 ? 1 : (int)std::min<long long>(std::min<long long>(sms / std::max<long long>(1, tiles256 * nkv), kv / 512), 16);
        if (cand >= 2 && (cand > 2 || kv >= 2048)) tc_slices = cand;
        else if (rows * nkv <= 128ll * sms) rows_large = 128;
    }
    const Plan *plan = nullptr;
    int rc = plan_for(*pl, step_serial, batch_host, batch_dev, layout, gs, rows_large, small_rows, captured != 0, stream, &plan);
    if (rc) return rc;
    int launches = 0;
    if (plan->ns > 0) {
        // Decode tokens.  As many slices as still let every CTA be resident at once (measured at
        // batch 1 to 64, contexts 2,048 to 65,536: a second wave of CTAs costs more than longer
        // slices), at least 128 keys a slice (256 for the mma.sync kernel), at most 32.  A window
        // is short; only full-length key ranges are cut.  The decode kernel merges up to 4 slices
        // inside a cluster, more through scratch and a second kernel of a few microseconds
        // (measured, one request: 8,192 keys 21.7 us with 8 slices, 12.2 us with 32).
        int slices = 1, slice_len = NO_SPLIT;
        if (window <= 0) {
            const int slots = use_decode ? kestrel_attention_decode_slots(hd) : kestrel_attention_mma_slots(hd);
            const int ctas = std::max(1, plan->ns * nkv);
            const int max_kv = std::max(1, plan->small_kv);
            const int cand = std::max(1, std::min(std::min(slots / ctas, ceil_div(max_kv, use_decode ? 128 : 256)), 32));
            slice_len = round_up(ceil_div(max_kv, cand), 128);
            slices = ceil_div(max_kv, slice_len);
            if (slices <= 1) { slices = 1; slice_len = NO_SPLIT; }
        }
        float *part_o = nullptr, *part_ml = nullptr;
        const bool needs_scratch = slices > (use_decode ? kestrel_attention_decode_cluster_slices() : 1);
        if (needs_scratch) {
            rc = slice_scratch(*pl, T, nq, hd, slices, stream, &part_o, &part_ml);
            if (rc) return rc;
        }
        const int *follow = (captured && slices > 1) ? max_kv_dev : nullptr;
        if (use_decode)
            rc = kestrel_attention_decode(q, k_cache, v_cache, out, part_o, part_ml, plan->small_seq, plan->small_row0, plan->ns,
                                          cu_seqlens, kv_lens, table, W, W, page_size, cache_pages, T, nq, nkv, hd, window, slices,
                                          slice_len, follow, scale, stream);
        else
            rc = kestrel_attention_mma(q, k_cache, v_cache, out, part_o, part_ml, plan->small_seq, plan->small_row0, plan->ns, 16,
                                       cu_seqlens, kv_lens, table, W, page_size, T, nq, nkv, hd, window, slices, slice_len, follow,
                                       scale, stream);
        if (rc) return rc;
        launches += needs_scratch ? 2 : 1;
    }
    if (plan->nl > 0) {
        if (use_tc) {
            // the number of slices was chosen above, with the tile size; here it is fitted to the
            // longest request among the portions
            int slices = 1, slice_len = NO_SPLIT;
            if (tc_slices > 1 && plan->large_kv >= 1024) {
                slice_len = round_up(ceil_div(plan->large_kv, tc_slices), 128);
                slices = ceil_div(plan->large_kv, slice_len);
                if (slices <= 1) { slices = 1; slice_len = NO_SPLIT; }
            }
            float *part_o = nullptr, *part_ml = nullptr;
            if (slices > 1) {
                rc = slice_scratch(*pl, T, nq, hd, slices, stream, &part_o, &part_ml);
                if (rc) return rc;
            }
            rc = kestrel_attention_tc(q, k_cache, v_cache, out, part_o, part_ml, plan->large_seq, plan->large_row0, plan->nl, rows_large,
                                      cu_seqlens, kv_lens, table, W, W, page_size, cache_pages, T, nq, nkv, hd, window, slices,
                                      slice_len, nullptr, scale, stream);
            launches += slices > 1 ? 2 : 1;
        } else {
            rc = kestrel_attention_mma(q, k_cache, v_cache, out, nullptr, nullptr, plan->large_seq, plan->large_row0, plan->nl, rows_large,
                                       cu_seqlens, kv_lens, table, W, page_size, T, nq, nkv, hd, window, 1, NO_SPLIT, nullptr, scale,
                                       stream);
            launches += 1;
        }
        if (rc) return rc;
    }
    pl->last_launches = launches;
    return 0;
}
