// The description of one step, packed for the device.
//
// A step runs a flat list of T tokens from n requests: prompt portions (several tokens of one
// request, in order) beside single decoded tokens.  Everything a kernel needs to place a token -
// its id, its position in its request, which request, that request's pages in every cache
// group - goes into ONE int32 buffer that the caller copies to the device in one transfer.  The
// reference never builds such a description: its three forward entry points each take one
// shape of work (src/model/vllm_safetensors.c:16356, :17926, :17041) and find a token's cache
// row by arithmetic on a private window (:9233-9238).
//
// Only generic facts about the step are written here.  What a particular kernel derives from
// them (tiles, slices) is made by the part that owns the kernel, from the host copy of this
// buffer.
#include <stdint.h>
#include <string.h>

#include <algorithm>

#include "../../include/kestrel.h"
#include "../kernels/step_checks.cuh"

namespace {

int needed_width(void *cache, int n, const long long *ids, const int *counts) {
    const int G = kcache_num_groups(cache);
    const int page = kcache_page_size(cache);
    int need = 1;
    for (int e = 0; e < n; ++e) {
        int len = kcache_length(cache, ids[e]);
        if (len < 0) return len;
        // blocks the request holds after its pages for this step were reserved
        need = std::max(need, (len + counts[e] + page - 1) / page);
        for (int g = 0; g < G; ++g) need = std::max(need, kcache_num_blocks(cache, ids[e], g));
    }
    return (need + 7) / 8 * 8;
}

}  // namespace

KESTREL_API int kbatch_ints_needed(void *cache, int n, const long long *ids, const int *counts, int n_wants, int table_width) {
    if (!cache || n < 0 || n_wants < 0) return -2;
    long long T = 0;
    for (int e = 0; e < n; ++e) {
        if (counts[e] <= 0) return -2;
        T += counts[e];
    }
    int W = table_width > 0 ? table_width : needed_width(cache, n, ids, counts);
    if (W < 0) return W;
    long long total = 3 * T + (n + 1) + 2ll * n + n_wants + 1 + (long long)kcache_num_groups(cache) * n * W;
    return total > INT32_MAX ? -2 : (int)std::max(total, 1ll);
}

KESTREL_API int kbatch_pack(void *cache, int n, const long long *ids, const int *counts, const int *tokens,
                            const int *want_counts, const int *wants, int table_width, int *out, int cap, int *layout) {
    if (!cache || n <= 0 || !ids || !counts || !out || !layout) return -2;
    const int G = kcache_num_groups(cache);
    long long T = 0, R = 0;
    for (int e = 0; e < n; ++e) {
        if (counts[e] <= 0) return -2;
        T += counts[e];
        if (want_counts) {
            if (want_counts[e] < 0) return -2;
            R += want_counts[e];
        }
    }
    if (T > INT32_MAX / 4 || R > INT32_MAX / 4) return -2;
    int W = table_width > 0 ? table_width : needed_width(cache, n, ids, counts);
    if (W < 0) return W;
    const int o_tok = 0, o_pos = (int)T, o_seq = 2 * (int)T, o_cu = 3 * (int)T;
    const int o_kv = o_cu + n + 1, o_slot = o_kv + n, o_rows = o_slot + n, o_maxkv = o_rows + (int)R, o_tab = o_maxkv + 1;
    const long long total = (long long)o_tab + (long long)G * n * W;
    if (total > cap) return -9;
    int cu = 0, max_count = 0, max_kv = 0, row = 0, w_at = 0;
    for (int e = 0; e < n; ++e) {
        const int c = counts[e];
        const int start = kcache_length(cache, ids[e]);
        if (start < 0) return -3;
        if (tokens) memcpy(out + o_tok + cu, tokens + cu, sizeof(int) * (size_t)c);
        for (int j = 0; j < c; ++j) {
            out[o_pos + cu + j] = start + j;
            out[o_seq + cu + j] = e;
        }
        out[o_cu + e] = cu;
        out[o_kv + e] = start + c;
        out[o_slot + e] = kcache_slot(cache, ids[e]);
        const int nw = want_counts ? want_counts[e] : 0;
        for (int j = 0; j < nw; ++j) {
            const int w = wants[w_at + j];
            if (w < 0 || w >= c) return -2;
            out[o_rows + row++] = cu + w;
        }
        w_at += nw;
        for (int g = 0; g < G; ++g) {
            int blocks = kcache_block_table(cache, ids[e], g, out + o_tab + ((size_t)g * n + e) * W, W);
            if (blocks < 0) return blocks;
            if (blocks > W) return -9;
        }
        max_count = std::max(max_count, c);
        max_kv = std::max(max_kv, start + c);
        cu += c;
    }
    out[o_cu + n] = cu;
    out[o_maxkv] = max_kv;
    memset(layout, 0, sizeof(int) * KBATCH_LAYOUT_INTS);
    layout[KB_NUM_TOKENS] = (int)T;
    layout[KB_NUM_SEQS] = n;
    layout[KB_NUM_ROWS] = (int)R;
    layout[KB_TABLE_WIDTH] = W;
    layout[KB_NUM_GROUPS] = G;
    layout[KB_MAX_COUNT] = max_count;
    layout[KB_MAX_KV_LEN] = max_kv;
    layout[KB_TOTAL_INTS] = (int)total;
    layout[KB_O_TOKEN_IDS] = o_tok;
    layout[KB_O_POSITIONS] = o_pos;
    layout[KB_O_SEQ_OF_TOKEN] = o_seq;
    layout[KB_O_CU_SEQLENS] = o_cu;
    layout[KB_O_KV_LENS] = o_kv;
    layout[KB_O_SLOTS] = o_slot;
    layout[KB_O_ROWS] = o_rows;
    layout[KB_O_MAX_KV] = o_maxkv;
    layout[KB_O_TABLES] = o_tab;
    return (int)total;
}

// The predicate of the runner's debug guards, on the host: walks every token of a packed
// description and returns 0 if the kernels can place it, else (rule << 16) | (token & 0xffff)
// for the first token that breaks a rule (STEP_CHECK_* in csrc/kernels/step_checks.cuh: 1 token
// id, 2 request index, 3 position, 4 block-table column, 5 page id, 6 token outside its request's
// rows).  `pages` holds the number of pages of each group's tensors.  Tests hand this bad
// descriptions; no kernel ever sees them.
KESTREL_API int kbatch_check(const int *batch, const int *layout, int vocab, int page_size, const int *pages) {
    if (!batch || !layout || !pages || page_size <= 0) return -2;
    StepCheckLayout lay = step_check_layout(layout, vocab, page_size);
    for (int g = 0; g < lay.num_groups && g < STEP_CHECK_MAX_GROUPS; ++g) lay.pages[g] = pages[g];
    for (int t = 0; t < lay.num_tokens; ++t) {
        int code = kestrel_check_token(batch, lay, t);
        if (code) return code * 65536 + (t & 0xffff);
    }
    return 0;
}
