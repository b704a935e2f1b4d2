// Checks of a step's description, as one predicate that runs on the host (tests) and on the
// device (the runner's debug guards): a token whose id, position or page would make a kernel
// index outside its tensors is named before any kernel uses it.  The reference only logs such
// an overflow ("[KV-OOB]", src/model/vllm_safetensors.c:16494-16496); its guard zones catch the
// damage afterwards (include/model/vllm_safetensors.h:32-36).
#pragma once
#include "../../include/kestrel.h"

#ifdef __CUDACC__
#define STEP_CHECK_FN __host__ __device__ inline
#else
#define STEP_CHECK_FN inline
#endif

#define STEP_CHECK_MAX_GROUPS 8

enum {
    STEP_CHECK_OK = 0,
    STEP_CHECK_TOKEN_ID = 1,      // token id outside the vocabulary
    STEP_CHECK_SEQ = 2,           // request index outside the step's requests
    STEP_CHECK_POSITION = 3,      // position negative or beyond the request's length after the step
    STEP_CHECK_TABLE_COLUMN = 4,  // position beyond the block-table row
    STEP_CHECK_PAGE = 5,          // page id outside the pool (the null page counts as inside)
    STEP_CHECK_ORDER = 6          // token outside its request's range of rows
};

struct StepCheckLayout {
    int num_tokens, num_seqs, table_width, num_groups, page_size, vocab;
    int o_token_ids, o_positions, o_seq_of_token, o_cu_seqlens, o_kv_lens, o_tables;
    int pages[STEP_CHECK_MAX_GROUPS];      // pages of each group's tensors, the null page included
};

// 0 if token t of the packed description can be placed by the kernels, else which rule it breaks
STEP_CHECK_FN int kestrel_check_token(const int *batch, const StepCheckLayout &lay, int t) {
    if (lay.vocab > 0) {
        const int id = batch[lay.o_token_ids + t];
        if (id < 0 || id >= lay.vocab) return STEP_CHECK_TOKEN_ID;
    }
    const int seq = batch[lay.o_seq_of_token + t];
    if (seq < 0 || seq >= lay.num_seqs) return STEP_CHECK_SEQ;
    if (t < batch[lay.o_cu_seqlens + seq] || t >= batch[lay.o_cu_seqlens + seq + 1]) return STEP_CHECK_ORDER;
    const int pos = batch[lay.o_positions + t];
    if (pos < 0 || pos >= batch[lay.o_kv_lens + seq]) return STEP_CHECK_POSITION;
    const int column = pos / lay.page_size;
    if (column >= lay.table_width) return STEP_CHECK_TABLE_COLUMN;
    for (int g = 0; g < lay.num_groups && g < STEP_CHECK_MAX_GROUPS; ++g) {
        // the page this token's keys and values are written to must exist in every group
        const int page = batch[lay.o_tables + (g * lay.num_seqs + seq) * lay.table_width + column];
        if (page < 0 || page >= lay.pages[g]) return STEP_CHECK_PAGE;
    }
    return STEP_CHECK_OK;
}

inline StepCheckLayout step_check_layout(const int *layout, int vocab, int page_size) {
    StepCheckLayout lay = {};
    lay.num_tokens = layout[KB_NUM_TOKENS];
    lay.num_seqs = layout[KB_NUM_SEQS];
    lay.table_width = layout[KB_TABLE_WIDTH];
    lay.num_groups = layout[KB_NUM_GROUPS];
    lay.page_size = page_size;
    lay.vocab = vocab;
    lay.o_token_ids = layout[KB_O_TOKEN_IDS];
    lay.o_positions = layout[KB_O_POSITIONS];
    lay.o_seq_of_token = layout[KB_O_SEQ_OF_TOKEN];
    lay.o_cu_seqlens = layout[KB_O_CU_SEQLENS];
    lay.o_kv_lens = layout[KB_O_KV_LENS];
    lay.o_tables = layout[KB_O_TABLES];
    return lay;
}

inline const char *step_check_text(int code) {
    switch (code) {
        case STEP_CHECK_TOKEN_ID: return "a token id outside the vocabulary";
        case STEP_CHECK_SEQ: return "a request index outside the step's requests";
        case STEP_CHECK_POSITION: return "a position outside its request";
        case STEP_CHECK_TABLE_COLUMN: return "a position beyond the block-table row";
        case STEP_CHECK_PAGE: return "a page id outside the pool";
        case STEP_CHECK_ORDER: return "a token outside its request's rows";
        default: return "no fault";
    }
}
