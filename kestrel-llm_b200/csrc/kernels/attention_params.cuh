// Arguments shared by the tensor-core attention kernels (attention_mma.cu, attention_tc.cu).
#pragma once
#include <cuda_bf16.h>

struct AttnParams {
    const __nv_bfloat16 *q;         // [T, nq * hd]
    const __nv_bfloat16 *k_cache;   // [pages, nkv, page_size, hd]
    const __nv_bfloat16 *v_cache;
    __nv_bfloat16 *out;             // [T, nq * hd]
    float *part_o;                  // [T * nq, slices, hd]   (slices > 1)
    float *part_ml;                 // [T * nq, slices, 2]
    const int *tile_seq;            // [tiles] request index of the tile
    const int *tile_row0;           // [tiles] first row (token-major, head-minor) among the request's rows
    const int *cu_seqlens;          // [nseq + 1] first token of each request in this step
    const int *kv_lens;             // [nseq] request length after this step
    const int *block_table;         // [nseq, table_stride]
    const int *slice_len_ptr;       // if not null, the slice length is read from here (a step of a captured graph)
    int table_width;                // entries of a request's row that may be read (attention_tc.cu)
    int table_stride, page_size, nq, nkv, hd, window, slices, slice_len;
    float scale_log2;
};

// attention_mma.cu: merges the key-range slices of the listed tiles (at most 16 rows each) into out
extern "C" int kestrel_attention_merge(const float *part_o, const float *part_ml, void *out, const int *tile_seq,
                                       const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, int slices,
                                       int hd, int nq, int nkv, cudaStream_t stream);
