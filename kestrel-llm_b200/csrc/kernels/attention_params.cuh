// Arguments shared by the tensor-core attention kernels (attention_mma.cu, attention_tc.cu).
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"

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
    const int *max_kv_ptr;          // if not null: the longest request's length on the device, from which the slice length follows (a captured step)
    int table_width;                // entries of a request's row that may be read (attention_tc.cu)
    int table_stride, page_size, nq, nkv, hd, window, slices, slice_len;
    float scale_log2;
};

// Keys per slice.  A launch recorded for replay fixes the number of slices; their length then
// follows the step's longest request, read on the device: its share of the keys rounded up to
// a multiple of 128 (a multiple of every kernel's key tile).
__device__ __forceinline__ int attn_slice_len(const AttnParams &p) {
    if (!p.max_kv_ptr) return p.slice_len;
    const int per = (*p.max_kv_ptr + p.slices - 1) / p.slices;
    const int len = (per + 127) / 128 * 128;
    return len < 128 ? 128 : len;
}

// attention_mma.cu: merges the key-range slices of the listed tiles (at most 16 rows each) into out
// (kestrel_attention_merge, declared in kestrel.h)
