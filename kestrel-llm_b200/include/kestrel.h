/* kestrel.h - the C interface of the kestrel-llm_b200 engine.
 *
 * Two shared libraries export it:
 *   libkestrel_host.so  cache manager (kcache_*), scheduler (ksched_*) and the packer of a step's
 *                       description (kbatch_*): plain C++ on the host, no CUDA needed;
 *   libkestrel_cuda.so  the sm_100a kernels (kestrel_<kernel>), the attention dispatcher, the step
 *                       program and the runner behind kestrel_step_raw (kprog_*, krunner_*); it
 *                       links against libkestrel_host.so.
 * The reference's header-level interface is include/model/vllm_safetensors.h:497-670
 * (st_qwen_inference_init, st_qwen_model_forward, st_qwen_model_prefill_batch,
 * st_qwen_model_forward_batch, st_qwen_inference_free); there one state object is one request on
 * the CPU, here one runner serves all live requests of a GPU.
 *
 * Conventions
 *  - Every function is extern "C".  Functions that return int return 0 (or a count, where the
 *    text says so) on success and a negative code on failure; the kernel library keeps the text
 *    of the last failure of the calling thread in kestrel_last_error().
 *  - Kernel entry points take raw device pointers, sizes and a CUDA stream, launch on that
 *    stream and do not synchronise.  Storage type codes: 0 = float32, 1 = bfloat16.
 *  - This file is included by every source file that defines one of these symbols, so a
 *    definition that drifts from its declaration does not compile; the Python bindings take
 *    their argument types from this file too (csrc/cdecl.py).  Keep one declaration per
 *    statement, with parameter names, in the plain types used below.
 */
#ifndef KESTREL_H
#define KESTREL_H

#ifdef __cplusplus
#define KESTREL_API extern "C" __attribute__((visibility("default")))
#else
#define KESTREL_API __attribute__((visibility("default")))
#endif

/* a CUDA stream (cudaStream_t is this same pointer type) */
typedef struct CUstream_st *kestrel_stream_t;

#define KESTREL_F32 0
#define KESTREL_BF16 1

/* ============================================================================================
 * Cache manager (libkestrel_host.so): pages of keys and values per group of layers, a block
 * table per request and group, one state slot per live request.  Host bookkeeping only.
 * ========================================================================================== */
KESTREL_API void *kcache_create(int n_groups, const int *windows, const int *num_pages, int page_size, int max_requests, int max_blocks_per_request);
KESTREL_API void kcache_destroy(void *h);
/* slot of the new request; -1 no slot free; -2 the id is live already */
KESTREL_API int kcache_admit(void *h, long long id);
/* 1 if kcache_reserve(id, n_new) would succeed, 0 if pages are short, negative on misuse */
KESTREL_API int kcache_can_reserve(void *h, long long id, int n_new);
/* pages for positions [length, length + n_new) in every group: 0 done, -1 pages short (nothing changed), -3 unknown request, -4 longer than the block table */
KESTREL_API int kcache_reserve(void *h, long long id, int n_new);
/* length += n_new (must be reserved); windowed groups give back pages no later query can reach */
KESTREL_API int kcache_commit(void *h, long long id, int n_new);
/* gives back everything the request holds, and its slot */
KESTREL_API int kcache_release(void *h, long long id);
KESTREL_API int kcache_length(void *h, long long id);
KESTREL_API int kcache_slot(void *h, long long id);
KESTREL_API int kcache_num_blocks(void *h, long long id, int group);
KESTREL_API int kcache_block_table(void *h, long long id, int group, int *out, int n);
KESTREL_API int kcache_describe_decode(void *h, const long long *ids, int n, int B, int W, int *pos, int *kv, int *slot, int *tables, int *bad);
KESTREL_API int kcache_free_pages(void *h, int group);
KESTREL_API int kcache_num_pages(void *h, int group);
KESTREL_API int kcache_num_groups(void *h);
KESTREL_API int kcache_page_size(void *h);
KESTREL_API int kcache_max_blocks(void *h);
KESTREL_API int kcache_live_requests(void *h);
KESTREL_API int kcache_free_slots(void *h);
KESTREL_API long long kcache_pages_handed_out(void *h);
KESTREL_API long long kcache_pages_given_back(void *h);
/* ids of the requests admitted since the last call (their state slots are to be cleared); returns how many there were */
KESTREL_API int kcache_take_admitted(void *h, long long *ids, int *slots, int cap);
/* puts the free pages of every group into a pseudo-random order fixed by `seed` (the layout a pool has after long serving) */
KESTREL_API int kcache_shuffle_free(void *h, long long seed);
/* 0 if every page and slot is free exactly once or held exactly once, else a negative code naming the broken invariant */
KESTREL_API int kcache_check(void *h);

/* ============================================================================================
 * Scheduler (libkestrel_host.so): admission, token budget, prompt portions, decode first,
 * preempt-youngest-and-recompute when pages run out.  It counts tokens; values live with the caller.
 * ========================================================================================== */
KESTREL_API void *ksched_create(void *cache, int max_step_tokens, int prefill_chunk, int batch_max, int max_queued, int max_model_len);
KESTREL_API void ksched_destroy(void *h);
/* 0 queued; -1 waiting queue full; -2 longer than max_model_len or the whole pool; -3 empty prompt or duplicate id */
KESTREL_API int ksched_add(void *h, long long id, int prompt_len, int max_new_tokens);
/* builds the next step, pages reserved: entry e runs tokens [starts[e], starts[e] + counts[e]) of ids[e]; wants[e] = 1 if it ends with the request's last known token.  Returns the number of entries. */
KESTREL_API int ksched_schedule(void *h, long long *ids_out, int *starts_out, int *counts_out, int *wants_out, int cap);
KESTREL_API int ksched_preempted(void *h, long long *out, int cap);
KESTREL_API int ksched_step_done(void *h);
/* one more token of the request is known; 1 if it has reached its token limit */
KESTREL_API int ksched_on_token(void *h, long long id);
KESTREL_API int ksched_finish(void *h, long long id);
KESTREL_API int ksched_num_running(void *h);
KESTREL_API int ksched_num_waiting(void *h);
KESTREL_API long long ksched_num_preemptions(void *h);
KESTREL_API int ksched_known(void *h, long long id);

/* ============================================================================================
 * The description of one step (libkestrel_host.so).  A step runs T tokens of n requests: prompt
 * portions beside single decoded tokens.  kbatch_pack writes everything a kernel needs to place
 * a token into ONE int32 buffer (copied to the device in one transfer) and describes it in
 * `layout`, KBATCH_LAYOUT_INTS ints indexed by the KB_* names: counts first, then offsets
 * (in ints) of the sections.
 * ========================================================================================== */
#define KB_NUM_TOKENS 0      /* T */
#define KB_NUM_SEQS 1        /* n */
#define KB_NUM_ROWS 2        /* R: places whose logits are wanted */
#define KB_TABLE_WIDTH 3     /* W: entries per block-table row */
#define KB_NUM_GROUPS 4      /* G */
#define KB_MAX_COUNT 5       /* most tokens of one request in this step */
#define KB_MAX_KV_LEN 6      /* longest request after this step */
#define KB_TOTAL_INTS 7
#define KB_O_TOKEN_IDS 8     /* [T] */
#define KB_O_POSITIONS 9     /* [T] position of each token in its request */
#define KB_O_SEQ_OF_TOKEN 10 /* [T] index of its request in this step */
#define KB_O_CU_SEQLENS 11   /* [n + 1] first token of each request */
#define KB_O_KV_LENS 12      /* [n] request length after this step */
#define KB_O_SLOTS 13        /* [n] state slot */
#define KB_O_ROWS 14         /* [R] token rows whose logits are wanted */
#define KB_O_MAX_KV 15       /* [1] KB_MAX_KV_LEN again, for kernels */
#define KB_O_TABLES 16       /* [G, n, W] pages, -1 where there is none */
#define KBATCH_LAYOUT_INTS 24
/* ints that kbatch_pack will write for these entries (table_width 0: the narrowest multiple of 8 that holds them) */
KESTREL_API int kbatch_ints_needed(void *cache, int n, const long long *ids, const int *counts, int n_wants, int table_width);
/* tokens: the entries' token ids one after the other (NULL leaves the section unwritten: ids that are on the device already);
 * want_counts[e] places of entry e are wanted, listed in `wants` as offsets among the entry's tokens.  Pages must be reserved.
 * Returns the ints written, or -2 bad argument, -3 unknown request, -9 buffer too small. */
KESTREL_API int kbatch_pack(void *cache, int n, const long long *ids, const int *counts, const int *tokens, const int *want_counts, const int *wants, int table_width, int *out, int cap, int *layout);

/* the check of the runner's debug guards, on the host: 0 if every token of the packed description can be placed by the kernels,
 * else (rule << 16) | (token & 0xffff) for the first that cannot (rules: 1 token id, 2 request index, 3 position,
 * 4 block-table column, 5 page id, 6 token outside its request's rows); pages[g] = pages of group g's tensors */
KESTREL_API int kbatch_check(const int *batch, const int *layout, int vocab, int page_size, const int *pages);

/* ============================================================================================
 * Kernel library (libkestrel_cuda.so): runtime
 * ========================================================================================== */
KESTREL_API const char *kestrel_last_error(void);
KESTREL_API int kestrel_device_arch(void);
KESTREL_API int kestrel_sm_count(void);
KESTREL_API void kestrel_set_pdl(int on);
KESTREL_API int kestrel_wait_probe(float *elapsed_ms);
/* 0 if no bounded wait of any kernel has run out since the last call, else which kernels' did (bit 0 product, 1 prompt attention, 2 decode attention); synchronises the device */
KESTREL_API int kestrel_kernel_errors(void);

/* ---- elementwise kernels ---- */
KESTREL_API int kestrel_embed(const void *table, int dtype, const int *ids, float *out, int T, int d, kestrel_stream_t stream);
KESTREL_API void kestrel_set_norm_warp_rows(int rows, int with_slices);   /* rows from which a norm that only reads the stream takes a warp a row (0: the default), and whether one that adds slices does too; for tests of both kernels */
KESTREL_API int kestrel_add_rmsnorm(float *residual, const float *partial, int S, long long slice_stride, const float *bias, const int *rows, const float *w, float eps, void *out, int out_dtype, int R, int d, int write_back, kestrel_stream_t stream);
KESTREL_API int kestrel_swiglu(const float *partial, int S, long long slice_stride, void *out, int out_dtype, int T, int ff, kestrel_stream_t stream);
/* rot_mode: 0 pairs dimension j with j + rot/2 (rotate-half), 1 pairs 2j with 2j + 1 (interleaved); rot_scale multiplies cos and sin */
KESTREL_API int kestrel_attn_prepare(const float *partial, int S, long long slice_stride, const float *bias, const float *q_norm_w, const float *k_norm_w, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, int dtype, int T, int nq, int nkv, int hd, int write_kv, kestrel_stream_t stream);
KESTREL_API int kestrel_reduce_partials(const float *partial, int S, long long slice_stride, const float *bias, void *out, int out_dtype, int T, int width, kestrel_stream_t stream);

/* ---- matrix products ---- */
KESTREL_API int kestrel_gemm_plain(const void *x, const void *w, float *out, int dtype, int T, int N, int K, long long ldx, long long ldw, long long ldo, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_supported(const void *x, const void *w, int T, int N, int K, long long ldx, long long ldw);
KESTREL_API int kestrel_gemm_tc_splits(int T, int N, int K);
KESTREL_API int kestrel_gemm_tc_plan(const void *x, const void *w, int T, int N, int K, long long ldx, long long ldw);
KESTREL_API int kestrel_gemm_tc_w(const void *x, const void *w, float *out, int T, int N, int K, long long ldx, long long ldw, long long ldo, int splits, long long slice_stride, int weights_static, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc(const void *x, const void *w, float *out, int T, int N, int K, long long ldx, long long ldw, long long ldo, int splits, long long slice_stride, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_add(const void *x, const void *w, float *residual, int T, int N, int K, long long ldx, long long ldw, long long ldo, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_swiglu_w(const void *x, const void *w, void *out, int T, int ff, int K, long long ldx, long long ldw, long long ldo, int weights_static, kestrel_stream_t stream);
KESTREL_API int kestrel_gemm_tc_swiglu(const void *x, const void *w, void *out, int T, int ff, int K, long long ldx, long long ldw, long long ldo, kestrel_stream_t stream);
/* the q, k, v product of many tokens with the prepare kernel's work in its epilogue (head size 128, rotate-half over the whole head); 0 done, 1 this form does not apply and nothing ran */
KESTREL_API int kestrel_gemm_tc_qkv_prepare(const void *x, const void *w, int T, int K, long long ldx, long long ldw, const float *bias, const float *q_norm_w, const float *k_norm_w, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *k_cache, void *v_cache, void *q_out, int nq, int nkv, int hd, int write_kv, kestrel_stream_t stream);
KESTREL_API void kestrel_gemm_tc_set_qkv_fused(int mode);   /* 0 never, 1 where the product is not cut along K (default), 2 wherever the kernel takes the sizes */
KESTREL_API int kestrel_gemm_tc_error(void);
KESTREL_API int kestrel_linear_bf16_noalloc(const void *x, const void *w, const float *bias, void *out, int out_dtype, int T, int N, int K, long long ldx, long long ldw, kestrel_stream_t stream);
/* tuning and test hooks of the products */
KESTREL_API void kestrel_gemm_tc_set_persistent(int on);
KESTREL_API void kestrel_gemm_tc_set_pairs(int on);
KESTREL_API void kestrel_gemm_tc_set_swiglu_tile(int bn);
/* the SwiGLU product on CTA pairs with the tokens as the M operand: 0 never, 1 where its finer tiles save a round (the default), 2 always */
KESTREL_API void kestrel_gemm_tc_set_swiglu_swapped(int mode);
KESTREL_API void kestrel_gemm_tc_set_pair_tuning(int min_tokens, int overhead_kb);
KESTREL_API void kestrel_gemm_tc_set_tuning(int overhead_kb, int ctas_per_sm);
KESTREL_API void kestrel_gemm_tc_set_wide(int on, int more_than_tokens);

/* ---- attention kernels (tile lists: request and first row of each tile).  max_kv_ptr, if not
 * NULL, points to the longest request's length on the device; the slice length is then
 * ceil(that / slices) rounded up to a multiple of 128 instead of slice_len (a captured launch
 * follows the context that way). ---- */
KESTREL_API int kestrel_attention_plain(const void *q, const void *k_cache, const void *v_cache, const int *positions, const int *seq_of_token, const int *block_table, int table_stride, int page_size, void *out, int dtype, int T, int nq, int nkv, int hd, int window, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_mma(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_stride, int page_size, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_mma_rows_per_tile(int hd);
KESTREL_API int kestrel_attention_mma_slots(int hd);
KESTREL_API int kestrel_attention_merge(const float *part_o, const float *part_ml, void *out, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, int slices, int hd, int nq, int nkv, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_tc(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, int rows_per_tile, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_width, int table_stride, int page_size, int cache_pages, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_tc_supported(int hd, int page_size);
KESTREL_API int kestrel_attention_tc_slots(void);
KESTREL_API int kestrel_attention_tc_error(void);
KESTREL_API int kestrel_attention_decode(const void *q, const void *k_cache, const void *v_cache, void *out, float *part_o, float *part_ml, const int *tile_seq, const int *tile_row0, int tiles, const int *cu_seqlens, const int *kv_lens, const int *block_table, int table_width, int table_stride, int page_size, int cache_pages, int T, int nq, int nkv, int hd, int window, int slices, int slice_len, const int *max_kv_ptr, float scale, kestrel_stream_t stream);
KESTREL_API int kestrel_attention_decode_supported(int hd, int page_size);
KESTREL_API int kestrel_attention_decode_slots(int hd);
KESTREL_API int kestrel_attention_decode_cluster_slices(void);
KESTREL_API int kestrel_attention_decode_error(void);

/* ---- attention of a whole step: picks kernels, tiles the step's rows, cuts key ranges ----
 * A planner belongs to the mixers of one model.  It keeps the tile lists of the current step on
 * the device (built once per step from the step's host description and copied in one small
 * transfer; steps of one token per request need none) and scratch for key-range slices.
 * `batch_host` / `batch_dev` are the packed step description (kbatch_pack) on the host and on
 * the device, `layout` its layout; `step_serial` changes with every step.  captured != 0: the
 * launch is being recorded for replay with other contents, so the number of slices follows
 * layout[KB_MAX_KV_LEN] (a nominal context) and their length is read on the device. */
/* short prompt portions on the kernel for decode tokens: the key limits in per cent of the defaults (0: never, negative: the default); for tests and tuning */
KESTREL_API void kestrel_attention_set_small_portions(int per_cent);
KESTREL_API void *kestrel_attn_planner_create(int max_tokens, int max_seqs);
KESTREL_API void kestrel_attn_planner_destroy(void *planner);
KESTREL_API int kestrel_attention(void *planner, long long step_serial, const int *batch_host, const int *batch_dev, const int *layout, int group, int captured, const void *q, const void *k_cache, const void *v_cache, void *out, int dtype, int cache_pages, int page_size, int nq, int nkv, int hd, int window, float scale, kestrel_stream_t stream);
/* kernels launched by the planner's last kestrel_attention call */
KESTREL_API int kestrel_attn_planner_last_launches(void *planner);

/* ---- sampling ---- */
KESTREL_API int kestrel_argmax(const float *logits, long long ld, int R, int V, int *out, float *cand_v, int *cand_i, kestrel_stream_t stream);
KESTREL_API int kestrel_argmax_chunks(int V);
KESTREL_API int kestrel_repetition_penalty(float *logits, long long ld, int R, int V, const int *history, int width, const int *counts, const float *penalty, kestrel_stream_t stream);
KESTREL_API void kestrel_sample_set_cluster(int on);
KESTREL_API int kestrel_sample(const float *logits, long long ld, int R, int V, const float *temperature, const int *top_k, const float *top_p, const float *min_p, const float *uniform, int *out, kestrel_stream_t stream);

/* ============================================================================================
 * The step program (libkestrel_cuda.so): a model as a list of kernel-level operations, written
 * once when the model is built and run natively for every step, so that a step costs the host
 * one call.  Operations read and write "registers": activations of the step, allocated by the
 * runner from its workspace.  kprog_* functions that make a value return its register (>= 0)
 * or a negative code.  `tag` names the phase an operation is timed under when profiling
 * (KPH_*).  Weights and cache tensors are device pointers that stay valid while the program
 * lives.  `dtype` arguments are storage type codes.
 * ========================================================================================== */
#define KPH_OTHER 0
#define KPH_NORM 1
#define KPH_QKV 2
#define KPH_ROPE 3
#define KPH_ATTN 4
#define KPH_O 5
#define KPH_GATE_UP 6
#define KPH_DOWN 7
#define KPH_LM_HEAD 8
#define KPH_EMBED 9
#define KPH_COUNT 10
KESTREL_API void *kprog_create(int dtype);
KESTREL_API void kprog_destroy(void *prog);
/* marks the start of a layer call: registers made in the call before it stay readable during this one, older ones do not */
KESTREL_API int kprog_begin_call(void *prog);
/* float32 residual stream [T, width] = table[token ids] */
KESTREL_API int kprog_embed(void *prog, const void *table, int table_dtype, int width);
/* residual += delta (a product register, or -1); result = rmsnorm(residual) * w in out_dtype; logit_rows != 0: only the wanted rows, nothing written back */
KESTREL_API int kprog_add_rmsnorm(void *prog, int residual, int delta, const float *w, float eps, int width, int out_dtype, int logit_rows, int tag);
/* x w^T (+ bias later, by the consumer) as float32 slices; add_to >= 0: the product may add itself to that float32 register in its epilogue, its own register is then empty */
KESTREL_API int kprog_linear(void *prog, int x, const void *w, long long ldw, int N, int K, const float *bias, int add_to, int tag);
/* silu(x Wg^T) * (x Wu^T), gate rows first in w [2 ff, K] */
KESTREL_API int kprog_gate_up_swiglu(void *prog, int x, const void *w, long long ldw, int ff, int K, int tag);
/* bias, per-head RMSNorm (weights may be NULL), rotation, K and V into their pages; returns the query register [T, nq * hd] */
KESTREL_API int kprog_attn_prepare(void *prog, int qkv, const float *q_norm_w, const float *k_norm_w, float norm_eps, const float *inv_freq, int rot, int rot_mode, float rot_scale, int group, int page_size, void *k_cache, void *v_cache, int nq, int nkv, int hd, int write_kv, int tag);
/* causal attention of the step's queries over their requests' pages */
KESTREL_API int kprog_attention(void *prog, int q, void *planner, int group, int page_size, int cache_pages, const void *k_cache, const void *v_cache, int nq, int nkv, int hd, int window, float scale, int tag);
/* float32 logits [R, V] = x w^T for the wanted rows: the program's result */
KESTREL_API int kprog_logits(void *prog, int x, const void *w, long long ldw, int V, int K, int tag);
KESTREL_API int kprog_num_ops(void *prog);

/* ---- the runner: a program, a cache manager, buffers for the step description and a workspace ---- */
KESTREL_API void *krunner_create(void *prog, void *cache, int max_tokens, int max_seqs);
KESTREL_API void krunner_destroy(void *runner);
/* flags of kestrel_step_raw */
#define KSTEP_RESERVED 1     /* the caller has reserved the pages already */
#define KSTEP_NO_COMMIT 2    /* the caller commits the cache manager itself */
#define KSTEP_PROFILE 4      /* time the phases of this step with CUDA events (synchronises) */
/* Runs one step: entry e brings counts[e] next tokens of request ids[e] (`tokens`: all entries' ids one after the other);
 * want_counts / wants as in kbatch_pack.  Reserves pages (unless KSTEP_RESERVED), packs and copies the description, runs the
 * program on `stream`, writes float32 logits [R, ld_logits] to `logits` (device memory; may be NULL if R = 0) and commits the
 * requests' new lengths (unless KSTEP_NO_COMMIT).  Nothing is synchronised.  Returns the number of kernels launched, or
 * -1 pages short (nothing ran, nothing changed), other negative codes on errors. */
KESTREL_API int kestrel_step_raw(void *runner, int n, const long long *ids, const int *counts, const int *tokens, const int *want_counts, const int *wants, float *logits, long long ld_logits, int flags, kestrel_stream_t stream);
/* host-to-device bytes of the last step's description */
KESTREL_API long long krunner_last_h2d_bytes(void *runner);
/* milliseconds per phase (KPH_COUNT floats) of the last step run with KSTEP_PROFILE */
KESTREL_API int krunner_phase_ms(void *runner, float *out);
/* bytes of workspace the runner holds */
KESTREL_API long long krunner_workspace_bytes(void *runner);
/* debug checks: nonzero makes every step write guard words behind each register and check them (synchronises); returns the old value */
KESTREL_API int krunner_set_guards(void *runner, int on);
/* registers whose guard words were found damaged since the runner was made */
KESTREL_API int krunner_guard_failures(void *runner);

#endif /* KESTREL_H */
