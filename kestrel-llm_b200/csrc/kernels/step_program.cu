// The step program and its runner: a model's step as a list of kernel-level operations that is
// written once, when the model is built, and run natively for every step.
//
// The reference's forward functions are C loops over layers that call its kernels directly
// (src/model/vllm_safetensors.c:16404-16812 for one token, :18140-18683 for a prompt's
// mini-batches).  Here the model is assembled from parts at run time, so the loop cannot be
// compiled in; instead every part writes the operations of its forward pass into a program
// (kprog_*), in the order in which they run, and the runner walks that list: a step of several
// hundred kernels costs the host one call (kestrel_step_raw) and a few microseconds a launch,
// where a walk through the parts from an interpreted language costs more than the kernels of a
// small step take to run.
//
// Values are "registers": activations of the step's tokens.  Their sizes depend on the step
// (T tokens, R wanted rows, the number of K slices a product is cut into), so they are laid
// out when the step runs: the float32 residual stream lives in a region of its own, everything
// else is bump-allocated in one of two regions that alternate from layer call to layer call, so
// that a call can still read what the call before it left (the not yet added output of the
// previous block) and memory use is that of two layers, whatever the depth.
//
// Debug guards (krunner_set_guards): every register is followed by guard words that are set
// before the step and read back after it, and a checking kernel walks the step's description on
// the device first - token ids against the vocabulary, block-table entries against the page
// count - with the same predicate the host tests use (step_checks.cuh).  The reference
// brackets its cache blocks and scratch buffers the same way (include/model/vllm_safetensors.h:32-36,
// src/model/vllm_safetensors.c:9219-9232).
#include "common.cuh"
#include "step_checks.cuh"

#include <string.h>

#include <algorithm>
#include <vector>

namespace {

enum OpKind { OP_BEGIN_CALL, OP_EMBED, OP_ADD_RMSNORM, OP_LINEAR, OP_GATE_UP_SWIGLU, OP_ATTN_PREPARE, OP_ATTENTION, OP_LOGITS };

struct Op {
    OpKind kind = OP_BEGIN_CALL;
    int tag = KPH_OTHER;
    int out = -1;                 // register made
    int a = -1, b = -1;           // input registers
    const void *w = nullptr;      // weights
    long long ldw = 0;
    const float *bias = nullptr;
    const float *w2 = nullptr, *w3 = nullptr;      // norm weights of attn_prepare; inv_freq
    const void *k_cache = nullptr, *v_cache = nullptr;
    void *planner = nullptr;
    int N = 0, K = 0, width = 0, dtype = 0, flag = 0;
    int nq = 0, nkv = 0, hd = 0, window = 0, group = 0, page_size = 0, cache_pages = 0, rot = 0, rot_mode = 0;
    float eps = 0.f, scale = 0.f, rot_scale = 1.f;
};

// what a register holds while a step runs
struct Reg {
    void *ptr = nullptr;
    int rows = 0, cols = 0;
    int dtype = KESTREL_F32;      // element type of a plain tensor
    int slices = -1;              // >= 0: float32 slices [slices, rows, cols] still to be summed (0: added already, nothing pending)
    const float *bias = nullptr;  // still to be added by the consumer of the slices
    void *prepared = nullptr;     // a q, k, v product whose kernel did the prepare op's work too: the queries it wrote
    void *q_room = nullptr;       // room taken for the queries when that kernel was tried and did not take the case
    bool persistent = false;
};

struct Program {
    int dtype = KESTREL_BF16;
    std::vector<Op> ops;
    int n_regs = 0;
    int vocab = 0;                // rows of the embedding table are not known here; set by kprog_logits
    int new_reg() { return n_regs++; }
};

constexpr size_t ALIGN = 256;
constexpr size_t GUARD_BYTES = 256;
constexpr int PIN_RING = 3;

size_t align_up(size_t v) { return (v + ALIGN - 1) / ALIGN * ALIGN; }
size_t elem_size(int dtype) { return dtype == KESTREL_BF16 ? 2 : 4; }

struct Runner {
    Program *prog = nullptr;
    void *cache = nullptr;
    int max_tokens = 0, max_seqs = 0;
    // step description: pinned staging ring and device ring
    int cap_ints = 0;
    int *h_ring[PIN_RING] = {}, *d_ring[PIN_RING] = {};
    cudaEvent_t copied[PIN_RING] = {};
    bool used[PIN_RING] = {};
    int turn = 0;
    long long serial = 0;
    long long last_h2d = 0;
    // workspace
    char *arena = nullptr;
    size_t arena_bytes = 0;
    // profiling
    std::vector<cudaEvent_t> events;
    float phase_ms[KPH_COUNT] = {};
    // debug guards
    int guards = 0;
    int guard_failures = 0;
    std::vector<char *> guard_at;
    int *d_check = nullptr;
    std::vector<Reg> regs;
};

// One walk over the program.  dry: only sizes are computed (bytes of the three regions);
// otherwise registers get addresses and kernels are launched.
struct Walk {
    Runner &r;
    const int *host, *dev, *layout;
    float *logits;
    long long ld_logits;
    cudaStream_t stream;
    bool dry, profile;
    size_t persistent_used = 0, call_used = 0, call_peak = 0;
    char *persistent_base = nullptr, *region[2] = {nullptr, nullptr};
    int parity = 0;
    int launches = 0;

    void *take(size_t bytes, bool persistent) {
        size_t padded = align_up(bytes) + (r.guards ? GUARD_BYTES : 0);
        size_t &used = persistent ? persistent_used : call_used;
        char *p = dry ? nullptr : (persistent ? persistent_base : region[parity]) + used;
        if (!dry && r.guards) r.guard_at.push_back(p + align_up(bytes));
        used += padded;
        if (!persistent) call_peak = std::max(call_peak, call_used);
        return p;
    }

    int run() {
        Program &pg = *r.prog;
        const int T = layout[KB_NUM_TOKENS], R = layout[KB_NUM_ROWS], n = layout[KB_NUM_SEQS], W = layout[KB_TABLE_WIDTH];
        std::vector<Reg> &regs = r.regs;
        regs.assign(pg.n_regs, Reg());
        const char *fake = (const char *)ALIGN;            // an aligned address for the products' planning in a dry walk
        int ev = 0;
        for (size_t oi = 0; oi < pg.ops.size(); ++oi) {
            const Op &op = pg.ops[oi];
            if (profile && !dry) cudaEventRecord(r.events[ev++], stream);
            int rc = 0;
            switch (op.kind) {
                case OP_BEGIN_CALL:
                    parity ^= 1;
                    call_used = 0;
                    break;
                case OP_EMBED: {
                    Reg &o = regs[op.out];
                    o.rows = T; o.cols = op.width; o.dtype = KESTREL_F32; o.persistent = true;
                    o.ptr = take((size_t)T * op.width * 4, true);
                    if (!dry) {
                        rc = kestrel_embed(op.w, op.dtype, dev + layout[KB_O_TOKEN_IDS], (float *)o.ptr, T, op.width, stream);
                        launches++;
                    }
                    break;
                }
                case OP_ADD_RMSNORM: {
                    const Reg &res = regs[op.a];
                    const Reg *delta = op.b >= 0 ? &regs[op.b] : nullptr;
                    if (delta && delta->slices == 0) delta = nullptr;         // the product added itself already
                    if (delta && delta->slices < 0) return kestrel_fail(-2, "step program: op %zu adds a register that is not a product", oi);
                    Reg &o = regs[op.out];
                    const int rows = op.flag ? R : T;
                    o.rows = rows; o.cols = op.width; o.dtype = op.dtype;
                    o.ptr = take((size_t)rows * op.width * elem_size(op.dtype), false);
                    if (!dry && rows > 0) {
                        if (res.cols != op.width || (delta && (delta->cols != op.width || delta->rows != T)))
                            return kestrel_fail(-2, "step program: op %zu: widths of norm, stream and product differ", oi);
                        rc = kestrel_add_rmsnorm((float *)res.ptr, delta ? (const float *)delta->ptr : nullptr, delta ? delta->slices : 0,
                                                 delta ? (long long)T * delta->cols : 0, delta ? delta->bias : nullptr,
                                                 op.flag ? dev + layout[KB_O_ROWS] : nullptr, (const float *)op.w, op.eps, o.ptr, op.dtype,
                                                 rows, op.width, (!op.flag && delta) ? 1 : 0, stream);
                        launches++;
                    }
                    break;
                }
                case OP_LINEAR: {
                    const Reg &x = regs[op.a];
                    Reg &o = regs[op.out];
                    o.rows = T; o.cols = op.N; o.dtype = KESTREL_F32; o.bias = op.bias;
                    const void *xp = dry ? (const void *)fake : x.ptr;
                    const bool bf16 = pg.dtype == KESTREL_BF16;
                    if (!dry && (x.cols != op.K || x.rows != T || x.slices >= 0))
                        return kestrel_fail(-2, "step program: op %zu: product of [%d, %d] with weights of %d columns", oi, x.rows, x.cols, op.K);
                    if (!dry && bf16 && op.b >= 0 && !op.bias) {
                        // the product may add itself to the float32 stream in its epilogue (a dry walk
                        // counts the slices it would need otherwise: an upper bound)
                        Reg &res = regs[op.b];
                        int added = kestrel_gemm_tc_add(xp, op.w, (float *)res.ptr, T, op.N, op.K, op.K, op.ldw, op.N, stream);
                        if (added < 0) return added;
                        if (added == 0) {
                            launches++;
                            o.slices = 0;
                            o.ptr = nullptr;
                            break;
                        }
                    }
                    if (!dry && bf16 && op.b < 0 && oi + 1 < pg.ops.size() && pg.ops[oi + 1].kind == OP_ATTN_PREPARE && pg.ops[oi + 1].a == op.out) {
                        // a q, k, v product of many tokens does its consumer's work in its epilogue, where
                        // that kernel takes the sizes; the product's float32 plane is then never made (a
                        // dry walk counts both the plane and the queries: an upper bound)
                        const Op &pp = pg.ops[oi + 1];
                        if (op.N == (pp.nq + 2 * pp.nkv) * pp.hd && pp.group >= 0 && pp.group < layout[KB_NUM_GROUPS]) {
                            void *q_out = take((size_t)T * pp.nq * pp.hd * elem_size(pg.dtype), false);
                            int fused = kestrel_gemm_tc_qkv_prepare(xp, op.w, T, op.K, op.K, op.ldw, op.bias, pp.w2, pp.w3, pp.eps, (const float *)pp.w,
                                                                    pp.rot, pp.rot_mode, pp.rot_scale, dev + layout[KB_O_POSITIONS],
                                                                    dev + layout[KB_O_SEQ_OF_TOKEN], dev + layout[KB_O_TABLES] + (size_t)pp.group * n * W, W,
                                                                    pp.page_size, (void *)pp.k_cache, (void *)pp.v_cache, q_out, pp.nq, pp.nkv, pp.hd,
                                                                    pp.flag, stream);
                            if (fused < 0) return fused;
                            if (fused == 0) {
                                launches++;
                                o.slices = 0;
                                o.ptr = nullptr;
                                o.prepared = q_out;
                                break;
                            }
                            o.q_room = q_out;              // the prepare op writes its queries there
                        }
                    }
                    const int S = bf16 ? kestrel_gemm_tc_plan(xp, op.w, T, op.N, op.K, op.K, op.ldw) : 0;
                    o.slices = S > 0 ? S : 1;
                    o.ptr = take((size_t)o.slices * T * op.N * 4, false);
                    if (!dry) {
                        if (S > 0)
                            rc = kestrel_gemm_tc_w(xp, op.w, (float *)o.ptr, T, op.N, op.K, op.K, op.ldw, op.N, S, (long long)T * op.N, 1, stream);
                        else
                            rc = kestrel_gemm_plain(xp, op.w, (float *)o.ptr, pg.dtype, T, op.N, op.K, op.K, op.ldw, op.N, stream);
                        launches++;
                    }
                    break;
                }
                case OP_GATE_UP_SWIGLU: {
                    const Reg &x = regs[op.a];
                    Reg &o = regs[op.out];
                    const int ff = op.N;
                    o.rows = T; o.cols = ff; o.dtype = pg.dtype;
                    o.ptr = take((size_t)T * ff * elem_size(pg.dtype), false);
                    const void *xp = dry ? (const void *)fake : x.ptr;
                    if (!dry && (x.cols != op.K || x.rows != T))
                        return kestrel_fail(-2, "step program: op %zu: gated product of [%d, %d] with weights of %d columns", oi, x.rows, x.cols, op.K);
                    if (pg.dtype == KESTREL_BF16 && kestrel_gemm_tc_supported(xp, op.w, T, 2 * ff, op.K, op.K, op.ldw)) {
                        // the activation is the product's epilogue: the gate/up product never reaches memory
                        if (!dry) {
                            rc = kestrel_gemm_tc_swiglu_w(xp, op.w, o.ptr, T, ff, op.K, op.K, op.ldw, ff, 1, stream);
                            launches++;
                        }
                    } else {
                        const int S = pg.dtype == KESTREL_BF16 ? kestrel_gemm_tc_plan(xp, op.w, T, 2 * ff, op.K, op.K, op.ldw) : 0;
                        const int slices = S > 0 ? S : 1;
                        float *gu = (float *)take((size_t)slices * T * 2 * ff * 4, false);
                        if (!dry) {
                            if (S > 0)
                                rc = kestrel_gemm_tc_w(xp, op.w, gu, T, 2 * ff, op.K, op.K, op.ldw, 2 * ff, S, (long long)T * 2 * ff, 1, stream);
                            else
                                rc = kestrel_gemm_plain(xp, op.w, gu, pg.dtype, T, 2 * ff, op.K, op.K, op.ldw, 2 * ff, stream);
                            if (rc) return rc;
                            rc = kestrel_swiglu(gu, slices, (long long)T * 2 * ff, o.ptr, pg.dtype, T, ff, stream);
                            launches += 2;
                        }
                    }
                    break;
                }
                case OP_ATTN_PREPARE: {
                    const Reg &qkv = regs[op.a];
                    Reg &o = regs[op.out];
                    o.rows = T; o.cols = op.nq * op.hd; o.dtype = pg.dtype;
                    if (!dry && qkv.prepared) {
                        o.ptr = qkv.prepared;
                        break;
                    }
                    o.ptr = (!dry && qkv.q_room) ? qkv.q_room : take((size_t)T * o.cols * elem_size(pg.dtype), false);
                    if (!dry) {
                        if (qkv.slices < 1 || qkv.cols != (op.nq + 2 * op.nkv) * op.hd)
                            return kestrel_fail(-2, "step program: op %zu: the register is not a q, k, v product of %d + 2 x %d heads", oi, op.nq, op.nkv);
                        if (op.group < 0 || op.group >= layout[KB_NUM_GROUPS])
                            return kestrel_fail(-2, "step program: op %zu: cache group %d of %d", oi, op.group, layout[KB_NUM_GROUPS]);
                        rc = kestrel_attn_prepare((const float *)qkv.ptr, qkv.slices, (long long)T * qkv.cols, qkv.bias, op.w2, op.w3, op.eps,
                                                  (const float *)op.w, op.rot, op.rot_mode, op.rot_scale, dev + layout[KB_O_POSITIONS],
                                                  dev + layout[KB_O_SEQ_OF_TOKEN], dev + layout[KB_O_TABLES] + (size_t)op.group * n * W, W,
                                                  op.page_size, (void *)op.k_cache, (void *)op.v_cache, o.ptr, pg.dtype, T, op.nq, op.nkv,
                                                  op.hd, op.flag, stream);
                        launches++;
                    }
                    break;
                }
                case OP_ATTENTION: {
                    const Reg &q = regs[op.a];
                    Reg &o = regs[op.out];
                    o.rows = T; o.cols = op.nq * op.hd; o.dtype = pg.dtype;
                    o.ptr = take((size_t)T * o.cols * elem_size(pg.dtype), false);
                    if (!dry) {
                        rc = kestrel_attention(op.planner, r.serial, host, dev, layout, op.group, 0, q.ptr, op.k_cache, op.v_cache, o.ptr, pg.dtype,
                                               op.cache_pages, op.page_size, op.nq, op.nkv, op.hd, op.window, op.scale, stream);
                        launches += op.planner ? kestrel_attn_planner_last_launches(op.planner) : 1;
                    }
                    break;
                }
                case OP_LOGITS: {
                    const Reg &x = regs[op.a];
                    if (!dry && R > 0) {
                        if (!logits) return kestrel_fail(-2, "step program: %d rows of logits are wanted and no buffer was given", R);
                        if (x.cols != op.K || x.rows != R) return kestrel_fail(-2, "step program: op %zu: output head over [%d, %d]", oi, x.rows, x.cols);
                        if (ld_logits < op.N) return kestrel_fail(-2, "step program: logits rows of %lld entries for a vocabulary of %d", ld_logits, op.N);
                        // not split over K: the logits have no consumer kernel that would sum slices
                        if (pg.dtype == KESTREL_BF16 && kestrel_gemm_tc_supported(x.ptr, op.w, R, op.N, op.K, op.K, op.ldw))
                            rc = kestrel_gemm_tc_w(x.ptr, op.w, logits, R, op.N, op.K, op.K, op.ldw, ld_logits, 1, 0, 1, stream);
                        else
                            rc = kestrel_gemm_plain(x.ptr, op.w, logits, pg.dtype, R, op.N, op.K, op.K, op.ldw, ld_logits, stream);
                        launches++;
                    }
                    break;
                }
            }
            if (rc) return rc;
        }
        if (profile && !dry) cudaEventRecord(r.events[ev++], stream);
        return 0;
    }
};

int ensure_buffers(Runner &r, int ints) {
    if (ints <= r.cap_ints) return 0;
    cudaDeviceSynchronize();
    for (int i = 0; i < PIN_RING; ++i) {
        if (r.h_ring[i]) cudaFreeHost(r.h_ring[i]);
        if (r.d_ring[i]) cudaFree(r.d_ring[i]);
        r.h_ring[i] = r.d_ring[i] = nullptr;
        r.used[i] = false;
    }
    r.cap_ints = ints + ints / 4;
    for (int i = 0; i < PIN_RING; ++i)
        if (cudaMallocHost(&r.h_ring[i], sizeof(int) * (size_t)r.cap_ints) != cudaSuccess ||
            cudaMalloc(&r.d_ring[i], sizeof(int) * (size_t)r.cap_ints) != cudaSuccess)
            return kestrel_fail(-3, "runner: no memory for a step description of %d ints", r.cap_ints);
    return 0;
}

__global__ void check_batch_kernel(const int *batch, StepCheckLayout lay, int *result) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= lay.num_tokens) return;
    const int code = kestrel_check_token(batch, lay, t);
    if (code) atomicCAS(result, 0, code * 65536 + (t & 0xffff));
}

}  // namespace

// ---- program ---------------------------------------------------------------------------------
KESTREL_API void *kprog_create(int dtype) {
    if (dtype != KESTREL_F32 && dtype != KESTREL_BF16) { kestrel_fail(-2, "step program: unknown storage type %d", dtype); return nullptr; }
    Program *p = new Program();
    p->dtype = dtype;
    return p;
}

KESTREL_API void kprog_destroy(void *prog) { delete (Program *)prog; }

KESTREL_API int kprog_num_ops(void *prog) { return (int)((Program *)prog)->ops.size(); }

#define PROG_REG_OK(pg, reg, what) KESTREL_REQUIRE((reg) >= 0 && (reg) < (pg).n_regs, "step program: %s names register %d, which does not exist", what, (reg))

KESTREL_API int kprog_begin_call(void *prog) {
    Program &pg = *(Program *)prog;
    Op op;
    op.kind = OP_BEGIN_CALL;
    pg.ops.push_back(op);
    return 0;
}

KESTREL_API int kprog_embed(void *prog, const void *table, int table_dtype, int width) {
    Program &pg = *(Program *)prog;
    KESTREL_REQUIRE(table && width > 0, "step program: embedding without a table");
    Op op;
    op.kind = OP_EMBED; op.tag = KPH_EMBED; op.w = table; op.dtype = table_dtype; op.width = width; op.out = pg.new_reg();
    pg.ops.push_back(op);
    return op.out;
}

KESTREL_API int kprog_add_rmsnorm(void *prog, int residual, int delta, const float *w, float eps, int width, int out_dtype,
                                  int logit_rows, int tag) {
    Program &pg = *(Program *)prog;
    PROG_REG_OK(pg, residual, "add_rmsnorm");
    if (delta >= 0) PROG_REG_OK(pg, delta, "add_rmsnorm");
    KESTREL_REQUIRE(w && width > 0, "step program: norm without weights");
    Op op;
    op.kind = OP_ADD_RMSNORM; op.tag = tag; op.a = residual; op.b = delta; op.w = w; op.eps = eps; op.width = width;
    op.dtype = out_dtype; op.flag = logit_rows ? 1 : 0; op.out = pg.new_reg();
    pg.ops.push_back(op);
    return op.out;
}

KESTREL_API int kprog_linear(void *prog, int x, const void *w, long long ldw, int N, int K, const float *bias, int add_to, int tag) {
    Program &pg = *(Program *)prog;
    PROG_REG_OK(pg, x, "linear");
    if (add_to >= 0) PROG_REG_OK(pg, add_to, "linear");
    KESTREL_REQUIRE(w && N > 0 && K > 0 && ldw >= K, "step program: product with weights [%d, %d], row stride %lld", N, K, ldw);
    Op op;
    op.kind = OP_LINEAR; op.tag = tag; op.a = x; op.b = add_to; op.w = w; op.ldw = ldw; op.N = N; op.K = K; op.bias = bias;
    op.out = pg.new_reg();
    pg.ops.push_back(op);
    return op.out;
}

KESTREL_API int kprog_gate_up_swiglu(void *prog, int x, const void *w, long long ldw, int ff, int K, int tag) {
    Program &pg = *(Program *)prog;
    PROG_REG_OK(pg, x, "gate_up_swiglu");
    KESTREL_REQUIRE(w && ff > 0 && K > 0 && ldw >= K, "step program: gated product with weights [2 x %d, %d]", ff, K);
    Op op;
    op.kind = OP_GATE_UP_SWIGLU; op.tag = tag; op.a = x; op.w = w; op.ldw = ldw; op.N = ff; op.K = K; op.out = pg.new_reg();
    pg.ops.push_back(op);
    return op.out;
}

KESTREL_API int kprog_attn_prepare(void *prog, int qkv, const float *q_norm_w, const float *k_norm_w, float norm_eps,
                                   const float *inv_freq, int rot, int rot_mode, float rot_scale, int group, int page_size,
                                   void *k_cache, void *v_cache, int nq, int nkv, int hd, int write_kv, int tag) {
    Program &pg = *(Program *)prog;
    PROG_REG_OK(pg, qkv, "attn_prepare");
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && hd > 0 && page_size > 0 && group >= 0, "step program: attn_prepare with bad sizes");
    KESTREL_REQUIRE(k_cache && v_cache, "step program: attn_prepare without cache tensors");
    KESTREL_REQUIRE(rot == 0 || inv_freq, "step program: rotation asked for without frequencies");
    Op op;
    op.kind = OP_ATTN_PREPARE; op.tag = tag; op.a = qkv; op.w2 = q_norm_w; op.w3 = k_norm_w; op.eps = norm_eps; op.w = inv_freq;
    op.rot = rot; op.rot_mode = rot_mode; op.rot_scale = rot_scale; op.group = group; op.page_size = page_size;
    op.k_cache = k_cache; op.v_cache = v_cache; op.nq = nq; op.nkv = nkv; op.hd = hd; op.flag = write_kv ? 1 : 0; op.out = pg.new_reg();
    pg.ops.push_back(op);
    return op.out;
}

KESTREL_API int kprog_attention(void *prog, int q, void *planner, int group, int page_size, int cache_pages, const void *k_cache,
                                const void *v_cache, int nq, int nkv, int hd, int window, float scale, int tag) {
    Program &pg = *(Program *)prog;
    PROG_REG_OK(pg, q, "attention");
    KESTREL_REQUIRE(nq > 0 && nkv > 0 && hd > 0 && page_size > 0 && group >= 0 && cache_pages > 0, "step program: attention with bad sizes");
    KESTREL_REQUIRE(k_cache && v_cache, "step program: attention without cache tensors");
    Op op;
    op.kind = OP_ATTENTION; op.tag = tag; op.a = q; op.planner = planner; op.group = group; op.page_size = page_size;
    op.cache_pages = cache_pages; op.k_cache = k_cache; op.v_cache = v_cache; op.nq = nq; op.nkv = nkv; op.hd = hd;
    op.window = window; op.scale = scale; op.out = pg.new_reg();
    pg.ops.push_back(op);
    return op.out;
}

KESTREL_API int kprog_logits(void *prog, int x, const void *w, long long ldw, int V, int K, int tag) {
    Program &pg = *(Program *)prog;
    PROG_REG_OK(pg, x, "logits");
    KESTREL_REQUIRE(w && V > 0 && K > 0 && ldw >= K, "step program: output head with weights [%d, %d]", V, K);
    Op op;
    op.kind = OP_LOGITS; op.tag = tag; op.a = x; op.w = w; op.ldw = ldw; op.N = V; op.K = K;
    pg.vocab = V;
    pg.ops.push_back(op);
    return 0;
}

// ---- runner ----------------------------------------------------------------------------------
KESTREL_API void *krunner_create(void *prog, void *cache, int max_tokens, int max_seqs) {
    if (!prog || !cache || max_tokens <= 0 || max_seqs <= 0) { kestrel_fail(-2, "runner: bad arguments"); return nullptr; }
    Runner *r = new Runner();
    r->prog = (Program *)prog;
    r->cache = cache;
    r->max_tokens = max_tokens;
    r->max_seqs = max_seqs;
    bool ok = true;
    for (int i = 0; ok && i < PIN_RING; ++i) ok = cudaEventCreateWithFlags(&r->copied[i], cudaEventDisableTiming) == cudaSuccess;
    const long long ints = 4ll * max_tokens + 3ll * max_seqs + 8 +
                           (long long)kcache_num_groups(cache) * max_seqs * ((kcache_max_blocks(cache) + 7) / 8 * 8);
    if (ok) ok = ints < 0x7fffffff && ensure_buffers(*r, (int)ints) == 0;
    if (ok) ok = cudaMalloc(&r->d_check, sizeof(int)) == cudaSuccess && cudaMemset(r->d_check, 0, sizeof(int)) == cudaSuccess;
    if (!ok) {
        kestrel_fail(-3, "runner: cannot allocate its buffers: %s", cudaGetErrorString(cudaGetLastError()));
        krunner_destroy(r);
        return nullptr;
    }
    return r;
}

KESTREL_API void krunner_destroy(void *runner) {
    Runner *r = (Runner *)runner;
    if (!r) return;
    cudaDeviceSynchronize();
    for (int i = 0; i < PIN_RING; ++i) {
        if (r->h_ring[i]) cudaFreeHost(r->h_ring[i]);
        if (r->d_ring[i]) cudaFree(r->d_ring[i]);
        if (r->copied[i]) cudaEventDestroy(r->copied[i]);
    }
    for (cudaEvent_t e : r->events) cudaEventDestroy(e);
    if (r->arena) cudaFree(r->arena);
    if (r->d_check) cudaFree(r->d_check);
    delete r;
}

KESTREL_API long long krunner_last_h2d_bytes(void *runner) { return ((Runner *)runner)->last_h2d; }
KESTREL_API long long krunner_workspace_bytes(void *runner) { return (long long)((Runner *)runner)->arena_bytes; }
KESTREL_API int krunner_guard_failures(void *runner) { return ((Runner *)runner)->guard_failures; }

KESTREL_API int krunner_set_guards(void *runner, int on) {
    Runner *r = (Runner *)runner;
    int old = r->guards;
    r->guards = on ? 1 : 0;
    return old;
}

KESTREL_API int krunner_phase_ms(void *runner, float *out) {
    Runner *r = (Runner *)runner;
    for (int i = 0; i < KPH_COUNT; ++i) out[i] = r->phase_ms[i];
    return 0;
}

KESTREL_API int kestrel_step_raw(void *runner, int n, const long long *ids, const int *counts, const int *tokens,
                                 const int *want_counts, const int *wants, float *logits, long long ld_logits, int flags,
                                 kestrel_stream_t stream) {
    Runner *rp = (Runner *)runner;
    KESTREL_REQUIRE(rp && n > 0 && ids && counts && tokens, "step: no entries");
    Runner &r = *rp;
    long long T = 0, R = 0;
    for (int e = 0; e < n; ++e) {
        KESTREL_REQUIRE(counts[e] > 0, "step: entry %d brings %d tokens", e, counts[e]);
        T += counts[e];
        if (want_counts) R += want_counts[e];
    }
    KESTREL_REQUIRE(T < (1ll << 30), "step: %lld tokens", T);
    for (int e = 0; e < n; ++e)
        for (int f = 0; f < e; ++f) KESTREL_REQUIRE(ids[e] != ids[f], "step: request %lld appears twice", ids[e]);
    if (!(flags & KSTEP_RESERVED)) {
        for (int e = 0; e < n; ++e) {
            if (kcache_slot(r.cache, ids[e]) < 0) {
                int slot = kcache_admit(r.cache, ids[e]);
                KESTREL_REQUIRE(slot >= 0, "step: no state slot is free for request %lld", ids[e]);
            }
            int rc = kcache_reserve(r.cache, ids[e], counts[e]);
            if (rc == -1) return kestrel_fail(-1, "step: no pages left for %d more tokens of request %lld", counts[e], ids[e]);
            KESTREL_REQUIRE(rc == 0, "step: the cache manager refused request %lld (code %d)", ids[e], rc);
        }
    }
    int need = kbatch_ints_needed(r.cache, n, ids, counts, (int)R, 0);
    KESTREL_REQUIRE(need > 0, "step: cannot describe the entries (code %d)", need);
    int rc = ensure_buffers(r, need);
    if (rc) return rc;
    const int slot = r.turn;
    r.turn = (r.turn + 1) % PIN_RING;
    if (r.used[slot]) cudaEventSynchronize(r.copied[slot]);
    int layout[KBATCH_LAYOUT_INTS];
    int total = kbatch_pack(r.cache, n, ids, counts, tokens, want_counts, wants, 0, r.h_ring[slot], r.cap_ints, layout);
    KESTREL_REQUIRE(total > 0, "step: packing the description failed (code %d)", total);
    if (cudaMemcpyAsync(r.d_ring[slot], r.h_ring[slot], sizeof(int) * (size_t)total, cudaMemcpyHostToDevice, stream) != cudaSuccess)
        return kestrel_fail(-3, "step: copy of the description failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaEventRecord(r.copied[slot], stream);
    r.used[slot] = true;
    r.last_h2d = (long long)sizeof(int) * total;
    r.serial++;

    // sizes of this step's registers, then the walk that launches
    Walk dry{r, r.h_ring[slot], r.d_ring[slot], layout, nullptr, ld_logits, stream, true, false};
    rc = dry.run();
    if (rc) return rc;
    const size_t persistent = align_up(dry.persistent_used), per_call = align_up(dry.call_peak);
    const size_t need_bytes = persistent + 2 * per_call + ALIGN;
    if (need_bytes > r.arena_bytes) {
        cudaDeviceSynchronize();
        if (r.arena) cudaFree(r.arena);
        r.arena = nullptr;
        r.arena_bytes = 0;
        const size_t want = need_bytes + need_bytes / 8;
        if (cudaMalloc(&r.arena, want) != cudaSuccess) return kestrel_fail(-3, "step: no memory for a workspace of %zu bytes", want);
        r.arena_bytes = want;
    }
    const bool profile = (flags & KSTEP_PROFILE) != 0;
    if (profile) {
        while (r.events.size() < r.prog->ops.size() + 1) {
            cudaEvent_t e;
            if (cudaEventCreate(&e) != cudaSuccess) return kestrel_fail(-3, "step: cannot create timing events");
            r.events.push_back(e);
        }
    }
    if (r.guards) {
        // the description is checked on the device before any kernel indexes with it
        StepCheckLayout lay = step_check_layout(layout, r.prog->vocab, kcache_page_size(r.cache));
        for (int g = 0; g < lay.num_groups && g < STEP_CHECK_MAX_GROUPS; ++g) lay.pages[g] = kcache_num_pages(r.cache, g) + 1;
        check_batch_kernel<<<(unsigned)((T + 127) / 128), 128, 0, stream>>>(r.d_ring[slot], lay, r.d_check);
        r.guard_at.clear();
    }
    Walk w{r, r.h_ring[slot], r.d_ring[slot], layout, logits, ld_logits, stream, false, profile};
    w.persistent_base = r.arena;
    w.region[0] = r.arena + persistent;
    w.region[1] = r.arena + persistent + per_call;
    // guard words behind every register: the whole workspace is filled with them before the first
    // kernel runs; the walk notes where each register ends
    if (r.guards) cudaMemsetAsync(r.arena, 0xA5, r.arena_bytes, stream);
    rc = w.run();
    if (rc) return rc;
    if (r.guards) {
        cudaStreamSynchronize(stream);
        int code = 0;
        cudaMemcpy(&code, r.d_check, sizeof(int), cudaMemcpyDeviceToHost);
        if (code) {
            cudaMemset(r.d_check, 0, sizeof(int));
            r.guard_failures++;
            return kestrel_fail(-6, "step: the description fails its check on the device: %s at token %d", step_check_text(code >> 16), code & 0xffff);
        }
        unsigned char words[GUARD_BYTES];
        for (char *g : r.guard_at) {
            cudaMemcpy(words, g, GUARD_BYTES, cudaMemcpyDeviceToHost);
            for (size_t i = 0; i < GUARD_BYTES; ++i)
                if (words[i] != 0xA5) {
                    r.guard_failures++;
                    return kestrel_fail(-6, "step: the guard words behind a register at workspace offset %lld were overwritten", (long long)(g - r.arena));
                }
        }
    }
    if (profile) {
        cudaStreamSynchronize(stream);
        for (int i = 0; i < KPH_COUNT; ++i) r.phase_ms[i] = 0.f;
        for (size_t oi = 0; oi < r.prog->ops.size(); ++oi) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, r.events[oi], r.events[oi + 1]);
            int tag = r.prog->ops[oi].tag;
            r.phase_ms[tag >= 0 && tag < KPH_COUNT ? tag : KPH_OTHER] += ms;
        }
    }
    if (!(flags & KSTEP_NO_COMMIT))
        for (int e = 0; e < n; ++e) {
            rc = kcache_commit(r.cache, ids[e], counts[e]);
            KESTREL_REQUIRE(rc == 0, "step: commit of request %lld failed (code %d)", ids[e], rc);
        }
    return w.launches;
}
