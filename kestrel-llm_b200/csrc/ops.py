"""Python face of the sm_100a kernel library: one function per exported entry point.

Tensors are torch CUDA tensors used as typed device memory; every function checks dtypes,
shapes and contiguity, then launches on torch's current stream.  There is no CPU fallback and
no other implementation behind these names: if the library cannot be built or loaded, the
first call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build
from . import cdecl as _cdecl

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None


def library() -> ctypes.CDLL:
    """The loaded kernel library, built on first use."""
    global _lib
    if _lib is None:
        path = _build.build_cuda()
        try:
            # the kernel library calls the host runtime (cache manager), which is found beside it
            ctypes.CDLL(_build.build_host(verbose=False), mode=ctypes.RTLD_GLOBAL)
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load {path}: {e}") from None
        _declare(lib)
        _lib = lib
        if os.environ.get("KESTREL_PDL", "1") == "0":      # for A/B measurements only
            set_pdl(False)
    return _lib


def library_path() -> str:
    library()
    return _build.build_cuda(verbose=False)


_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _declare(lib) -> None:
    """Argument and result types of every exported function, from the package's C header."""
    _cdecl.declare(lib, ("kestrel_", "kprog_", "krunner_"))


launches = 0     # kernels launched through this module since import (graph replays are counted by their runner)


def _check(rc: int) -> None:
    global launches
    launches += 1
    if rc != 0:
        raise KernelError(library().kestrel_last_error().decode("utf-8", "replace"))


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current device's current stream as a raw handle.  Asked for at every launch, so it
    takes torch's two C calls where they exist (a step of a few tokens is bound by the host)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if t.is_cuda and t.is_contiguous() and (dtype is None or t.dtype == dtype) and (dims is None or t.dim() == dims):
        return
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name}: expected {dims} dimensions, got shape {tuple(t.shape)}")


def _code(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DT:
        raise KernelError(f"{name}: dtype {t.dtype} is neither float32 nor bfloat16")
    return _DT[t.dtype]


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for all kernels of the library (default on)."""
    fn = library().kestrel_set_pdl
    fn(1 if on else 0)


def device_arch() -> int:
    return library().kestrel_device_arch()


class Partials:
    """A projection's output before its consumer: ``data`` float32 [S, T, N] whose slices sum to
    the result, plus an optional float32 bias [N] still to be added."""

    __slots__ = ("data", "bias")

    def __init__(self, data: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if data.dim() == 2:
            data = data.unsqueeze(0)
        _need(data, "partials", torch.float32, 3)
        self.data = data
        self.bias = bias

    @property
    def slices(self) -> int:
        return self.data.shape[0]

    @property
    def tokens(self) -> int:
        return self.data.shape[1]

    @property
    def width(self) -> int:
        return self.data.shape[2]

    @property
    def slice_stride(self) -> int:
        return self.data.stride(0)

    def reduce(self, dtype: torch.dtype) -> torch.Tensor:
        """The summed result [T, N] in ``dtype``, for consumers without a fused form."""
        out = torch.empty((self.tokens, self.width), dtype=dtype, device=self.data.device)
        _check(library().kestrel_reduce_partials(self.data.data_ptr(), self.slices, self.slice_stride,
                                                 _p(self.bias), out.data_ptr(), _code(out, "reduce"),
                                                 self.tokens, self.width, _stream()))
        return out


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] widened to float32."""
    _need(table, "embed.table", dims=2)
    _need(ids, "embed.ids", torch.int32, 1)
    _need(out, "embed.out", torch.float32, 2)
    T, d = out.shape
    if ids.shape[0] != T or table.shape[1] != d:
        raise KernelError(f"embed: ids {tuple(ids.shape)}, table {tuple(table.shape)}, out {tuple(out.shape)}")
    _check(library().kestrel_embed(table.data_ptr(), _code(table, "embed.table"), ids.data_ptr(),
                                   out.data_ptr(), T, d, _stream()))


def norm_set_warp_rows(rows: int = 0, with_slices: bool = False) -> None:
    """From how many rows on a norm that only reads the stream takes the kernel with a warp a row
    (0: the default, 1024), and whether a norm that adds slices takes it too (by default it does
    not: the block-a-row kernel is faster there).  For tests of both kernels."""
    library().kestrel_set_norm_warp_rows(int(rows), 1 if with_slices else 0)


def add_rmsnorm(residual: torch.Tensor, delta: Optional[Partials], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
    """x = residual[t] + delta[t]; residual[t] = x if write_back; out[r] = rmsnorm(x) * weight,
    where t = rows[r] if rows is given, else r."""
    _need(residual, "add_rmsnorm.residual", torch.float32, 2)
    _need(weight, "add_rmsnorm.weight", torch.float32, 1)
    _need(out, "add_rmsnorm.out", dims=2)
    T, d = residual.shape
    R = out.shape[0]
    if weight.shape[0] != d or out.shape[1] != d:
        raise KernelError("add_rmsnorm: widths differ")
    if rows is not None:
        _need(rows, "add_rmsnorm.rows", torch.int32, 1)
        if rows.shape[0] != R:
            raise KernelError("add_rmsnorm: rows and out differ in length")
        write_back = False
    elif R != T:
        raise KernelError("add_rmsnorm: out and residual differ in rows")
    if delta is not None and (delta.tokens != T or delta.width != d):
        raise KernelError(f"add_rmsnorm: delta [{delta.tokens},{delta.width}] against residual [{T},{d}]")
    _check(library().kestrel_add_rmsnorm(
        residual.data_ptr(), _p(delta.data) if delta else None, delta.slices if delta else 0,
        delta.slice_stride if delta else 0, _p(delta.bias) if delta else None, _p(rows),
        weight.data_ptr(), float(eps), out.data_ptr(), _code(out, "add_rmsnorm.out"), R, d,
        1 if (write_back and delta is not None) else 0, _stream()))


def swiglu(gate_up: Partials, out: torch.Tensor) -> None:
    """out[t, i] = silu(g[t, i]) * u[t, i] with g, u the two halves of gate_up's width."""
    _need(out, "swiglu.out", dims=2)
    T, ff = out.shape
    if gate_up.tokens != T or gate_up.width != 2 * ff or gate_up.bias is not None:
        raise KernelError("swiglu: shapes differ, or a bias is pending")
    _check(library().kestrel_swiglu(gate_up.data.data_ptr(), gate_up.slices, gate_up.slice_stride,
                                    out.data_ptr(), _code(out, "swiglu.out"), T, ff, _stream()))


def attn_prepare(qkv: Partials, q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor],
                 norm_eps: float, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                 positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                 page_size: int, k_cache: torch.Tensor, v_cache: torch.Tensor, q_out: torch.Tensor,
                 nq: int, nkv: int, hd: int, write_kv: bool = True, rot_mode: int = 0, rot_scale: float = 1.0) -> None:
    """Bias, per-head RMSNorm, rotation; q to q_out, K and V into their cache pages.  ``rot_mode``
    0 pairs dimension j with j + rotary_dim / 2 (rotate-half), 1 pairs 2j with 2j + 1
    (interleaved); ``rot_scale`` multiplies cos and sin."""
    _need(q_out, "attn_prepare.q_out", dims=2)
    _need(positions, "attn_prepare.positions", torch.int32, 1)
    _need(seq_of_token, "attn_prepare.seq_of_token", torch.int32, 1)
    _need(block_table, "attn_prepare.block_table", torch.int32, 2)
    _need(k_cache, "attn_prepare.k_cache", q_out.dtype)
    _need(v_cache, "attn_prepare.v_cache", q_out.dtype)
    T = q_out.shape[0]
    if qkv.tokens != T or qkv.width != (nq + 2 * nkv) * hd or q_out.shape[1] != nq * hd:
        raise KernelError("attn_prepare: shapes differ")
    if rotary_dim and inv_freq is None:
        raise KernelError("attn_prepare: rotation asked for without frequencies")
    _check(library().kestrel_attn_prepare(
        qkv.data.data_ptr(), qkv.slices, qkv.slice_stride, _p(qkv.bias), _p(q_norm_w), _p(k_norm_w),
        float(norm_eps), _p(inv_freq), int(rotary_dim), int(rot_mode), float(rot_scale), positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), int(page_size), k_cache.data_ptr(),
        v_cache.data_ptr(), q_out.data_ptr(), _code(q_out, "attn_prepare.q_out"), T, nq, nkv, hd,
        1 if write_kv else 0, _stream()))


def qkv_prepare_fused(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_norm_w: Optional[torch.Tensor],
                      k_norm_w: Optional[torch.Tensor], norm_eps: float, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                      positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor, page_size: int,
                      k_cache: torch.Tensor, v_cache: torch.Tensor, q_out: torch.Tensor, nq: int, nkv: int, hd: int,
                      write_kv: bool = True, rot_mode: int = 0, rot_scale: float = 1.0) -> bool:
    """The q, k, v product of x [T, K] with w [(nq + 2 nkv) hd, K] and all of ``attn_prepare`` in
    one tcgen05 kernel.  False, and nothing launched, where that kernel does not take the case
    (float32, few tokens, a head size or rotation other than 128 / rotate-half over the whole
    head): the caller then runs the product and ``attn_prepare``."""
    if x.dtype != torch.bfloat16 or inv_freq is None or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    _need(x, "qkv_prepare.x", torch.bfloat16, 2)
    _need(w, "qkv_prepare.w", torch.bfloat16, 2)
    _need(q_out, "qkv_prepare.q_out", torch.bfloat16, 2)
    _need(positions, "qkv_prepare.positions", torch.int32, 1)
    _need(seq_of_token, "qkv_prepare.seq_of_token", torch.int32, 1)
    _need(block_table, "qkv_prepare.block_table", torch.int32, 2)
    _need(k_cache, "qkv_prepare.k_cache", torch.bfloat16)
    _need(v_cache, "qkv_prepare.v_cache", torch.bfloat16)
    T, K = x.shape
    if w.shape != ((nq + 2 * nkv) * hd, K) or q_out.shape != (T, nq * hd) or not q_out.is_contiguous():
        raise KernelError("qkv_prepare: shapes differ")
    rc = library().kestrel_gemm_tc_qkv_prepare(
        x.data_ptr(), w.data_ptr(), T, K, x.stride(0), w.stride(0), _p(bias), _p(q_norm_w), _p(k_norm_w), float(norm_eps),
        _p(inv_freq), int(rotary_dim), int(rot_mode), float(rot_scale), positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), int(page_size), k_cache.data_ptr(), v_cache.data_ptr(),
        q_out.data_ptr(), nq, nkv, hd, 1 if write_kv else 0, _stream())
    if rc == 1:
        return False
    _check(rc)
    return True


def gemm_plain(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, n] = sum_k x[t, k] w[n, k] on the CUDA cores, float32 accumulation in ascending k."""
    _need(x, "gemm.x", dims=2)
    _need(w, "gemm.w", x.dtype, 2)
    _need(out, "gemm.out", torch.float32, 2)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N):
        raise KernelError(f"gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(library().kestrel_gemm_plain(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(x, "gemm.x"),
                                        T, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()))


def attention_plain(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                    page_size: int, out: torch.Tensor, nq: int, nkv: int, hd: int, window: int,
                    scale: float) -> None:
    _need(q, "attention.q", dims=2)
    _need(out, "attention.out", q.dtype, 2)
    _need(k_cache, "attention.k_cache", q.dtype)
    _need(v_cache, "attention.v_cache", q.dtype)
    _need(block_table, "attention.block_table", torch.int32, 2)
    T = q.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape:
        raise KernelError("attention: shapes differ")
    _check(library().kestrel_attention_plain(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
        seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0), int(page_size),
        out.data_ptr(), _code(q, "attention.q"), T, nq, nkv, hd, int(window), float(scale), _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r]."""
    _need(logits, "argmax.logits", torch.float32, 2)
    _need(out, "argmax.out", torch.int32, 1)
    R, V = logits.shape
    lib = library()
    chunks = lib.kestrel_argmax_chunks(V)
    cand_v = cand_i = None
    if chunks > 1:              # a large vocabulary is scanned by many blocks; their candidates go to scratch
        cand_v = torch.empty((R, chunks), dtype=torch.float32, device=logits.device)
        cand_i = torch.empty((R, chunks), dtype=torch.int32, device=logits.device)
    _check(lib.kestrel_argmax(logits.data_ptr(), logits.stride(0), R, V, out.data_ptr(), _p(cand_v), _p(cand_i),
                              _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
    """One token per row; per-row options; rows with temperature <= 0 take the first maximum."""
    _need(logits, "sample.logits", torch.float32, 2)
    R, V = logits.shape
    for t, name, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                        (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                        (uniform, "uniform", torch.float32), (out, "out", torch.int32)):
        _need(t, f"sample.{name}", dt, 1)
        if t.shape[0] != R:
            raise KernelError(f"sample.{name}: {t.shape[0]} entries for {R} rows")
    _check(library().kestrel_sample(logits.data_ptr(), logits.stride(0), R, V, temperature.data_ptr(),
                                    top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
                                    uniform.data_ptr(), out.data_ptr(), _stream()))


def repetition_penalty(logits: torch.Tensor, history: torch.Tensor, counts: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: for each of the first counts[r] tokens of history[r] (int32 [R, width], a request's
    last generated tokens), logits[r, token] becomes l / penalty[r] if l >= 0, else l * penalty[r] -
    once per occurrence; rows with penalty <= 1 are left alone."""
    _need(logits, "repetition_penalty.logits", torch.float32, 2)
    _need(history, "repetition_penalty.history", torch.int32, 2)
    _need(counts, "repetition_penalty.counts", torch.int32, 1)
    _need(penalty, "repetition_penalty.penalty", torch.float32, 1)
    R, V = logits.shape
    if history.shape[0] != R or counts.shape[0] != R or penalty.shape[0] != R:
        raise KernelError("repetition_penalty: one row of history, one count and one penalty per row of logits")
    fn = library().kestrel_repetition_penalty
    _check(fn(logits.data_ptr(), logits.stride(0), R, V, history.data_ptr(), history.shape[1], counts.data_ptr(),
              penalty.data_ptr(), _stream()))


def sample_set_cluster(on: bool = True) -> None:
    """Whether `sample` may take the kernel that keeps a row in the shared memory of a cluster
    (the default); off: always the one-block kernel over global memory.  For tests of the latter."""
    fn = library().kestrel_sample_set_cluster
    fn(1 if on else 0)


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands: bfloat16, K and both row strides
    multiples of 8 elements, bases 16-byte aligned (the TMA rules)."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    return bool(library().kestrel_gemm_tc_supported(x.data_ptr(), w.data_ptr(), x.shape[0], w.shape[0], x.shape[1],
                                                    x.stride(0), w.stride(0)))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
            splits: Optional[int] = None, weights_static: bool = False) -> torch.Tensor:
    """y = x w^T on the tensor cores (tcgen05, TMA, TMEM) as float32 slices [S, T, N].
    ``weights_static``: w was complete before the kernel that precedes this call in the stream
    began (a model's weights, never something the step itself computes); few-token products then
    fetch their first weight tiles while that kernel still runs."""
    _need(x, "gemm_tc.x", torch.bfloat16, 2)
    _need(w, "gemm_tc.w", torch.bfloat16, 2)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_tc: x {tuple(x.shape)}, w {tuple(w.shape)}")
    lib = library()
    if out is not None:
        if out.dim() == 2:
            out = out.unsqueeze(0)
        _need(out, "gemm_tc.out", torch.float32, 3)
        if out.shape[1:] != (T, N):
            raise KernelError(f"gemm_tc: out {tuple(out.shape)} for T={T}, N={N}")
        S = out.shape[0]
    else:
        S = splits if splits is not None else lib.kestrel_gemm_tc_splits(T, N, K)
        out = torch.empty((S, T, N), dtype=torch.float32, device=x.device)
    _check(lib.kestrel_gemm_tc_w(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, x.stride(0), w.stride(0),
                                 out.stride(1), S, out.stride(0), 1 if weights_static else 0, _stream()))
    return out


def gemm_tc_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, weights_static: bool = False) -> None:
    """out = silu(x Wg^T) * (x Wu^T) in one tcgen05 kernel with two accumulators."""
    _need(x, "gemm_tc_swiglu.x", torch.bfloat16, 2)
    _need(w_gate_up, "gemm_tc_swiglu.w", torch.bfloat16, 2)
    _need(out, "gemm_tc_swiglu.out", torch.bfloat16, 2)
    T, K = x.shape
    ff = out.shape[1]
    if w_gate_up.shape != (2 * ff, K) or out.shape[0] != T:
        raise KernelError("gemm_tc_swiglu: shapes differ")
    _check(library().kestrel_gemm_tc_swiglu_w(x.data_ptr(), w_gate_up.data_ptr(), out.data_ptr(), T, ff, K,
                                              x.stride(0), w_gate_up.stride(0), out.stride(0),
                                              1 if weights_static else 0, _stream()))


def gemm_tc_set_tuning(overhead_kb: int = -1, ctas_per_sm: int = 0) -> None:
    """Tuning of the split heuristic of few-token products (see gemm_tcgen05.cu)."""
    fn = library().kestrel_gemm_tc_set_tuning
    fn(int(overhead_kb), int(ctas_per_sm))


def gemm_tc_set_wide(on: bool = True, more_than_tokens: int = -1) -> None:
    """Whether products of more than ``more_than_tokens`` (32) and at most 128 tokens take two
    weight tiles a CTA (the default).  For tests and measurements of the one-tile kernel."""
    fn = library().kestrel_gemm_tc_set_wide
    fn(1 if on else 0, int(more_than_tokens))


def gemm_tc_set_pair_tuning(min_tokens: int = -1, overhead_kb: int = -1) -> None:
    """Tuning of many-token products on CTA pairs: products of more than ``min_tokens`` tokens
    take them; a K slice is priced at ``overhead_kb`` k-blocks beyond its own (see gemm_tcgen05.cu)."""
    fn = library().kestrel_gemm_tc_set_pair_tuning
    fn(int(min_tokens), int(overhead_kb))


def gemm_tc_set_many_token_path(pairs: bool = True, persistent: bool = True, swiglu_tile: int = 256,
                                swiglu_swapped: Optional[bool] = None) -> None:
    """Which kernel a many-token product (more than 128 tokens) takes: CTA pairs (the default),
    else one persistent CTA per SM (what runs where pairs cannot be scheduled; ``swiglu_tile``
    128 or 256 tokens for its SwiGLU form), else one tile per CTA.  ``swiglu_swapped``: the
    SwiGLU product on pairs takes the tokens as the M operand always (True), never (False), or
    where its finer tiles save a round of tiles (None, the default).  For tests of every path."""
    lib = library()
    for name, v in (("kestrel_gemm_tc_set_pairs", 1 if pairs else 0), ("kestrel_gemm_tc_set_persistent", 1 if persistent else 0),
                    ("kestrel_gemm_tc_set_swiglu_tile", int(swiglu_tile)), ("kestrel_gemm_tc_set_swiglu_swapped", 1 if swiglu_swapped is None else (2 if swiglu_swapped else 0))):
        fn = getattr(lib, name)
        fn(v)


def gemm_tc_set_qkv_fused(on: Optional[bool] = None) -> None:
    """Whether a q, k, v product of many tokens does ``attn_prepare``'s work in its epilogue: where
    the product would not be cut along K (None, the default), wherever the kernel takes the
    sizes (True), never (False).  For tests of both paths."""
    library().kestrel_gemm_tc_set_qkv_fused(1 if on is None else (2 if on else 0))


def gemm_tc_error() -> int:
    """Error word of the tcgen05 kernels' bounded waits (0 = none); synchronises the device."""
    return library().kestrel_gemm_tc_error()


def linear(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
           weights_static: bool = False) -> torch.Tensor:
    """y = x w^T as float32 slices [S, T, N] (S = 1 unless a split-K kernel ran).
    ``weights_static`` as in `gemm_tc`.

    float32 operands always take the CUDA-core product; bfloat16 operands take the tcgen05
    product when its tiling rules hold (see `gemm_tc_supported`) and the CUDA-core one
    otherwise."""
    T, N = x.shape[0], w.shape[0]
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2:
        # one question to the library: do the operands fit, and into how many K slices
        plan = library().kestrel_gemm_tc_plan(x.data_ptr(), w.data_ptr(), T, N, x.shape[1], x.stride(0), w.stride(0))
        if plan > 0:
            return gemm_tc(x, w, out, splits=plan if out is None else None, weights_static=weights_static)
    if out is None:
        out = torch.empty((1, T, N), dtype=torch.float32, device=x.device)
    elif out.dim() == 2:
        out = out.unsqueeze(0)
    gemm_plain(x, w, out[0])
    return out


def linear_add_into(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> bool:
    """residual += x w^T inside the product's epilogue, where the product can do that (bfloat16,
    many tokens, one pass over K); False if it cannot - nothing has run then and the caller takes
    the product as slices."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    _need(x, "linear_add_into.x", torch.bfloat16, 2)
    _need(w, "linear_add_into.w", torch.bfloat16, 2)
    _need(residual, "linear_add_into.residual", torch.float32, 2)
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or residual.shape != (T, N):
        raise KernelError(f"linear_add_into: x {tuple(x.shape)}, w {tuple(w.shape)}, residual {tuple(residual.shape)}")
    rc = library().kestrel_gemm_tc_add(x.data_ptr(), w.data_ptr(), residual.data_ptr(), T, N, K, x.stride(0), w.stride(0),
                                       residual.stride(0), _stream())
    if rc == 1:
        return False
    _check(rc)
    return True


def gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, ff: int, weights_static: bool = False) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) in x's dtype, Wg and Wu being the two halves of w_gate_up's rows.
    ``weights_static`` as in `gemm_tc`."""
    out = torch.empty((x.shape[0], ff), dtype=x.dtype, device=x.device)
    if gemm_tc_supported(x, w_gate_up):
        # the activation is the product's epilogue: the K range is not split, whatever the number of
        # tokens, and the gate/up product never reaches memory
        gemm_tc_swiglu(x, w_gate_up, out, weights_static=weights_static)
    else:
        swiglu(Partials(linear(x, w_gate_up, weights_static=weights_static)), out)
    return out


def attention_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                  tile_seq: torch.Tensor, tile_row0: torch.Tensor, rows_per_tile: int, cu_seqlens: torch.Tensor,
                  kv_lens: torch.Tensor, block_table: torch.Tensor, page_size: int, nq: int, nkv: int, hd: int,
                  window: int, scale: float, slices: int = 1, slice_len: int = 1 << 30,
                  max_kv_dev: Optional[torch.Tensor] = None) -> None:
    """Tensor-core attention (mma.sync) of the tiles listed in tile_seq / tile_row0; rows of
    other requests in ``out`` are left alone.  With ``slices`` > 1 the key range is cut into
    slices of ``slice_len`` keys (a multiple of 64) that are merged in ascending order;
    ``slices * slice_len`` must reach the longest request, keys beyond it are not seen."""
    _need(q, "attention_mma.q", torch.bfloat16, 2)
    _need(out, "attention_mma.out", torch.bfloat16, 2)
    _need(k_cache, "attention_mma.k_cache", torch.bfloat16)
    _need(v_cache, "attention_mma.v_cache", torch.bfloat16)
    _need(block_table, "attention_mma.block_table", torch.int32, 2)
    _need(tile_seq, "attention_mma.tile_seq", torch.int32, 1)
    _need(tile_row0, "attention_mma.tile_row0", torch.int32, 1)
    T = q.shape[0]
    tiles = tile_seq.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape or tile_row0.shape[0] != tiles:
        raise KernelError("attention_mma: shapes differ")
    part_o = part_ml = None
    if slices > 1:
        part_o = torch.empty((T * nq, slices, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T * nq, slices, 2), dtype=torch.float32, device=q.device)
    slice_len = min(int(slice_len), 1 << 30)
    _check(library().kestrel_attention_mma(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(part_o), _p(part_ml),
        tile_seq.data_ptr(), tile_row0.data_ptr(), tiles, rows_per_tile, cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), int(page_size), T, nq, nkv, hd, int(window), int(slices),
        slice_len, _p(max_kv_dev), float(scale), _stream()))
    if slices > 1:
        global launches
        launches += 1          # the merge kernel


def attention_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                 tile_seq: torch.Tensor, tile_row0: torch.Tensor, cu_seqlens: torch.Tensor, kv_lens: torch.Tensor,
                 block_table: torch.Tensor, page_size: int, nq: int, nkv: int, hd: int, window: int, scale: float,
                 slices: int = 1, slice_len: int = 1 << 30, max_kv_dev: Optional[torch.Tensor] = None,
                 rows_per_tile: int = 128) -> None:
    """tcgen05 attention of the listed tiles, head size 128: tiles of ``rows_per_tile`` rows, up
    to 256 (prompt portions; 16 for decode tokens); the key range may be cut into
    ``slices`` slices of ``slice_len`` keys (a multiple of 128) that are merged in ascending
    order; ``slices * slice_len`` must reach the longest request.  The cache tensors are
    [pages, kv heads, page size, 128], contiguous, with a page size the kernel's page-wise TMA
    boxes fit (``attention_tc_supported``)."""
    _need(q, "attention_tc.q", torch.bfloat16, 2)
    _need(out, "attention_tc.out", torch.bfloat16, 2)
    _need(k_cache, "attention_tc.k_cache", torch.bfloat16)
    _need(v_cache, "attention_tc.v_cache", torch.bfloat16)
    _need(block_table, "attention_tc.block_table", torch.int32, 2)
    _need(tile_seq, "attention_tc.tile_seq", torch.int32, 1)
    _need(tile_row0, "attention_tc.tile_row0", torch.int32, 1)
    T, tiles = q.shape[0], tile_seq.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape or tile_row0.shape[0] != tiles:
        raise KernelError("attention_tc: shapes differ")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention_tc: cache of shape {tuple(k_cache.shape)}, expected [pages, {nkv}, {page_size}, {hd}]")
    part_o = part_ml = None
    if slices > 1:
        part_o = torch.empty((T * nq, slices, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T * nq, slices, 2), dtype=torch.float32, device=q.device)
    slice_len = min(int(slice_len), (1 << 30) // 128 * 128)
    _check(library().kestrel_attention_tc(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(part_o), _p(part_ml),
        tile_seq.data_ptr(), tile_row0.data_ptr(), tiles, int(rows_per_tile), cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], block_table.stride(0), int(page_size), int(k_cache.shape[0]), T, nq, nkv, hd,
        int(window), int(slices), slice_len, _p(max_kv_dev), float(scale), _stream()))
    if slices > 1:
        global launches
        launches += 1          # the merge kernel


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     tile_seq: torch.Tensor, tile_row0: torch.Tensor, cu_seqlens: torch.Tensor, kv_lens: torch.Tensor,
                     block_table: torch.Tensor, page_size: int, nq: int, nkv: int, hd: int, window: int, scale: float,
                     slices: int = 1, slice_len: int = 1 << 30, max_kv_dev: Optional[torch.Tensor] = None) -> None:
    """Attention of decode tokens (tiles of at most 16 rows) with a TMA loader warp in front of
    four mma.sync warps, head size 64 or 128; the key range is cut into ``slices`` slices of
    ``slice_len`` keys (a multiple of 64) that are merged in ascending order (up to 4 inside the
    kernel, by the CTAs of a cluster; more through scratch and a second kernel), and
    ``slices * slice_len`` must reach the longest request.  The cache tensors are
    [pages, kv heads, page size, head size], contiguous (``attention_decode_supported``).  Keys
    and values of positions before a request's first token of this step must have been written
    by earlier steps, not by the kernel in front of this one: they are fetched before it ends."""
    _need(q, "attention_decode.q", torch.bfloat16, 2)
    _need(out, "attention_decode.out", torch.bfloat16, 2)
    _need(k_cache, "attention_decode.k_cache", torch.bfloat16)
    _need(v_cache, "attention_decode.v_cache", torch.bfloat16)
    _need(block_table, "attention_decode.block_table", torch.int32, 2)
    _need(tile_seq, "attention_decode.tile_seq", torch.int32, 1)
    _need(tile_row0, "attention_decode.tile_row0", torch.int32, 1)
    T, tiles = q.shape[0], tile_seq.shape[0]
    if q.shape[1] != nq * hd or out.shape != q.shape or tile_row0.shape[0] != tiles:
        raise KernelError("attention_decode: shapes differ")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention_decode: cache of shape {tuple(k_cache.shape)}, expected [pages, {nkv}, {page_size}, {hd}]")
    part_o = part_ml = None
    scratch = slices > library().kestrel_attention_decode_cluster_slices()    # fewer are merged inside the kernel
    if scratch:
        part_o = torch.empty((T * nq, slices, hd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T * nq, slices, 2), dtype=torch.float32, device=q.device)
    slice_len = min(int(slice_len), (1 << 30) // 128 * 128)
    _check(library().kestrel_attention_decode(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _p(part_o), _p(part_ml),
        tile_seq.data_ptr(), tile_row0.data_ptr(), tiles, cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], block_table.stride(0), int(page_size), int(k_cache.shape[0]), T,
        nq, nkv, hd, int(window), int(slices), slice_len, _p(max_kv_dev), float(scale), _stream()))
    if scratch:
        global launches
        launches += 1          # the merge kernel


def attention_decode_supported(hd: int, page_size: int) -> bool:
    """Whether the decode attention kernel takes this head size and page size."""
    return bool(library().kestrel_attention_decode_supported(int(hd), int(page_size)))


def attention_decode_error() -> int:
    """Error word of the decode attention kernel's bounded waits (0 = none); synchronises the device."""
    return library().kestrel_attention_decode_error()


def attention_tc_supported(hd: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernel takes this head size and page size."""
    return bool(library().kestrel_attention_tc_supported(int(hd), int(page_size)))


def raise_on_kernel_error() -> None:
    """Reads the error words of the kernels with bounded waits (matrix product, the two attention
    kernels) and raises if one of them gave up a wait: its output is not to be trusted.
    Synchronises the device; callers use it where they synchronise anyway."""
    lib = library()
    bad = [(name, code) for name, code in (("gemm_tcgen05", lib.kestrel_gemm_tc_error()),
                                           ("attention_tc", lib.kestrel_attention_tc_error()),
                                           ("attention_decode", lib.kestrel_attention_decode_error())) if code]
    if bad:
        raise KernelError("a bounded wait ran out in " + ", ".join(f"{n} (wait {c})" for n, c in bad) +
                          ": the step's results are invalid")


def wait_probe():
    """Runs one block that waits, with the kernels' bounded wait, on a barrier nobody completes.
    Returns (gave_up, milliseconds): the wait must give up within seconds and leave the
    device usable."""
    ms = ctypes.c_float(0.0)
    rc = library().kestrel_wait_probe(ctypes.addressof(ms))
    if rc < 0:
        raise KernelError(library().kestrel_last_error().decode("utf-8", "replace"))
    return rc == 1, float(ms.value)


def attention_tc_error() -> int:
    """Error word of the tcgen05 attention kernel's bounded waits (0 = none); synchronises the device."""
    return library().kestrel_attention_tc_error()


def attention_set_small_portions(per_cent: int = -1) -> None:
    """Short prompt portions (at most 512 rows of (token, head) per kv head) go to the attention
    kernel for decode tokens while their keys stay under limits by row count; ``per_cent`` scales
    those limits (0: never, negative: the default).  For tests of both routes."""
    library().kestrel_attention_set_small_portions(int(per_cent))


class AttentionPlanner:
    """What the attention kernels keep between the layers of a step: the tile lists of the
    step's requests on the device (made once per step from the step's host description) and
    scratch for key-range slices.  One planner serves all attention layers of a model; its
    launches must stay on one stream."""

    def __init__(self, max_tokens: int = 4096, max_seqs: int = 256):
        self._lib = library()
        self._h = self._lib.kestrel_attn_planner_create(int(max_tokens), int(max_seqs))
        if not self._h:
            raise KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))

    @property
    def handle(self):
        return self._h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.kestrel_attn_planner_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def attention(planner: Optional[AttentionPlanner], q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch,
              group: int, page_size: int, out: torch.Tensor, nq: int, nkv: int, hd: int, window: int, scale: float) -> None:
    """Causal attention of this step's queries over their requests' cache pages.  ``batch``
    is the step's description: its packed int32 buffer on the host (``host``) and on the device
    (``device_buffer``), the buffer's ``layout``, a ``serial`` that changes with every step, and
    ``captured`` (the launch is being recorded for replay).  Which kernel takes which requests,
    the tiling of their rows and the cutting of key ranges into slices are decided natively
    (csrc/kernels/attention_dispatch.cu); float32 always takes the plain kernel."""
    _need(q, "attention.q", dims=2)
    _need(out, "attention.out", q.dtype, 2)
    _need(k_cache, "attention.k_cache", q.dtype, 4)
    _need(v_cache, "attention.v_cache", q.dtype, 4)
    if q.shape[1] != nq * hd or out.shape != q.shape:
        raise KernelError("attention: shapes differ")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"attention: cache of shape {tuple(k_cache.shape)}, expected [pages, {nkv}, {page_size}, {hd}]")
    if q.shape[0] != batch.num_tokens:
        raise KernelError(f"attention: {q.shape[0]} query rows for a step of {batch.num_tokens} tokens")
    lib = library()
    global launches
    rc = lib.kestrel_attention(planner.handle if planner is not None else None, int(batch.serial), batch.host.ctypes.data,
                               batch.device_buffer.data_ptr(), batch.layout.ctypes.data, int(group), 1 if batch.captured else 0,
                               q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _code(q, "attention.q"),
                               int(k_cache.shape[0]), int(page_size), nq, nkv, hd, int(window), float(scale), _stream())
    if rc != 0:
        raise KernelError(lib.kestrel_last_error().decode("utf-8", "replace"))
    launches += lib.kestrel_attn_planner_last_launches(planner.handle) if planner is not None else 1


# ---- the step program and its runner ---------------------------------------------------------
PHASES = {name[4:].lower(): value for name, value in _cdecl.constants().items() if name.startswith("KPH_") and name != "KPH_COUNT"}
PHASE_COUNT = _cdecl.constants()["KPH_COUNT"]


class StepProgram:
    """A model's step as a list of kernel-level operations (csrc/kernels/step_program.cu).  Parts
    write their operations into it once, in the order in which they run (`emit` methods); the
    methods below return registers - small integers that name activations - or raise."""

    def __init__(self, dtype: torch.dtype):
        self._lib = library()
        self.dtype = dtype
        self._h = self._lib.kprog_create(_DT[dtype])
        if not self._h:
            raise KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))
        self._keep = []          # tensors the program points into

    @property
    def handle(self):
        return self._h

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.kprog_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _reg(self, rc: int) -> int:
        if rc < 0:
            raise KernelError(self._lib.kestrel_last_error().decode("utf-8", "replace"))
        return rc

    def _ptr(self, t: Optional[torch.Tensor], name: str, dtype=None):
        if t is None:
            return None
        _need(t, name, dtype)
        self._keep.append(t)
        return t.data_ptr()

    def begin_call(self) -> None:
        self._reg(self._lib.kprog_begin_call(self._h))

    def embed(self, table: torch.Tensor) -> int:
        _need(table, "program.embed.table", dims=2)
        return self._reg(self._lib.kprog_embed(self._h, self._ptr(table, "table"), _code(table, "table"), table.shape[1]))

    def add_rmsnorm(self, residual: int, delta: Optional[int], weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                    logit_rows: bool = False, phase: str = "norm") -> int:
        return self._reg(self._lib.kprog_add_rmsnorm(self._h, residual, -1 if delta is None else delta,
                                                     self._ptr(weight, "norm weight", torch.float32), float(eps), weight.shape[0],
                                                     _DT[out_dtype], 1 if logit_rows else 0, PHASES[phase]))

    def linear(self, x: int, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, add_to: Optional[int] = None,
               phase: str = "other") -> int:
        _need(weight, "program.linear.weight", self.dtype, 2)
        return self._reg(self._lib.kprog_linear(self._h, x, self._ptr(weight, "weight"), weight.stride(0), weight.shape[0],
                                                weight.shape[1], self._ptr(bias, "bias", torch.float32),
                                                -1 if add_to is None else add_to, PHASES[phase]))

    def gate_up_swiglu(self, x: int, weight: torch.Tensor, ff: int, phase: str = "gate_up") -> int:
        _need(weight, "program.gate_up.weight", self.dtype, 2)
        if weight.shape[0] != 2 * ff:
            raise KernelError("program.gate_up_swiglu: the weight has not 2 x ff rows")
        return self._reg(self._lib.kprog_gate_up_swiglu(self._h, x, self._ptr(weight, "weight"), weight.stride(0), ff,
                                                        weight.shape[1], PHASES[phase]))

    def attn_prepare(self, qkv: int, q_norm_w, k_norm_w, norm_eps: float, inv_freq, rotary_dim: int, rot_mode: int,
                     rot_scale: float, group: int, page_size: int, k_cache: torch.Tensor, v_cache: torch.Tensor, nq: int,
                     nkv: int, hd: int, write_kv: bool, phase: str = "rope") -> int:
        return self._reg(self._lib.kprog_attn_prepare(
            self._h, qkv, self._ptr(q_norm_w, "q_norm", torch.float32), self._ptr(k_norm_w, "k_norm", torch.float32),
            float(norm_eps), self._ptr(inv_freq, "inv_freq", torch.float32), int(rotary_dim), int(rot_mode), float(rot_scale),
            int(group), int(page_size), self._ptr(k_cache, "k_cache", self.dtype), self._ptr(v_cache, "v_cache", self.dtype),
            nq, nkv, hd, 1 if write_kv else 0, PHASES[phase]))

    def attention(self, q: int, planner: Optional[AttentionPlanner], group: int, page_size: int, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, nq: int, nkv: int, hd: int, window: int, scale: float, phase: str = "attn") -> int:
        if planner is not None:
            self._keep.append(planner)
        return self._reg(self._lib.kprog_attention(
            self._h, q, planner.handle if planner is not None else None, int(group), int(page_size), int(k_cache.shape[0]),
            self._ptr(k_cache, "k_cache", self.dtype), self._ptr(v_cache, "v_cache", self.dtype), nq, nkv, hd, int(window),
            float(scale), PHASES[phase]))

    def logits(self, x: int, weight: torch.Tensor, phase: str = "lm_head") -> None:
        _need(weight, "program.logits.weight", self.dtype, 2)
        self._reg(self._lib.kprog_logits(self._h, x, self._ptr(weight, "weight"), weight.stride(0), weight.shape[0],
                                         weight.shape[1], PHASES[phase]))

    @property
    def num_ops(self) -> int:
        return self._lib.kprog_num_ops(self._h)


def kernel_errors() -> int:
    """Bits of the kernels whose bounded waits ran out since the last call (0 = none); synchronises."""
    return library().kestrel_kernel_errors()
