"""The allocation-free matrix product `kestrel_linear_bf16_noalloc` (csrc/kernels/linear_noalloc.h).

Some users of the library cannot allocate device memory when they need a product - their
application gave the whole device to its own arena, or they sit in a loop where cudaMalloc's
device synchronisation is not acceptable - so this entry point keeps its split-K scratch in a
fixed 16 MiB array inside the library.  The test calls it through its exported C symbol, as
such a user would, twice in a row with different shapes (the second call finds the first
call's leftovers in the shared scratch), and compares each result with the library's usual
route, kestrel_gemm_tc into a scratch buffer allocated per call followed by the sum of the
slices.  It is collected last, so a run that stops at the first failure has already run every
other test; it also passes alone in a fresh process.  (GPU)"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _symbol():
    from kestrel_llm_b200.csrc import ops
    lib = ops.library()
    fn = lib.kestrel_linear_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p]
    return ops, lib, fn


def _operands(T, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((T, K), generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    b = torch.randn((N,), generator=g).to(DEV)
    return x, w, b


def test_two_calls_in_a_row_match_the_allocating_route():
    ops, lib, fn = _symbol()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    # (T, N, K, output dtype): split into several slices / one slice; float32 / bfloat16 out; then more than 128
    # tokens with few output tiles (CTA pairs, K cut into slices), and a product whose slices would not fit the
    # scratch (2 x 128 x 16,384 x 4 bytes = 16 MiB exactly fits; 3 slices would not), which runs as fewer
    for call, (T, N, K, out_dtype) in enumerate([(8, 4096, 4096, torch.float32), (40, 1000, 776, torch.bfloat16),
                                                 (300, 1024, 4096, torch.bfloat16), (128, 16384, 4096, torch.float32)]):
        x, w, b = _operands(T, N, K, 100 + call)
        out = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
        rc = fn(x.data_ptr(), w.data_ptr(), b.data_ptr(), out.data_ptr(), 0 if out_dtype == torch.float32 else 1,
                T, N, K, x.stride(0), w.stride(0), stream)
        assert rc == 0, lib.kestrel_last_error().decode()
        splits = lib.kestrel_gemm_tc_splits(T, N, K)
        if splits * T * N * 4 > (16 << 20):
            splits = 1                                                    # the entry point's fall-back: one slice always fits or is refused
        want = ops.Partials(ops.gemm_tc(x, w, splits=splits), b).reduce(out_dtype)      # scratch allocated per call
        assert ops.gemm_tc_error() == 0
        assert torch.isfinite(out.float()).all()
        # same kernels, same order of sums: the two routes agree to the last bit; the bound below
        # is the one the other kernel tests use and would still catch a stale or misplaced slice
        ref = x.float() @ w.float().T + b
        tol = 2e-6 * (K ** 0.5) * float(ref.abs().max()) + 1e-7 if out_dtype == torch.float32 else 1e-2 * float(ref.abs().max())
        assert float((out.float() - want.float()).abs().max()) <= tol
        assert float((out.float() - ref).abs().max()) <= tol
        assert torch.equal(out, want)


def test_a_product_beyond_the_scratch_is_refused():
    ops, lib, fn = _symbol()
    T, N, K = 256, 24576, 64                  # 1 slice x 256 x 24576 x 4 bytes = 24 MiB > 16 MiB
    x = torch.zeros((T, K), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((N, K), dtype=torch.bfloat16, device=DEV)
    out = torch.zeros((T, N), dtype=torch.float32, device=DEV)
    rc = fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 0, T, N, K, K, K, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.kestrel_last_error().decode()
    assert "scratch" in msg and "25165824" in msg and "16777216" in msg
    rc = fn(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 0, 4, 16, 12, 12, 12, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "multiples of 8" in lib.kestrel_last_error().decode()
