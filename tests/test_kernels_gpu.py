"""Each kernel alone against a plain float32 (numpy/torch) statement of the same operation,
at sizes other than the engine's tiny models: widths and vocabularies that are no power of
two, head sizes in steps of 16, odd numbers of heads and groups (GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _ops():
    from kestrel_llm_b200.csrc import ops
    return ops


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    t = (torch.randn(shape, generator=g) * scale).to(dtype)
    return t.to(DEV), t.float().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,N,K", [(1, 509, 96), (37, 200, 96), (130, 96, 200), (65, 1000, 777), (3, 64, 1)])
def test_gemm_plain(dtype, T, N, K):
    ops = _ops()
    x, xr = _rand((T, K), DT[dtype], 1)
    w, wr = _rand((N, K), DT[dtype], 2, 0.05)
    out = torch.full((T, N), float("nan"), device=DEV)
    ops.gemm_plain(x, w, out)
    ref = xr.astype(np.float64) @ wr.astype(np.float64).T
    np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max() + 1e-7)


def test_gemm_plain_is_the_same_for_any_batch():
    ops = _ops()
    x, _ = _rand((70, 333), torch.float32, 3)
    w, _ = _rand((129, 333), torch.float32, 4)
    full = torch.empty((70, 129), device=DEV)
    ops.gemm_plain(x, w, full)
    one = torch.empty((1, 129), device=DEV)
    ops.gemm_plain(x[41:42].contiguous(), w, one)
    assert torch.equal(one[0], full[41])            # bit-identical: the k order does not depend on T


@pytest.mark.parametrize("T,N,K,splits", [(1, 509, 96, None), (8, 4096, 4096, None), (37, 200, 96, 1), (130, 96, 200, 1),
                                          (65, 1000, 776, 3), (16, 128, 64, 1), (17, 129, 72, 1), (300, 640, 512, None),
                                          (2048, 384, 256, 1), (64, 6144, 1024, 2), (3, 260, 4096, None), (600, 40000, 512, 1), (257, 129, 8, 1),
                                          (300, 640, 2048, 2), (512, 4096, 4096, None), (200, 1100, 3080, 3), (1000, 520, 4096, 4),
                                          (129, 6144, 4096, None), (128, 6144, 4096, None)])
def test_gemm_tcgen05(T, N, K, splits):
    """The tensor-core product against the CUDA-core product of the same bfloat16 operands."""
    ops = _ops()
    x, xr = _rand((T, K), torch.bfloat16, 1)
    w, wr = _rand((N, K), torch.bfloat16, 2, 0.05)
    assert ops.gemm_tc_supported(x, w)
    out = ops.gemm_tc(x, w, splits=splits)
    assert ops.gemm_tc_error() == 0
    if splits is not None:
        assert out.shape[0] == splits
    got = out.sum(0).cpu().numpy()
    ref = xr.astype(np.float64) @ wr.astype(np.float64).T
    np.testing.assert_allclose(got, ref, rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max() + 1e-7)
    plain = torch.empty((T, N), device=DEV)
    ops.gemm_plain(x, w, plain)
    np.testing.assert_allclose(got, plain.cpu().numpy(), rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max() + 1e-7)


@pytest.mark.parametrize("T,N,K", [(300, 384, 512), (2048, 1100, 1096), (700, 4096, 256)])
def test_gemm_tcgen05_adds_into_the_residual(T, N, K):
    """The many-token product with the residual add in its epilogue: residual += x w^T gives the
    bits of the product as a slice added afterwards; a few-token product declines."""
    ops = _ops()
    x, xr = _rand((T, K), torch.bfloat16, T + 1)
    w, wr = _rand((N, K), torch.bfloat16, N + 1, 0.05)
    res, rr = _rand((T, N), torch.float32, 9)
    want = res + ops.gemm_tc(x, w, splits=1)[0]
    assert ops.linear_add_into(x, w, res)
    assert ops.gemm_tc_error() == 0
    assert torch.equal(res, want)
    ref = rr.astype(np.float64) + xr.astype(np.float64) @ wr.astype(np.float64).T
    np.testing.assert_allclose(res.cpu().numpy(), ref, rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max())
    few = torch.zeros((8, N), device=DEV)
    assert not ops.linear_add_into(x[:8].contiguous(), w, few) and float(few.abs().max()) == 0.0


@pytest.mark.parametrize("pairs,persistent,tile", [(False, True, 256), (False, True, 128), (False, False, 256)])
def test_gemm_tcgen05_fallbacks_for_many_tokens(pairs, persistent, tile):
    """The kernels a many-token product takes where CTA pairs cannot be scheduled (one persistent
    CTA per SM) or are switched off altogether (one tile per CTA), plain and with the SwiGLU epilogue."""
    ops = _ops()
    T, N, K, ff = 700, 1100, 520, 648
    x, xr = _rand((T, K), torch.bfloat16, 41)
    w, wr = _rand((N, K), torch.bfloat16, 42, 0.05)
    w2, w2r = _rand((2 * ff, K), torch.bfloat16, 43, 0.1)
    act = torch.empty((T, ff), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc_set_many_token_path(pairs, persistent, tile)
    try:
        got = ops.gemm_tc(x, w, splits=1)[0].cpu().numpy()
        cut = ops.gemm_tc(x, w, splits=3).sum(0).cpu().numpy()          # K in slices: one tile per CTA, whatever the setting
        ops.gemm_tc_swiglu(x, w2, act)
        assert ops.gemm_tc_error() == 0
    finally:
        ops.gemm_tc_set_many_token_path()
    ref = xr.astype(np.float64) @ wr.astype(np.float64).T
    np.testing.assert_allclose(got, ref, rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max())
    np.testing.assert_allclose(cut, ref, rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max())
    y = xr.astype(np.float64) @ w2r.astype(np.float64).T
    ref2 = (y[:, :ff] / (1 + np.exp(-y[:, :ff]))) * y[:, ff:]
    np.testing.assert_allclose(act.float().cpu().numpy(), ref2, rtol=1e-2, atol=1e-2 * np.abs(ref2).max())


def test_gemm_tcgen05_tuning_moves_the_kernel_not_the_result():
    """The tuning knobs choose among kernels and numbers of K slices; whatever they choose, the
    product is the same within float32 rounding: CTA pairs already from 65 tokens on, a slice
    priced at nothing (many slices) or at a fortune (one)."""
    ops = _ops()
    T, N, K = 100, 1100, 2048
    x, xr = _rand((T, K), torch.bfloat16, 51)
    w, wr = _rand((N, K), torch.bfloat16, 52, 0.05)
    ref = xr.astype(np.float64) @ wr.astype(np.float64).T
    seen = set()
    try:
        for min_tokens, pair_kb, few_kb in ((128, 12, 6), (64, 12, 6), (64, 0, 6), (64, 1000, 6), (128, 12, 0), (128, 12, 1000)):
            ops.gemm_tc_set_pair_tuning(min_tokens, pair_kb)
            ops.gemm_tc_set_tuning(few_kb, 0)
            out = ops.gemm_tc(x, w)
            seen.add(out.shape[0])
            np.testing.assert_allclose(out.sum(0).cpu().numpy(), ref, rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max())
        assert ops.gemm_tc_error() == 0
    finally:
        ops.gemm_tc_set_pair_tuning(128, 12)
        ops.gemm_tc_set_tuning(6, 2)
    assert len(seen) > 1, "the knobs never changed the number of slices"


@pytest.mark.parametrize("T,N,K,splits", [(33, 512, 512, 2), (64, 768, 1096, 3), (65, 256, 520, 1), (100, 1280, 2048, 4), (128, 6144, 1024, 2)])
def test_gemm_tcgen05_two_weight_tiles_a_cta(T, N, K, splits):
    """33 to 128 tokens: a CTA takes rows n and N / 2 + n of the weights against one token tile.
    The same bits as one tile a CTA gives (each output element is the same chain of MMAs), and a
    width that is no multiple of 256 takes one tile a CTA."""
    ops = _ops()
    x, xr = _rand((T, K), torch.bfloat16, T)
    w, wr = _rand((N, K), torch.bfloat16, N, 0.05)
    try:
        ops.gemm_tc_set_wide(False)
        one = ops.gemm_tc(x, w, splits=splits)
        ops.gemm_tc_set_wide(True)
        two = ops.gemm_tc(x, w, splits=splits)
        odd = ops.gemm_tc(x, w[:N - 128].contiguous(), splits=splits)       # N - 128 is no multiple of 256
    finally:
        ops.gemm_tc_set_wide(True)
    assert ops.gemm_tc_error() == 0
    assert torch.equal(one, two)
    assert torch.equal(odd, one[:, :, :N - 128])
    ref = xr.astype(np.float64) @ wr.astype(np.float64).T
    np.testing.assert_allclose(two.sum(0).cpu().numpy(), ref, rtol=0, atol=2e-6 * math.sqrt(K) * np.abs(ref).max() + 1e-7)


def test_gemm_tcgen05_static_weights_wait_for_the_activations():
    """With weights_static the product fetches weight tiles before the kernel in front of it has
    ended; the activations, which that kernel writes, must still be the new ones.  A chain of
    norm -> product, run several times over with a changing residual: every result follows its
    own input."""
    ops = _ops()
    T, d, N = 8, 1024, 640
    w, wr = _rand((N, d), torch.bfloat16, 11, 0.05)
    gain = torch.ones(d, device=DEV)
    xs = torch.empty((T, d), dtype=torch.bfloat16, device=DEV)
    outs, refs = [], []
    for it in range(6):
        res, rr = _rand((T, d), torch.float32, 20 + it, 1.0 + it)
        ops.add_rmsnorm(res, None, gain, 1e-6, xs, write_back=False)
        outs.append(ops.gemm_tc(xs, w, weights_static=True).sum(0))
        xn = rr / np.sqrt((rr.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6)
        xn = torch.from_numpy(xn.astype(np.float32)).to(torch.bfloat16).float().numpy()
        refs.append(xn.astype(np.float64) @ wr.astype(np.float64).T)
    assert ops.gemm_tc_error() == 0
    for got, ref in zip(outs, refs):
        np.testing.assert_allclose(got.cpu().numpy(), ref, rtol=0, atol=1e-2 * np.abs(ref).max())


def test_gemm_tcgen05_row_does_not_depend_on_the_batch():
    ops = _ops()
    x, _ = _rand((300, 512), torch.bfloat16, 3)
    w, _ = _rand((384, 512), torch.bfloat16, 4, 0.05)
    full = ops.gemm_tc(x, w, splits=1)[0]
    one = ops.gemm_tc(x[41:42].contiguous(), w, splits=1)[0]
    assert torch.equal(one[0], full[41])


@pytest.mark.parametrize("T,ff,K", [(5, 200, 96), (300, 200, 96), (257, 640, 512), (1024, 384, 320), (700, 20000, 256),
                                    (1, 64, 64), (8, 1000, 512), (40, 72, 136), (100, 333 * 8, 264), (256, 520, 1024)])
def test_gemm_tcgen05_swiglu(T, ff, K):
    ops = _ops()
    x, xr = _rand((T, K), torch.bfloat16, 5)
    w, wr = _rand((2 * ff, K), torch.bfloat16, 6, 0.1)
    out = torch.empty((T, ff), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc_swiglu(x, w, out)
    assert ops.gemm_tc_error() == 0
    y = xr.astype(np.float64) @ wr.astype(np.float64).T
    ref = (y[:, :ff] / (1 + np.exp(-y[:, :ff]))) * y[:, ff:]
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=1e-2, atol=1e-2 * np.abs(ref).max())
    if T > 128:
        # on CTA pairs the product has two forms, weights or tokens as the MMA's M operand; which one
        # runs follows the number of tiles, and both give the same bits
        try:
            forms = []
            for swapped in (False, True):
                ops.gemm_tc_set_many_token_path(swiglu_swapped=swapped)
                o = torch.full((T, ff), float("nan"), dtype=torch.bfloat16, device=DEV)
                ops.gemm_tc_swiglu(x, w, o)
                forms.append(o)
        finally:
            ops.gemm_tc_set_many_token_path()
        assert ops.gemm_tc_error() == 0
        assert torch.equal(forms[0], forms[1]) and torch.equal(forms[0], out)


def test_gemm_tcgen05_refuses_what_tma_cannot_address():
    ops = _ops()
    x, _ = _rand((4, 100), torch.bfloat16, 7)          # K = 100 is no multiple of 8
    w, _ = _rand((16, 100), torch.bfloat16, 8)
    assert not ops.gemm_tc_supported(x, w)
    with pytest.raises(ops.KernelError, match="TMA rules"):
        ops.gemm_tc(x, w)
    out = ops.linear(x, w)                               # the dispatcher takes the CUDA-core kernel instead
    ref = x.float() @ w.float().T
    assert torch.allclose(out.sum(0), ref, atol=1e-4)


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [96, 1000, 5120, 13000])
def test_add_rmsnorm(out_dtype, d):
    ops = _ops()
    T, S = 7, 3
    res, rr = _rand((T, d), torch.float32, 5)
    part, pr = _rand((S, T, d), torch.float32, 6, 0.3)
    bias, br = _rand((d,), torch.float32, 7, 0.1)
    w, wr = _rand((d,), torch.float32, 8)
    out = torch.empty((T, d), dtype=DT[out_dtype], device=DEV)
    res_in = res.clone()
    ops.add_rmsnorm(res, ops.Partials(part, bias), w, 1e-5, out)
    x = rr + (pr.sum(0) + br)
    np.testing.assert_allclose(res.cpu().numpy(), x, rtol=1e-6, atol=1e-6)
    ref = P.rms_norm(x, wr, 1e-5)
    tol = 1e-5 if out_dtype == "float32" else 1e-2
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol * np.abs(ref).max())
    # gathered rows: the residual stays untouched
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out2 = torch.empty((3, d), dtype=DT[out_dtype], device=DEV)
    res2 = res_in.clone()
    ops.add_rmsnorm(res2, ops.Partials(part, bias), w, 1e-5, out2, rows=rows)
    assert torch.equal(res2, res_in)
    assert torch.equal(out2[0], out[5]) and torch.equal(out2[1], out[0]) and torch.equal(out2[2], out[5])
    # no delta: a plain norm
    out3 = torch.empty((T, d), dtype=DT[out_dtype], device=DEV)
    ops.add_rmsnorm(res_in.clone(), None, w, 1e-5, out3)
    ref3 = P.rms_norm(rr, wr, 1e-5)
    np.testing.assert_allclose(out3.float().cpu().numpy(), ref3, rtol=tol, atol=tol * np.abs(ref3).max())


@pytest.mark.parametrize("d,S,with_bias", [(4096, 5, False), (2048, 1, True), (5120, 3, True), (6144, 2, False), (3000, 4, True),
                                          (8192, 1, False), (4096, 0, False)])
def test_add_rmsnorm_row_does_not_depend_on_the_batch(d, S, with_bias):
    """Few rows take the variant of the kernel that spreads a row over a whole block, many rows
    the one that gives a row to a warp (widths up to 6144) or to a narrow block; a row's bits -
    the norm in both storage types and the residual written back - are the same."""
    ops = _ops()
    res, _ = _rand((400, d), torch.float32, 21)
    w, _ = _rand((d,), torch.float32, 23)
    delta = one_delta = None
    if S:
        part, _ = _rand((S, 400, d), torch.float32, 22, 0.3)
        bias = _rand((d,), torch.float32, 24, 0.1)[0] if with_bias else None
        delta = ops.Partials(part, bias)
        one_delta = ops.Partials(part[:, 123:124].contiguous(), bias)
    for dt in (torch.float32, torch.bfloat16):
        many = torch.empty((400, d), dtype=dt, device=DEV)
        r1 = res.clone()
        ops.add_rmsnorm(r1, delta, w, 1e-6, many)
        one = torch.empty((1, d), dtype=dt, device=DEV)
        r2 = res[123:124].clone()
        ops.add_rmsnorm(r2, one_delta, w, 1e-6, one)
        assert torch.equal(one[0], many[123]) and torch.equal(r2[0], r1[123])
        rows = torch.arange(399, -1, -1, dtype=torch.int32, device=DEV)        # many gathered rows
        gathered = torch.empty((400, d), dtype=dt, device=DEV)
        ops.add_rmsnorm(res.clone(), delta, w, 1e-6, gathered, rows=rows)
        assert torch.equal(gathered[399 - 123], many[123])
        # the kernel with a warp a row, which is otherwise taken from 1,024 rows on and without slices
        ops.norm_set_warp_rows(100, with_slices=True)
        try:
            warp = torch.empty((400, d), dtype=dt, device=DEV)
            r3 = res.clone()
            ops.add_rmsnorm(r3, delta, w, 1e-6, warp)
        finally:
            ops.norm_set_warp_rows()
        assert torch.equal(warp, many) and torch.equal(r3, r1)


def test_add_rmsnorm_refuses_what_it_cannot_hold():
    ops = _ops()
    d = 60000
    with pytest.raises(ops.KernelError, match="exceeds"):
        ops.add_rmsnorm(torch.zeros((1, d), device=DEV), None, torch.ones(d, device=DEV), 1e-6,
                        torch.empty((1, d), device=DEV))


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("ff", [200, 777])
def test_swiglu(out_dtype, ff):
    ops = _ops()
    T, S = 5, 2
    part, pr = _rand((S, T, 2 * ff), torch.float32, 9, 2.0)
    out = torch.empty((T, ff), dtype=DT[out_dtype], device=DEV)
    ops.swiglu(ops.Partials(part), out)
    s = pr.sum(0)
    ref = P.silu(s[:, :ff]) * s[:, ff:]
    tol = 1e-6 if out_dtype == "float32" else 1e-2
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol * np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    ops = _ops()
    table, tr = _rand((301, 80), DT[dtype], 10)
    ids = torch.tensor([300, 0, 17, 17], dtype=torch.int32, device=DEV)
    out = torch.empty((4, 80), device=DEV)
    ops.embed(table, ids, out)
    np.testing.assert_array_equal(out.cpu().numpy(), tr[[300, 0, 17, 17]])


def _r16(a):
    """The values a bfloat16 tensor holds, as float32."""
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def _paged(dense_k, dense_v, page_size, num_pages, seed):
    """Scatter dense [L, nkv, hd] keys/values of ONE request into pages picked at random.
    Unused slots are filled with large numbers so that a read beyond the request shows."""
    L, nkv, hd = dense_k.shape
    nb = (L + page_size - 1) // page_size
    rng = np.random.default_rng(seed)
    pages = rng.permutation(num_pages)[:nb]
    kc = np.full((num_pages, nkv, page_size, hd), 1e4, dtype=np.float32)
    vc = np.full((num_pages, nkv, page_size, hd), -1e4, dtype=np.float32)
    for s in range(L):
        kc[pages[s // page_size], :, s % page_size, :] = dense_k[s]
        vc[pages[s // page_size], :, s % page_size, :] = dense_v[s]
    return kc, vc, pages.astype(np.int32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,hd,window,page", [(6, 2, 32, 0, 16), (5, 5, 48, 40, 16), (8, 1, 128, 0, 4),
                                                   (3, 3, 80, 7, 16), (4, 2, 16, 0, 1), (2, 1, 256, 100, 32)])
def test_attention_plain(dtype, nq, nkv, hd, window, page):
    ops = _ops()
    L = 150
    rng = np.random.default_rng(nq * 100 + hd)
    td = DT[dtype]

    def r16(a):
        return torch.from_numpy(a.astype(np.float32)).to(td).float().numpy()
    q = r16(rng.normal(size=(L, nq, hd)))
    k = r16(rng.normal(size=(L, nkv, hd)))
    v = r16(rng.normal(size=(L, nkv, hd)))
    ref = P.causal_attention(q, k, v, window)
    kc, vc, pages = _paged(k, v, page, 64 if page >= 4 else 200, 1)
    # queries: a portion of the request (positions 100..149) as the last step would hold
    lo = 100
    pos = torch.arange(lo, L, dtype=torch.int32, device=DEV)
    seq = torch.zeros(L - lo, dtype=torch.int32, device=DEV)
    table = torch.from_numpy(pages)[None, :].contiguous().to(DEV)
    out = torch.empty((L - lo, nq * hd), dtype=td, device=DEV)
    ops.attention_plain(torch.from_numpy(q[lo:].reshape(L - lo, -1)).to(td).to(DEV),
                        torch.from_numpy(kc).to(td).to(DEV), torch.from_numpy(vc).to(td).to(DEV),
                        pos, seq, table, page, out, nq, nkv, hd, window, 1.0 / math.sqrt(hd))
    tol = 2e-6 if dtype == "float32" else 1e-2
    np.testing.assert_allclose(out.float().cpu().numpy().reshape(L - lo, nq, hd), ref[lo:], rtol=0,
                               atol=tol * np.abs(ref).max())


def _mma_case(nq, nkv, hd, window, page, lens_new, lens_ctx, rows_per_tile, slices, slice_len, seed=0, tc=False, decode=False):
    """Several requests in one launch of the tensor-core kernel: request i holds lens_ctx[i]
    earlier tokens in its pages and lens_new[i] new ones whose queries run now."""
    ops = _ops()
    rng = np.random.default_rng(seed)
    G = nq // nkv

    def r16(a):
        return torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16).float().numpy()
    nseq = len(lens_new)
    total = [c + n for c, n in zip(lens_ctx, lens_new)]
    num_pages = sum((t + page - 1) // page for t in total) + 3
    perm = rng.permutation(num_pages)
    # slots no request owns: large values for the mma.sync kernel, NaN for the kernels that fetch
    # whole pages with TMA and have to keep what lies beyond a request's end out of the sums
    kc = np.full((num_pages, nkv, page, hd), np.nan if (tc or decode) else 1e4, dtype=np.float32)
    vc = np.full((num_pages, nkv, page, hd), np.nan if (tc or decode) else -1e4, dtype=np.float32)
    width = max((t + page - 1) // page for t in total)
    table = np.full((nseq, width), -1, dtype=np.int32)
    qs, refs, used = [], [], 0
    for i in range(nseq):
        L = total[i]
        q = r16(rng.normal(size=(L, nq, hd)))
        k = r16(rng.normal(size=(L, nkv, hd)))
        v = r16(rng.normal(size=(L, nkv, hd)))
        nb = (L + page - 1) // page
        table[i, :nb] = perm[used:used + nb]
        used += nb
        for s_ in range(L):
            kc[table[i, s_ // page], :, s_ % page] = k[s_]
            vc[table[i, s_ // page], :, s_ % page] = v[s_]
        refs.append(P.causal_attention(q, k, v, window)[lens_ctx[i]:])
        qs.append(q[lens_ctx[i]:])
    qcat = np.concatenate(qs).reshape(-1, nq * hd)
    T = qcat.shape[0]
    cu = np.concatenate([[0], np.cumsum(lens_new)]).astype(np.int32)
    tile_seq, tile_row0 = [], []
    for i in range(nseq):
        for r0 in range(0, lens_new[i] * G, rows_per_tile):
            tile_seq.append(i)
            tile_row0.append(r0)
    dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    if tc:
        ops.attention_tc(torch.from_numpy(qcat).to(torch.bfloat16).to(DEV), torch.from_numpy(kc).to(torch.bfloat16).to(DEV),
                         torch.from_numpy(vc).to(torch.bfloat16).to(DEV), out, dev(tile_seq), dev(tile_row0), dev(cu),
                         dev(total), dev(table), page, nq, nkv, hd, window, 1.0 / math.sqrt(hd),
                         slices if slices > 1 else 1, slice_len if slices > 1 else 1 << 30, rows_per_tile=rows_per_tile)
        assert ops.attention_tc_error() == 0
    elif decode:
        ops.attention_decode(torch.from_numpy(qcat).to(torch.bfloat16).to(DEV), torch.from_numpy(kc).to(torch.bfloat16).to(DEV),
                             torch.from_numpy(vc).to(torch.bfloat16).to(DEV), out, dev(tile_seq), dev(tile_row0), dev(cu),
                             dev(total), dev(table), page, nq, nkv, hd, window, 1.0 / math.sqrt(hd),
                             slices if slices > 1 else 1, slice_len if slices > 1 else 1 << 30)
        assert ops.attention_decode_error() == 0
    else:
        ops.attention_mma(torch.from_numpy(qcat).to(torch.bfloat16).to(DEV), torch.from_numpy(kc).to(torch.bfloat16).to(DEV),
                          torch.from_numpy(vc).to(torch.bfloat16).to(DEV), out, dev(tile_seq), dev(tile_row0), rows_per_tile,
                          dev(cu), dev(total), dev(table), page, nq, nkv, hd, window, 1.0 / math.sqrt(hd), slices, slice_len)
    ref = np.concatenate(refs).reshape(T, nq * hd)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, ref, rtol=0, atol=1e-2 * np.abs(ref).max())


@pytest.mark.parametrize("nq,nkv,hd,window,page", [(6, 2, 32, 0, 16), (5, 5, 48, 40, 16), (8, 1, 128, 0, 4),
                                                   (3, 3, 80, 7, 16), (4, 2, 16, 0, 1), (2, 1, 256, 100, 32),
                                                   (32, 8, 128, 0, 16), (40, 2, 64, 0, 16)])
def test_attention_mma_prompt_portions(nq, nkv, hd, window, page):
    """ROWS mode: portions of three requests, one of them from position 0, one deep into its context."""
    _mma_case(nq, nkv, hd, window, page, lens_new=(50, 3, 130), lens_ctx=(100, 0, 77),
              rows_per_tile=_ops().library().kestrel_attention_mma_rows_per_tile(hd),
              slices=1, slice_len=(1 << 30) // 64 * 64, seed=hd)


@pytest.mark.parametrize("nq,nkv,window,page", [(32, 8, 0, 16), (8, 1, 0, 8), (4, 4, 100, 16), (6, 2, 0, 128), (5, 1, 33, 32),
                                                (4, 2, 0, 256), (2, 2, 150, 64)])
@pytest.mark.parametrize("rows", [256, 128])
def test_attention_tcgen05_prompt_portions(nq, nkv, window, page, rows):
    """The tcgen05 kernel (head size 128): portions of three requests, one from position 0, one
    deep into its context, key tiles of 128 with the last one cut; two row tiles a CTA, or one."""
    _mma_case(nq, nkv, 128, window, page, lens_new=(50, 3, 300), lens_ctx=(100, 0, 77), rows_per_tile=rows,
              slices=1, slice_len=0, seed=nq, tc=True)


@pytest.mark.parametrize("nq,nkv,page,rows,slices,slice_len", [(8, 2, 16, 256, 3, 256), (4, 1, 32, 128, 5, 128), (6, 2, 128, 256, 2, 384)])
def test_attention_tcgen05_prompt_portions_in_slices(nq, nkv, page, rows, slices, slice_len):
    """Portions deep into their contexts with the key range cut into slices that are merged:
    some slices lie wholly before a portion, one holds its diagonal, later ones are empty for the
    shorter request."""
    _mma_case(nq, nkv, 128, 0, page, lens_new=(70, 130, 3), lens_ctx=(500, 90, 0), rows_per_tile=rows,
              slices=slices, slice_len=slice_len, seed=nq + 21, tc=True)


def test_attention_tcgen05_rescales_when_the_maximum_grows():
    """Scores that grow steeply along the keys: the running reference has to move (and the output
    accumulated so far be rescaled) at almost every key tile."""
    ops = _ops()
    L, nq, nkv, hd, page = 700, 4, 1, 128, 16
    rng = np.random.default_rng(1)
    k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.05
    k[:, :, 0] += np.linspace(0.0, 60.0, L)[:, None]            # q[0] = 1: the score rises by 60 / sqrt(128) * log2(e) * ... along the keys
    v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
    q = rng.normal(size=(L, nq, hd)).astype(np.float32) * 0.05
    q[:, :, 0] = 8.0
    r16 = lambda a: torch.from_numpy(a).to(torch.bfloat16).float().numpy()
    q, k, v = r16(q), r16(k), r16(v)
    ref = P.causal_attention(q, k, v, 0)
    kc, vc, pages = _paged(k, v, page, 50, 4)
    G = nq // nkv
    tiles = list(range(0, L * G, 256))
    dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    out = torch.empty((L, nq * hd), dtype=torch.bfloat16, device=DEV)
    ops.attention_tc(torch.from_numpy(q.reshape(L, -1)).to(torch.bfloat16).to(DEV),
                     torch.from_numpy(kc).to(torch.bfloat16).to(DEV), torch.from_numpy(vc).to(torch.bfloat16).to(DEV), out,
                     dev([0] * len(tiles)), dev(tiles), dev([0, L]), dev([L]), dev(pages[None, :]), page,
                     nq, nkv, hd, 0, 1.0 / math.sqrt(hd), rows_per_tile=256)
    assert ops.attention_tc_error() == 0
    got = out.float().cpu().numpy().reshape(L, nq, hd)
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, ref, rtol=0, atol=1e-2 * np.abs(ref).max())


@pytest.mark.parametrize("nq,nkv,window,page,slices,slice_len", [(32, 8, 0, 16, 1, 1 << 24), (32, 8, 0, 16, 3, 128), (8, 1, 0, 8, 2, 256),
                                                                 (4, 4, 100, 16, 1, 1 << 24), (16, 1, 0, 128, 4, 128)])
def test_attention_tcgen05_decode_tokens(nq, nkv, window, page, slices, slice_len):
    """The tcgen05 kernel on decode tokens: one new token for each of five requests of very
    different lengths, few rows per tile, the key range cut into slices that are merged."""
    _mma_case(nq, nkv, 128, window, page, lens_new=(1, 1, 1, 1, 1), lens_ctx=(0, 15, 64, 200, 330), rows_per_tile=16,
              slices=slices, slice_len=slice_len, seed=nq + 3, tc=True)


@pytest.mark.parametrize("far", [0, 15, 16, 127, 128, 255, 256])
def test_attention_tcgen05_finds_one_far_key(far):
    ops = _ops()
    L, nq, nkv, hd, page, n_new = 300, 4, 2, 128, 16, 40
    rng = np.random.default_rng(far)
    k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
    v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
    k[far] = 4.0
    q = np.full((n_new, nq, hd), 4.0, dtype=np.float32)
    kc, vc, pages = _paged(k, v, page, 40, 2)
    G = nq // nkv
    tiles = list(range(0, n_new * G, 128))
    dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    out = torch.empty((n_new, nq * hd), dtype=torch.bfloat16, device=DEV)
    ops.attention_tc(torch.from_numpy(q.reshape(n_new, -1)).to(torch.bfloat16).to(DEV),
                     torch.from_numpy(kc).to(torch.bfloat16).to(DEV), torch.from_numpy(vc).to(torch.bfloat16).to(DEV), out,
                     dev([0] * len(tiles)), dev(tiles), dev([0, n_new]), dev([L]), dev(pages[None, :]), page,
                     nq, nkv, hd, 0, 1.0 / math.sqrt(hd))
    assert ops.attention_tc_error() == 0
    got = out.float().cpu().numpy().reshape(n_new, nq, hd)
    want = np.stack([v[far, (h * nkv) // nq] for h in range(nq)])
    want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    for t in range(n_new):
        np.testing.assert_allclose(got[t], want, atol=2e-2)


@pytest.mark.parametrize("nq,nkv,hd,window,page,slices,slice_len", [
    (6, 2, 32, 0, 16, 1, 1 << 24), (32, 8, 128, 0, 16, 4, 128), (32, 8, 128, 0, 16, 3, 192), (5, 5, 48, 40, 16, 1, 1 << 24),
    (8, 1, 128, 0, 4, 7, 64), (3, 3, 80, 0, 16, 2, 256), (16, 1, 64, 0, 16, 6, 64), (2, 1, 256, 0, 32, 2, 192)])
def test_attention_mma_decode_tokens(nq, nkv, hd, window, page, slices, slice_len):
    """KEYS mode: one new token for each of five requests of very different lengths, the key
    range cut into slices; requests shorter than a slice leave later slices empty."""
    _mma_case(nq, nkv, hd, window, page, lens_new=(1, 1, 1, 1, 1), lens_ctx=(0, 15, 64, 200, 330), rows_per_tile=16,
              slices=slices, slice_len=slice_len, seed=hd + 1)


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 255, 256, 299])
@pytest.mark.parametrize("mode", ["decode", "decode-sliced", "portion"])
def test_attention_mma_finds_one_far_key(far, mode):
    """One key among 300 matches the query strongly; the output must be that key's value."""
    ops = _ops()
    L, nq, nkv, hd, page = 300, 4, 2, 64, 16
    rng = np.random.default_rng(far)
    k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
    v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
    k[far] = 4.0
    n_new = 1 if mode != "portion" else 40
    q = np.full((n_new, nq, hd), 4.0, dtype=np.float32)
    kc, vc, pages = _paged(k, v, page, 40, 2)
    if far >= L - n_new + 1 and mode == "portion":
        pytest.skip("the key lies inside the portion: earlier queries do not see it")
    G = nq // nkv
    rpt = 16 if mode != "portion" else ops.library().kestrel_attention_mma_rows_per_tile(hd)
    tiles = list(range(0, n_new * G, rpt))
    dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    out = torch.empty((n_new, nq * hd), dtype=torch.bfloat16, device=DEV)
    slices, slice_len = (5, 64) if mode == "decode-sliced" else (1, 1 << 24)
    ops.attention_mma(torch.from_numpy(q.reshape(n_new, -1)).to(torch.bfloat16).to(DEV),
                      torch.from_numpy(kc).to(torch.bfloat16).to(DEV), torch.from_numpy(vc).to(torch.bfloat16).to(DEV), out,
                      dev([0] * len(tiles)), dev(tiles), rpt, dev([0, n_new]), dev([L]), dev(pages[None, :]), page,
                      nq, nkv, hd, 0, 1.0 / math.sqrt(hd), slices, slice_len)
    got = out.float().cpu().numpy().reshape(n_new, nq, hd)
    want = np.stack([v[far, (h * nkv) // nq] for h in range(nq)])
    want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    for t in range(n_new):
        np.testing.assert_allclose(got[t], want, atol=2e-2)


@pytest.mark.parametrize("nq,nkv,hd,window,page,slices,slice_len", [
    (32, 8, 128, 0, 16, 1, 1 << 24), (32, 8, 128, 0, 16, 4, 128), (32, 8, 128, 0, 16, 3, 192), (8, 1, 128, 0, 8, 7, 64),
    (4, 4, 128, 100, 16, 1, 1 << 24), (16, 1, 64, 0, 16, 6, 64), (6, 2, 64, 0, 64, 2, 256), (5, 5, 64, 40, 32, 1, 1 << 24),
    (12, 3, 128, 0, 128, 3, 128), (2, 1, 128, 33, 256, 1, 1 << 24), (8, 2, 128, 0, 16, 8, 64), (8, 2, 128, 0, 16, 11, 64),
    (4, 1, 64, 0, 8, 9, 64)])
def test_attention_decode_tokens(nq, nkv, hd, window, page, slices, slice_len):
    """The decode kernel (TMA loader warp): one new token for each of five requests of very
    different lengths, the key range cut into slices; unused cache slots hold NaN."""
    _mma_case(nq, nkv, hd, window, page, lens_new=(1, 1, 1, 1, 1), lens_ctx=(0, 15, 64, 200, 330), rows_per_tile=16,
              slices=slices, slice_len=slice_len, seed=hd + 7, decode=True)


def test_attention_decode_merges_many_slices():
    """37 slices of 64 keys through scratch and the merge kernel (its unrolled loop and the
    remainder), some of them empty for the shorter requests."""
    _mma_case(8, 2, 128, 0, 16, lens_new=(1, 1, 2), lens_ctx=(2330, 70, 1000), rows_per_tile=16, slices=37, slice_len=64,
              seed=11, decode=True)
    _mma_case(6, 1, 64, 0, 32, lens_new=(1, 1), lens_ctx=(1100, 5), rows_per_tile=16, slices=9, slice_len=128,
              seed=12, decode=True)


def test_attention_decode_takes_short_portions_too():
    """Tiles of up to 16 rows need not be single tokens: portions of two to four tokens."""
    _mma_case(8, 2, 128, 0, 16, lens_new=(4, 2, 3), lens_ctx=(100, 0, 130), rows_per_tile=16, slices=1, slice_len=1 << 24,
              seed=3, decode=True)


@pytest.mark.parametrize("nq,nkv,hd,window,slices,slice_len", [(8, 2, 128, 0, 1, 1 << 24), (10, 2, 128, 0, 3, 128), (6, 2, 64, 40, 1, 1 << 24),
                                                               (3, 1, 128, 0, 5, 64)])
def test_attention_decode_takes_portions_of_many_tiles(nq, nkv, hd, window, slices, slice_len):
    """What the dispatcher hands this kernel since short portions near a request's start go to it:
    portions of tens of tokens cut into tiles of 16 rows, a token's heads split over two tiles
    where the group size does not divide 16, beside single tokens; tiles whose first row is not
    the request's first."""
    _mma_case(nq, nkv, hd, window, 16, lens_new=(40, 1, 100, 7, 1), lens_ctx=(100, 300, 0, 0, 9), rows_per_tile=16, slices=slices,
              slice_len=slice_len, seed=21, decode=True)


@pytest.mark.parametrize("far", [0, 15, 16, 63, 64, 255, 256, 299])
@pytest.mark.parametrize("sliced", [False, True])
def test_attention_decode_finds_one_far_key(far, sliced):
    """One key among 300 matches the query strongly; the output must be that key's value."""
    ops = _ops()
    L, nq, nkv, hd, page = 300, 4, 2, 64, 16
    rng = np.random.default_rng(far)
    k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
    v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
    k[far] = 4.0
    q = np.full((1, nq, hd), 4.0, dtype=np.float32)
    kc, vc, pages = _paged(k, v, page, 40, 2)
    dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    out = torch.empty((1, nq * hd), dtype=torch.bfloat16, device=DEV)
    slices, slice_len = (5, 64) if sliced else (1, 1 << 24)
    ops.attention_decode(torch.from_numpy(q.reshape(1, -1)).to(torch.bfloat16).to(DEV),
                         torch.from_numpy(kc).to(torch.bfloat16).to(DEV), torch.from_numpy(vc).to(torch.bfloat16).to(DEV), out,
                         dev([0]), dev([0]), dev([0, 1]), dev([L]), dev(pages[None, :]), page,
                         nq, nkv, hd, 0, 1.0 / math.sqrt(hd), slices, slice_len)
    assert ops.attention_decode_error() == 0
    got = out.float().cpu().numpy().reshape(nq, hd)
    want = np.stack([v[far, (h * nkv) // nq] for h in range(nq)])
    want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    np.testing.assert_allclose(got, want, atol=2e-2)


def test_attention_decode_window_edge():
    """The key at distance window - 1 is the last one seen; pages behind the window are gone (-1)."""
    ops = _ops()
    L, nq, nkv, hd, page, window = 200, 2, 2, 64, 16, 48
    for offset, inside in ((window - 1, True), (window, False)):
        rng = np.random.default_rng(5)
        k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
        v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
        q = np.full((1, nq, hd), 4.0, dtype=np.float32)
        spot = L - 1 - offset
        k[spot] = 4.0
        kc, vc, pages = _paged(k, v, page, 40, 3)
        pages = pages.copy()
        pages[: (L - window) // page] = -1            # pages behind the window were given back
        dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
        out = torch.empty((1, nq * hd), dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(torch.from_numpy(q.reshape(1, -1)).to(torch.bfloat16).to(DEV),
                             torch.from_numpy(kc).to(torch.bfloat16).to(DEV), torch.from_numpy(vc).to(torch.bfloat16).to(DEV),
                             out, dev([0]), dev([0]), dev([0, 1]), dev([L]), dev(pages[None, :]), page, nq, nkv, hd,
                             window, 1.0 / math.sqrt(hd))
        assert ops.attention_decode_error() == 0
        got = out.float().cpu().numpy().reshape(nq, hd)
        close = np.abs(got - v[spot]).max() < 3e-2
        assert close == inside, f"key at distance {offset} (window {window}): inside={inside}, output follows it={close}"


def test_attention_decode_refuses_what_its_boxes_do_not_fit():
    ops = _ops()
    assert ops.attention_decode_supported(128, 16) and ops.attention_decode_supported(64, 128)
    assert not ops.attention_decode_supported(128, 4) and not ops.attention_decode_supported(128, 48)
    assert not ops.attention_decode_supported(80, 16) and not ops.attention_decode_supported(256, 16)
    q = torch.zeros((1, 80), dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros((2, 1, 16, 80), dtype=torch.bfloat16, device=DEV)
    i = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="head size"):
        ops.attention_decode(q, cache, cache, torch.empty_like(q), i[:1], i[:1], i, i[:1], i[None, :1], 16, 1, 1, 80, 0, 1.0)


def test_attention_mma_window_edge():
    ops = _ops()
    L, nq, nkv, hd, page, window = 200, 2, 2, 32, 16, 48
    for offset, inside in ((window - 1, True), (window, False)):
        rng = np.random.default_rng(5)
        k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
        v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
        q = np.full((1, nq, hd), 4.0, dtype=np.float32)
        spot = L - 1 - offset
        k[spot] = 4.0
        kc, vc, pages = _paged(k, v, page, 40, 3)
        pages = pages.copy()
        pages[: (L - window) // page] = -1            # pages behind the window were given back
        dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
        out = torch.empty((1, nq * hd), dtype=torch.bfloat16, device=DEV)
        ops.attention_mma(torch.from_numpy(q.reshape(1, -1)).to(torch.bfloat16).to(DEV),
                          torch.from_numpy(kc).to(torch.bfloat16).to(DEV), torch.from_numpy(vc).to(torch.bfloat16).to(DEV),
                          out, dev([0]), dev([0]), 16, dev([0, 1]), dev([L]), dev(pages[None, :]), page, nq, nkv, hd,
                          window, 1.0 / math.sqrt(hd))
        got = out.float().cpu().numpy().reshape(nq, hd)
        close = np.abs(got - v[spot]).max() < 3e-2
        assert close == inside, f"key at distance {offset} (window {window}): inside={inside}, output follows it={close}"


@pytest.mark.parametrize("rows", [128, 256])
def test_attention_tcgen05_window_edge(rows):
    """The prompt-portion kernel at a window's edge: for the query in the LAST row of a row tile,
    one key stands out; at distance window - 1 the output follows it, at distance window it must
    not.  Pages that lie behind the window for every query of the portion are gone (-1)."""
    ops = _ops()
    ctx, new, nq, nkv, hd, page, window = 128, 272, 2, 2, 128, 16, 48
    L = ctx + new
    probe = rows - 1                                   # row of the portion under test (one row a token: nq == nkv)
    for offset, inside in ((window - 1, True), (window, False)):
        rng = np.random.default_rng(7)
        k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
        v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
        q = rng.normal(size=(new, nq, hd)).astype(np.float32) * 0.1
        q[probe] = 4.0
        spot = ctx + probe - offset
        k[spot] = 4.0
        kc, vc, pages = _paged(k, v, page, 40, 3)
        pages = pages.copy()
        pages[: (ctx - window + 1) // page] = -1      # behind the window of the portion's first query
        dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
        tiles = list(range(0, new * (nq // nkv), rows))
        out = torch.full((new, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_tc(torch.from_numpy(q.reshape(new, -1)).to(torch.bfloat16).to(DEV),
                         torch.from_numpy(kc).to(torch.bfloat16).to(DEV), torch.from_numpy(vc).to(torch.bfloat16).to(DEV),
                         out, dev([0] * len(tiles)), dev(tiles), dev([0, new]), dev([L]), dev(pages[None, :]), page, nq, nkv, hd,
                         window, 1.0 / math.sqrt(hd), rows_per_tile=rows)
        assert ops.attention_tc_error() == 0
        got = out.float().cpu().numpy().reshape(new, nq, hd)
        assert np.isfinite(got).all()
        close = np.abs(got[probe] - v[spot]).max() < 3e-2
        assert close == inside, f"rows {rows}: key at distance {offset} (window {window}): inside={inside}, output follows it={close}"
        # every other row agrees with the plain attention of the window
        ref = P.causal_attention(np.concatenate([np.zeros((ctx, nq, hd), np.float32), _r16(q)]), _r16(k), _r16(v), window)[ctx:]
        np.testing.assert_allclose(got, ref, rtol=0, atol=2e-2 * np.abs(ref).max())


def test_attention_mma_refuses_odd_head_sizes():
    ops = _ops()
    z = torch.zeros((1, 12), dtype=torch.bfloat16, device=DEV)
    i = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.attention_mma(z, z, z, torch.empty_like(z), i[:1], i[:1], 16, i, i[:1], i[None, :1], 4, 1, 1, 12, 0, 1.0)


def test_attention_tcgen05_refuses_pages_its_boxes_do_not_fit():
    """Pages of 4 or 48 keys do not tile the kernel's 128-key TMA boxes; the dispatcher sends such
    caches to the mma.sync kernel and the kernel itself says no."""
    ops = _ops()
    assert ops.attention_tc_supported(128, 16) and ops.attention_tc_supported(128, 256)
    assert not ops.attention_tc_supported(128, 4) and not ops.attention_tc_supported(128, 48)
    assert not ops.attention_tc_supported(64, 16)
    q = torch.zeros((1, 128), dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros((2, 1, 4, 128), dtype=torch.bfloat16, device=DEV)
    i = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="page size"):
        ops.attention_tc(q, cache, cache, torch.empty_like(q), i[:1], i[:1], i, i[:1], i[None, :1], 4, 1, 1, 128, 0, 1.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 15, 16, 255, 256, 299])
def test_attention_finds_one_far_key(dtype, far):
    """One key among 300 matches the query strongly; the output must be that key's value.
    Random keys alone would hide a kernel that skips a page edge or the first position."""
    ops = _ops()
    L, nq, nkv, hd, page = 300, 4, 2, 64, 16
    rng = np.random.default_rng(far)
    k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
    v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
    q = rng.normal(size=(1, nq, hd)).astype(np.float32) * 0.1
    direction = np.ones(hd, dtype=np.float32)
    k[far, :, :] = 4.0 * direction
    q[0, :, :] = 4.0 * direction             # score 16*64/8 = 128 against ~0 elsewhere
    td = DT[dtype]
    kc, vc, pages = _paged(k, v, page, 40, 2)
    out = torch.empty((1, nq * hd), dtype=td, device=DEV)
    ops.attention_plain(torch.from_numpy(q.reshape(1, -1)).to(td).to(DEV), torch.from_numpy(kc).to(td).to(DEV),
                        torch.from_numpy(vc).to(td).to(DEV), torch.tensor([L - 1], dtype=torch.int32, device=DEV),
                        torch.zeros(1, dtype=torch.int32, device=DEV),
                        torch.from_numpy(pages)[None, :].contiguous().to(DEV), page, out, nq, nkv, hd, 0,
                        1.0 / math.sqrt(hd))
    got = out.float().cpu().numpy().reshape(nq, hd)
    want = np.stack([v[far, (h * nkv) // nq] for h in range(nq)])
    np.testing.assert_allclose(got, torch.from_numpy(want).to(td).float().numpy(), atol=2e-2 if dtype == "bfloat16" else 1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_window_edge(dtype):
    """A strongly matching key just inside the window decides the output; the same key one
    position further back, just outside, must have no influence at all."""
    ops = _ops()
    L, nq, nkv, hd, page, window = 200, 2, 2, 32, 16, 48
    td = DT[dtype]
    for offset, inside in ((window - 1, True), (window, False)):
        rng = np.random.default_rng(5)
        k = rng.normal(size=(L, nkv, hd)).astype(np.float32) * 0.1
        v = rng.normal(size=(L, nkv, hd)).astype(np.float32)
        q = np.full((1, nq, hd), 4.0, dtype=np.float32)
        spot = L - 1 - offset
        k[spot] = 4.0
        kc, vc, pages = _paged(k, v, page, 40, 3)
        out = torch.empty((1, nq * hd), dtype=td, device=DEV)
        ops.attention_plain(torch.from_numpy(q.reshape(1, -1)).to(td).to(DEV), torch.from_numpy(kc).to(td).to(DEV),
                            torch.from_numpy(vc).to(td).to(DEV), torch.tensor([L - 1], dtype=torch.int32, device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV),
                            torch.from_numpy(pages)[None, :].contiguous().to(DEV), page, out, nq, nkv, hd, window,
                            1.0 / math.sqrt(hd))
        got = out.float().cpu().numpy().reshape(nq, hd)
        close = np.abs(got - v[spot]).max() < 3e-2
        assert close == inside, f"key at distance {offset} (window {window}): inside={inside}, output follows it={close}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,hd,rot,bias,norm", [(6, 2, 32, 32, True, True), (5, 5, 48, 48, False, True),
                                                     (3, 1, 80, 40, True, False), (8, 2, 128, 128, False, True), (6, 3, 128, 128, True, True), (9, 1, 128, 128, True, False), (4, 4, 128, 64, False, True),
                                                     (2, 2, 16, 0, False, False)])
def test_attn_prepare(dtype, nq, nkv, hd, rot, bias, norm):
    ops = _ops()
    td = DT[dtype]
    T, S, page, num_pages = 9, 2, 4, 12
    width = (nq + 2 * nkv) * hd
    part, pr = _rand((S, T, width), torch.float32, 11)
    b, br = _rand((width,), torch.float32, 12, 0.2) if bias else (None, None)
    qw, qwr = _rand((hd,), torch.float32, 13) if norm else (None, None)
    kw, kwr = _rand((hd,), torch.float32, 14) if norm else (None, None)
    theta = 1e6
    inv = (np.float32(1) / np.power(np.float32(theta), np.arange(rot // 2, dtype=np.float32) / np.float32(max(rot // 2, 1)))).astype(np.float32)
    # two requests: tokens 0..4 are positions 7..11 of request 0, tokens 5..8 positions 0..3 of request 1
    positions = np.array([7, 8, 9, 10, 11, 0, 1, 2, 3], dtype=np.int32)
    seqs = np.array([0, 0, 0, 0, 0, 1, 1, 1, 1], dtype=np.int32)
    table = np.array([[5, 9, 2, -1], [7, -1, -1, -1]], dtype=np.int32)
    kc = torch.zeros((num_pages, nkv, page, hd), dtype=td, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty((T, nq * hd), dtype=td, device=DEV)
    ops.attn_prepare(ops.Partials(part, b), qw, kw, 1e-5, torch.from_numpy(inv).to(DEV) if rot else None, rot,
                     torch.from_numpy(positions).to(DEV), torch.from_numpy(seqs).to(DEV),
                     torch.from_numpy(table).to(DEV), page, kc, vc, q_out, nq, nkv, hd)
    x = pr.sum(0) + (br if bias else 0)
    q = x[:, :nq * hd].reshape(T, nq, hd)
    k = x[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
    v = x[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
    if norm:
        q, k = P.head_rms_norm(q, qwr, 1e-5), P.head_rms_norm(k, kwr, 1e-5)
    if rot:
        ang = positions.astype(np.float32)[:, None] * inv[None, :]
        cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
        q = np.concatenate([P.rope(q[..., :rot], cos, sin), q[..., rot:]], -1)
        k = np.concatenate([P.rope(k[..., :rot], cos, sin), k[..., rot:]], -1)
    tol = 1e-5 if dtype == "float32" else 1e-2
    np.testing.assert_allclose(q_out.float().cpu().numpy().reshape(T, nq, hd), q, rtol=tol, atol=tol * 4)
    kcn, vcn = kc.float().cpu().numpy(), vc.float().cpu().numpy()
    for t in range(T):
        pg = table[seqs[t], positions[t] // page]
        np.testing.assert_allclose(kcn[pg, :, positions[t] % page, :], k[t], rtol=tol, atol=tol * 4)
        np.testing.assert_allclose(vcn[pg, :, positions[t] % page, :], v[t], rtol=tol, atol=tol * 4)
    written = {(table[seqs[t], positions[t] // page], positions[t] % page) for t in range(T)}
    for pg in range(num_pages):
        for sl in range(page):
            if (pg, sl) not in written:
                assert not kcn[pg, :, sl].any() and not vcn[pg, :, sl].any(), f"page {pg} slot {sl} was written"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,S,bias,interleaved", [(32, 8, 1, False, False), (5, 1, 3, True, False), (6, 2, 2, False, True)])
def test_attn_prepare_token_does_not_depend_on_the_batch(dtype, nq, nkv, S, bias, interleaved):
    """Head size 128 (the kernel of its own) and the general kernel with another rotation: a
    token's queries, keys and values are the same bits in a step of 200 tokens and in a step of
    3, and agree with the plain parts."""
    ops = _ops()
    td = DT[dtype]
    hd, page, T = 128, 16, 200
    width = (nq + 2 * nkv) * hd
    part, pr = _rand((S, T, width), torch.float32, 31)
    b, br = _rand((width,), torch.float32, 32, 0.2) if bias else (None, None)
    qw, qwr = _rand((hd,), torch.float32, 33)
    kw, kwr = _rand((hd,), torch.float32, 34)
    inv = (np.float32(1) / np.power(np.float32(1e6), np.arange(hd // 2, dtype=np.float32) / np.float32(hd // 2))).astype(np.float32)
    inv_d = torch.from_numpy(inv).to(DEV)
    positions = (np.arange(T, dtype=np.int32) * 37) % 3000
    pages = 3000 // page + 1
    table = torch.from_numpy(np.random.default_rng(1).permutation(pages).astype(np.int32)[None, :]).to(DEV)
    mode = 1 if interleaved else 0

    def run(tokens):
        n = len(tokens)
        kc = torch.zeros((pages, nkv, page, hd), dtype=td, device=DEV)
        vc = torch.zeros_like(kc)
        q = torch.empty((n, nq * hd), dtype=td, device=DEV)
        idx = torch.tensor(tokens, device=DEV)
        ops.attn_prepare(ops.Partials(part[:, idx].contiguous(), b), qw, kw, 1e-6, inv_d, hd,
                         torch.from_numpy(positions[tokens]).to(DEV), torch.zeros(n, dtype=torch.int32, device=DEV), table, page,
                         kc, vc, q, nq, nkv, hd, rot_mode=mode)
        return q, kc, vc

    q_all, k_all, v_all = run(list(range(T)))
    few = [150, 7, 63]
    q_few, k_few, v_few = run(few)
    tab = table[0].cpu().numpy()
    for i, t in enumerate(few):
        assert torch.equal(q_few[i], q_all[t])
        pg, sl = tab[positions[t] // page], positions[t] % page
        assert torch.equal(k_few[pg, :, sl], k_all[pg, :, sl]) and torch.equal(v_few[pg, :, sl], v_all[pg, :, sl])
    # and against the plain parts
    x = pr.sum(0) + (br if bias else 0)
    qr = P.head_rms_norm(x[:, :nq * hd].reshape(T, nq, hd), qwr, 1e-6)
    ang = positions.astype(np.float32)[:, None] * inv[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    if interleaved:
        ref = qr.copy()
        a0, b0 = qr[..., 0::2], qr[..., 1::2]
        ref[..., 0::2] = a0 * cos[:, None, :] - b0 * sin[:, None, :]
        ref[..., 1::2] = b0 * cos[:, None, :] + a0 * sin[:, None, :]
    else:
        ref = P.rope(qr, cos, sin)
    tol = 1e-5 if dtype == "float32" else 1e-2
    np.testing.assert_allclose(q_all.float().cpu().numpy().reshape(T, nq, hd), ref, rtol=tol, atol=tol * 4)


@pytest.mark.parametrize("nq,nkv,bias,norm,T,K,write_kv", [(5, 2, True, True, 300, 192, True), (32, 8, False, True, 1100, 256, True),
                                                           (3, 1, True, False, 513, 128, True), (4, 2, False, True, 257, 320, False)])
def test_qkv_product_with_prepare_in_its_epilogue(nq, nkv, bias, norm, T, K, write_kv):
    """The q, k, v product of many tokens at head size 128 with bias, head norms, rotation and the
    cache write in its epilogue, against the plain parts and against the two kernels it
    replaces; head counts that leave a tile half empty, token counts that are no multiple of a
    tile, two requests at far positions, pages in random order."""
    ops = _ops()
    hd, page = 128, 16
    heads = nq + 2 * nkv
    x, xr = _rand((T, K), torch.bfloat16, 41)
    w, wr = _rand((heads * hd, K), torch.bfloat16, 42, K ** -0.5)
    b, br = _rand((heads * hd,), torch.float32, 43, 0.2) if bias else (None, None)
    qw, qwr = _rand((hd,), torch.float32, 44) if norm else (None, None)
    kw, kwr = _rand((hd,), torch.float32, 45) if norm else (None, None)
    inv = (np.float32(1) / np.power(np.float32(1e6), np.arange(hd // 2, dtype=np.float32) / np.float32(hd // 2))).astype(np.float32)
    inv_d = torch.from_numpy(inv).to(DEV)
    first = T // 3
    positions = np.concatenate([np.arange(first) + 30000, np.arange(T - first) + 5]).astype(np.int32)
    seqs = np.concatenate([np.zeros(first), np.ones(T - first)]).astype(np.int32)
    width = (30000 + T) // page + 1
    num_pages = 2 * (T // page + 3)
    order = np.random.default_rng(2).permutation(num_pages).astype(np.int32)
    table = np.full((2, width), -1, dtype=np.int32)
    used = 0
    for r, (lo, n) in enumerate(((30000, first), (5, T - first))):
        for col in range(lo // page, (lo + n - 1) // page + 1):
            table[r, col] = order[used]
            used += 1
    args = dict(q_norm_w=qw, k_norm_w=kw, norm_eps=1e-6, inv_freq=inv_d, rotary_dim=hd, positions=torch.from_numpy(positions).to(DEV),
                seq_of_token=torch.from_numpy(seqs).to(DEV), block_table=torch.from_numpy(table).to(DEV), page_size=page, nq=nq,
                nkv=nkv, hd=hd, write_kv=write_kv)

    def caches():
        kc = torch.zeros((num_pages, nkv, page, hd), dtype=torch.bfloat16, device=DEV)
        return kc, torch.zeros_like(kc), torch.empty((T, nq * hd), dtype=torch.bfloat16, device=DEV)

    kc, vc, q_out = caches()
    assert ops.qkv_prepare_fused(x, w, b, k_cache=kc, v_cache=vc, q_out=q_out, **args)
    assert ops.gemm_tc_error() == 0
    kc2, vc2, q2 = caches()
    ops.attn_prepare(ops.Partials(ops.linear(x, w), b), k_cache=kc2, v_cache=vc2, q_out=q2, **args)
    # the plain parts, from the same bfloat16 operands
    y = (xr.astype(np.float64) @ wr.astype(np.float64).T).astype(np.float32) + (br if bias else 0)
    q = y[:, :nq * hd].reshape(T, nq, hd)
    k = y[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
    v = y[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
    if norm:
        q, k = P.head_rms_norm(q, qwr, 1e-6), P.head_rms_norm(k, kwr, 1e-6)
    ang = positions.astype(np.float32)[:, None] * inv[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    q, k = P.rope(q, cos, sin), P.rope(k, cos, sin)
    tol = 1e-2
    np.testing.assert_allclose(q_out.float().cpu().numpy().reshape(T, nq, hd), q, rtol=tol, atol=tol * 4)
    np.testing.assert_allclose(q_out.float().cpu().numpy(), q2.float().cpu().numpy(), rtol=tol, atol=tol * 4)
    kcn, vcn = kc.float().cpu().numpy(), vc.float().cpu().numpy()
    if not write_kv:
        assert not kcn.any() and not vcn.any()
        return
    written = np.zeros((num_pages, page), dtype=bool)
    for t in range(T):
        pg, sl = table[seqs[t], positions[t] // page], positions[t] % page
        written[pg, sl] = True
        np.testing.assert_allclose(kcn[pg, :, sl, :], k[t], rtol=tol, atol=tol * 4)
        np.testing.assert_allclose(vcn[pg, :, sl, :], v[t], rtol=tol, atol=tol * 4)
    assert not kcn.transpose(0, 2, 1, 3)[~written].any() and not vcn.transpose(0, 2, 1, 3)[~written].any(), \
        "a cache row of no token was written"
    np.testing.assert_allclose(kcn, kc2.float().cpu().numpy(), rtol=tol, atol=tol * 4)


def test_qkv_product_with_prepare_leaves_other_cases_alone():
    """Few tokens, float32, another head size, a partial rotation: nothing is launched and the
    caller is told so."""
    ops = _ops()
    i32 = torch.zeros(300, dtype=torch.int32, device=DEV)
    inv = torch.ones(64, device=DEV)

    def tried(T, hd, dtype, rot):
        x = torch.zeros((T, 128), dtype=dtype, device=DEV)
        w = torch.zeros((3 * hd, 128), dtype=dtype, device=DEV)
        kc = torch.zeros((32, 1, 16, hd), dtype=dtype, device=DEV)
        return ops.qkv_prepare_fused(x, w, None, None, None, 0.0, inv[:max(rot // 2, 1)], rot, i32[:T], i32[:T], i32[None, :32].contiguous(), 16,
                                     kc, kc.clone(), torch.empty((T, hd), dtype=dtype, device=DEV), 1, 1, hd)

    assert not tried(100, 128, torch.bfloat16, 128)
    assert not tried(300, 64, torch.bfloat16, 64)
    assert not tried(300, 128, torch.bfloat16, 64)
    assert not tried(300, 128, torch.float32, 128)
    assert tried(300, 128, torch.bfloat16, 128)


def test_attn_prepare_refuses_odd_sizes():
    ops = _ops()
    z = torch.zeros((1, 1, (1 + 2) * 600), device=DEV)
    i32 = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(ops.KernelError, match="head size"):
        ops.attn_prepare(ops.Partials(z), None, None, 0.0, None, 0, i32, i32, i32[None], 4,
                         torch.zeros(4, device=DEV), torch.zeros(4, device=DEV), torch.empty((1, 600), device=DEV), 1, 1, 600)


def test_argmax_first_maximum_wins():
    ops = _ops()
    V = 151936 + 7
    l = torch.randn((5, V), device=DEV)
    l[0, 77] = 50.0; l[0, 90000] = 50.0
    l[1, V - 1] = 60.0
    l[2, 0] = 70.0
    l[3, :] = -3.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(l, out)
    got = out.cpu().tolist()
    assert got[:4] == [77, V - 1, 0, 0] and got[4] == int(l[4].argmax())


@pytest.mark.parametrize("V,cluster,reps", [(509, True, 3), (509, False, 3), (9001, True, 2), (40000, True, 2), (151936, True, 3),
                                            (151936, False, 1), (262144, True, 1)])
def test_sample_against_plain_sampler(V, cluster, reps):
    """Temperature, top-k, min-p and top-p against the plain sampler, on the kernel that keeps a
    row in the shared memory of a cluster (1, 2 and 8 CTAs; with and without room for the
    probabilities) and on the one-block kernel over global memory.  Rows are flat (random
    logits) or peaked (a few tokens far above the rest, as a trained model gives them)."""
    ops = _ops()
    from kestrel_llm_b200.sampling import uniform_for
    rng = np.random.default_rng(V)
    rows = [(0.8, 0, 0.0, 1.0), (1.0, 20, 0.0, 1.0), (0.7, 0, 0.05, 1.0), (1.3, 0, 0.0, 0.9), (0.9, 50, 0.02, 0.8),
            (0.0, 0, 0.0, 1.0), (1.0, 0, 0.0, 0.0), (2.0, 1, 0.0, 1.0), (0.5, 0, 0.0, 0.3), (1.0, 3, 0.0, 0.999)] * reps
    R = len(rows)
    logits = (rng.normal(size=(R, V)) * 3).astype(np.float32)
    for r in range(1, R, 2):            # every other row peaked: five tokens 8 to 12 above the rest
        logits[r, rng.choice(V, size=5, replace=False)] += rng.uniform(8, 12, size=5).astype(np.float32)
    u = np.array([uniform_for(123, i) for i in range(R)], dtype=np.float32)
    assert ((u > 0) & (u <= 1)).all()
    dev = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)
    out = torch.full((R,), -7, dtype=torch.int32, device=DEV)
    ops.sample_set_cluster(cluster)
    try:
        ops.sample(torch.from_numpy(logits).to(DEV), dev([r[0] for r in rows], torch.float32),
                   dev([r[1] for r in rows], torch.int32), dev([r[3] for r in rows], torch.float32),
                   dev([r[2] for r in rows], torch.float32), torch.from_numpy(u).to(DEV), out)
        got = out.cpu().tolist()
    finally:
        ops.sample_set_cluster(True)
    for r, (temp, tk, mp, tp) in enumerate(rows):
        assert 0 <= got[r] < V, f"row {r}: no token written ({got[r]})"
        if temp <= 0 or tp <= 0:
            assert got[r] == P.greedy(logits[r])
            continue
        p = P.sample_probs(logits[r], temp, tk, mp, tp)
        assert p[got[r]] > 0, f"row {r}: token {got[r]} was filtered out by the plain sampler"
        want = P.sample_from(p, float(u[r]))
        if got[r] != want:
            # sums run in another order on the device: accept a neighbour only if u*total lies
            # within rounding of the boundary between the two
            c = np.cumsum(p.astype(np.float64))
            target = float(u[r]) * c[-1]
            edge = c[min(got[r], want)]
            assert abs(edge - target) <= 1e-5 * c[-1], f"row {r}: got {got[r]}, plain {want}"
    # a draw depends on (seed, index) only
    assert uniform_for(5, 3) == uniform_for(5, 3) and uniform_for(5, 3) != uniform_for(5, 4) != uniform_for(6, 4)


def test_repetition_penalty_against_the_plain_one():
    """Rows with and without a penalty, windows shorter and longer than what was generated, a
    token twice in the window (penalised twice), negative and positive logits, ids outside the
    vocabulary skipped."""
    ops = _ops()
    V, W = 5003, 64
    rng = np.random.default_rng(8)
    logits = (rng.normal(size=(5, V)) * 4).astype(np.float32)
    gens = [list(rng.integers(0, V, size=50)), [7, 7, 9, 7], [], list(rng.integers(0, V, size=10)), [3, V + 5, -2, 4]]
    gens[0][-3] = gens[0][-1]
    pens, wins = [1.3, 2.0, 1.5, 1.0, 1.1], [32, 64, 8, 5, 64]
    hist = np.full((5, W), -1, dtype=np.int32)
    counts = np.zeros(5, dtype=np.int32)
    for r, (g, w) in enumerate(zip(gens, wins)):
        last = [int(x) for x in g[-w:]][::-1]
        hist[r, :len(last)] = last
        counts[r] = len(last)
    dev_logits = torch.from_numpy(logits).to(DEV)
    ops.repetition_penalty(dev_logits, torch.from_numpy(hist).to(DEV), torch.from_numpy(counts).to(DEV),
                           torch.tensor(pens, dtype=torch.float32, device=DEV))
    got = dev_logits.cpu().numpy()
    for r in range(5):
        want = P.repetition_penalty(logits[r], [int(x) for x in gens[r]], pens[r], wins[r])
        np.testing.assert_array_equal(got[r], want)
    assert (got[3] == logits[3]).all() and (got[1] != logits[1]).sum() == 2


@pytest.mark.parametrize("V", [1000, 151936])
def test_sample_odd_rows(V):
    """Rows that a sampler must not stumble over: all logits equal (every token kept, the draw
    walks the indices), -inf almost everywhere, NaN everywhere (first maximum = index 0 as a
    strict scan gives), top-k beyond ties at the cut; and a row's token does not depend on the
    rows beside it."""
    ops = _ops()
    dev = lambda a, dt: torch.tensor(a, dtype=dt, device=DEV)
    logits = np.zeros((5, V), dtype=np.float32)
    logits[1, :] = -np.inf; logits[1, V - 3] = 1.0; logits[1, 7] = 0.5
    logits[2, :] = np.nan
    logits[3, :] = -1.0; logits[3, [5, V // 2, V - 1]] = 2.0                 # three equal maxima, top-k 2: all three stay
    logits[4] = np.random.default_rng(1).normal(size=V).astype(np.float32) * 4
    temps, tks, tps, mps = [1.0, 1.0, 1.0, 1.0, 0.7], [0, 0, 0, 2, 40], [1.0, 0.95, 0.9, 1.0, 0.9], [0.0, 0.0, 0.0, 0.0, 0.01]
    u = np.array([0.5, 0.9, 0.3, 0.99, 0.42], dtype=np.float32)
    out = torch.full((5,), -7, dtype=torch.int32, device=DEV)
    args = lambda sel: (torch.from_numpy(logits[sel]).to(DEV), dev([temps[i] for i in sel], torch.float32), dev([tks[i] for i in sel], torch.int32),
                        dev([tps[i] for i in sel], torch.float32), dev([mps[i] for i in sel], torch.float32), torch.from_numpy(u[sel]).to(DEV))
    ops.sample(*args([0, 1, 2, 3, 4]), out)
    got = out.cpu().tolist()
    assert abs(got[0] - (V // 2 - 1)) <= 1                      # uniform: the index at half the mass
    assert got[1] == V - 3                                      # p(7) = 0.38, p(V - 3) = 0.62; u = 0.9 lands in the latter
    assert got[2] == 0
    assert got[3] == V - 1                                      # three tokens of 1/3 each (all of the tie stay); u = 0.99: the last
    alone = torch.full((1,), -7, dtype=torch.int32, device=DEV)
    ops.sample(*args([4]), alone)
    assert int(alone[0]) == got[4]
    p = P.sample_probs(logits[4], 0.7, 40, 0.01, 0.9)
    assert p[got[4]] > 0


def test_a_wait_that_nothing_ends_gives_up():
    """The tensor-core kernels' mbarrier waits are bounded: on a barrier that nobody completes the
    wait returns after its limit (seconds, not minutes), the kernel reports it, and the
    device goes on working - here the next product is right."""
    ops = _ops()
    gave_up, ms = ops.wait_probe()
    assert gave_up and 1.0 < ms < 10000.0, f"gave up: {gave_up}, after {ms:.0f} ms"
    print(f"the wait gave up after {ms:.0f} ms")
    x, xr = _rand((8, 256), torch.bfloat16, 31)
    w, wr = _rand((128, 256), torch.bfloat16, 32, 0.05)
    got = ops.gemm_tc(x, w).sum(0).cpu().numpy()
    ops.raise_on_kernel_error()
    np.testing.assert_allclose(got, xr.astype(np.float64) @ wr.astype(np.float64).T, rtol=0, atol=1e-3)


def test_kernels_refuse_host_tensors():
    ops = _ops()
    with pytest.raises(ops.KernelError, match="CUDA device only"):
        ops.gemm_plain(torch.zeros((2, 2)), torch.zeros((2, 2)), torch.zeros((2, 2)))
