"""The plain implementation against the reference's own compiled float32 forward pass.

tests/golden/reference_logits_<name>.npy were written by tests/golden/make_reference_golden.py,
which builds six of the reference's C files on the CPU and runs st_qwen_model_forward token by
token on tests/golden/tiny_model_<name>: two configurations that differ in every size, 100
tokens each, so that the reference's attention for fewer than 64 keys and its tiled kernel for
more are both the oracle.  This test needs neither the reference nor a GPU."""
import json
import os

import numpy as np
import pytest

import plain_qwen3 as P

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_matches_reference_code(name):
    cfg, W = P.read_model(os.path.join(GOLD, f"tiny_model_{name}"))
    tokens = json.load(open(os.path.join(GOLD, f"reference_tokens_{name}.json")))
    ref = np.load(os.path.join(GOLD, f"reference_logits_{name}.npy"))
    assert len(tokens) >= 96                                     # beyond the reference's switch of attention kernels at 64 keys
    mine = P.forward_logits(cfg, W, tokens)
    assert mine.shape == ref.shape
    err = np.abs(mine - ref).max(axis=1)
    assert err.max() <= 2e-6 * max(1.0, np.abs(ref).max()), f"first wrong position {int((err > 2e-6).argmax())}: {err.max():.2e}"
    assert (mine.argmax(1) == ref.argmax(1)).all()
    # the comparison can fail: a different rope base must show
    cfg2 = dict(cfg, rope_theta=10000.0)
    assert np.abs(P.forward_logits(cfg2, W, tokens) - ref).max() > 1e-4


def test_plain_parts():
    x = np.array([[3.0, 4.0]], dtype=np.float32)
    out = P.rms_norm(x, np.ones(2, np.float32), 0.0)
    np.testing.assert_allclose(out, x / np.sqrt(12.5), rtol=1e-6)
    cos, sin = P.rope_angles([0, 1], 4, 10000.0)
    assert cos.shape == (2, 2) and np.allclose(cos[0], 1) and np.allclose(sin[0], 0)
    v = np.arange(8, dtype=np.float32).reshape(1, 2, 4)
    r = P.rope(np.repeat(v, 2, 0), cos, sin)
    np.testing.assert_allclose(r[0], v[0])                      # position 0 rotates nothing
    np.testing.assert_allclose(np.linalg.norm(r[1], axis=-1), np.linalg.norm(v[0], axis=-1), rtol=1e-6)
    assert P.greedy(np.array([1.0, 5.0, 5.0, 2.0], np.float32)) == 1
    q = np.random.default_rng(0).normal(size=(5, 2, 4)).astype(np.float32)
    k = np.random.default_rng(1).normal(size=(5, 1, 4)).astype(np.float32)
    a = P.causal_attention(q, k, k)
    np.testing.assert_allclose(a[0, 0], k[0, 0], rtol=1e-6)     # the first token sees itself only
    w = P.causal_attention(q, k, k, window=1)
    np.testing.assert_allclose(w[:, 0], k[:, 0], rtol=1e-6)     # window 1: every token sees itself only


def test_plain_sampling_filters():
    l = np.log(np.array([0.5, 0.2, 0.15, 0.1, 0.05], dtype=np.float32))
    p = P.sample_probs(l, 1.0, top_k=3)
    assert (p > 0).tolist() == [True, True, True, False, False]
    p = P.sample_probs(l, 1.0, top_p=0.6)
    assert (p > 0).tolist() == [True, True, False, False, False]
    p = P.sample_probs(l, 1.0, min_p=0.25)
    assert (p > 0).tolist() == [True, True, True, False, False]
    p = P.sample_probs(l, 1.0)
    assert P.sample_from(p, 0.49) == 0 and P.sample_from(p, 0.51) == 1 and P.sample_from(p, 1.0) == 4


def test_plain_repetition_penalty_and_its_options(monkeypatch):
    """A token twice among the last generated ones is penalised twice; positive logits are
    divided, negative ones multiplied; tokens before the window are left alone.  The command
    line takes penalty and window from the flags, else from the reference's two environment
    variables, and ignores values outside the reference's ranges (main.c:3741-3752)."""
    l = np.array([2.0, -1.0, 4.0, 0.5, -3.0], dtype=np.float32)
    out = P.repetition_penalty(l, [4, 0, 2, 0, 1], 2.0, 4)
    np.testing.assert_array_equal(out, np.array([0.5, -2.0, 2.0, 0.5, -3.0], dtype=np.float32))
    np.testing.assert_array_equal(P.repetition_penalty(l, [0, 1], 1.0, 4), l)
    from kestrel_llm_b200.cli import _repetition_options, build_parser
    args = build_parser().parse_args(["--model", "x"])
    monkeypatch.delenv("VLLM_STREAM_REPPEN", raising=False)
    monkeypatch.delenv("VLLM_STREAM_REPWIN", raising=False)
    assert _repetition_options(args) == (1.0, 32)
    monkeypatch.setenv("VLLM_STREAM_REPPEN", "1.25")
    monkeypatch.setenv("VLLM_STREAM_REPWIN", "70")          # outside 1..64: the default stays
    assert _repetition_options(args) == (1.25, 32)
    args = build_parser().parse_args(["--model", "x", "--repetition-penalty", "1.5", "--repetition-window", "8"])
    assert _repetition_options(args) == (1.5, 8)
    args = build_parser().parse_args(["--model", "x", "--repetition-penalty", "0.9"])
    assert _repetition_options(args) == (1.0, 32)
