"""The engine at the layer sizes of Qwen3-8B (width 4096, 32/8 heads of 128, feed-forward 12288,
vocabulary 151936) with two layers and random weights: the kernels' fast paths at the sizes they
were written for (tcgen05 products in all their tilings, tcgen05 attention, the head-size-128
rotary kernel) against the plain implementation, in float32 and in bfloat16, whole prompt against
portions against single tokens.  The plain implementation gets the model's own weights as numpy
arrays; nothing is written to disk.  (GPU, about a minute)"""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as R

pytestmark = pytest.mark.gpu

# Rounding of a float32 sum of K terms in sequence grows like sqrt(K) * 2^-24; the engine's
# float32 products sum 4096 and 12288 terms here against 64..200 in the tiny models for which
# replay_util.TOL was set, and numpy's blocked sums are tighter than either.  The bound for this
# file follows that law: 2e-7 * sqrt(12288) = 2.2e-5 of the largest logit.  bfloat16 is bounded
# by the rounding of activations, which does not grow with K: replay_util.TOL applies unchanged.
TOL_F32 = 2e-7 * (12288 ** 0.5)

RAW = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=4096,
           num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
           rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
           max_position_embeddings=1024, hidden_act="silu")


@pytest.fixture(scope="module")
def full_size():
    from kestrel_llm_b200.config import Qwen3Config
    from kestrel_llm_b200.models.qwen3 import build_qwen3
    from kestrel_llm_b200.weights import fill_random_
    cfg = Qwen3Config.from_dict(RAW)
    m16 = build_qwen3(cfg, torch.bfloat16, "cuda:0")
    fill_random_(m16, 7)
    W = {s.name: s.dest.detach().float().cpu().numpy() for s in m16.weight_slots()}
    rng = np.random.default_rng(11)
    toks = rng.integers(0, cfg.vocab_size, size=300).tolist()
    pcfg = dict(RAW, qk_norm_eps=RAW["rms_norm_eps"])
    ref = P.forward_logits(pcfg, W, toks)
    m32 = build_qwen3(cfg, torch.float32, "cuda:0")
    with torch.no_grad():                       # the float32 model holds the bfloat16 values widened
        for a, b in zip(m32.weight_slots(), m16.weight_slots()):
            a.dest.copy_(b.dest.float())
    return {"bfloat16": m16, "float32": m32, "tokens": toks, "ref": ref}


def _logits(model, dtype, toks, cuts, graphs=False):
    """Feeds toks cut into portions of the given sizes; returns logits of every position."""
    from kestrel_llm_b200.config import EngineOptions
    from kestrel_llm_b200.engine import Engine, Entry
    eng = Engine(model, EngineOptions(dtype=dtype, page_size=16, batch_max=2, num_pages=32, cuda_graphs=graphs))
    out, pos = [], 0
    for n in cuts:
        piece = toks[pos:pos + n]
        out.append(eng.step([Entry(0, piece, list(range(len(piece))))]).float().cpu().numpy())
        pos += len(piece)
    assert pos == len(toks)
    eng.release(0)
    return np.concatenate(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_size_layers_against_plain(full_size, dtype):
    toks, ref = full_size["tokens"], full_size["ref"]
    model = full_size[dtype]
    scale = float(np.abs(ref).max())
    whole = _logits(model, dtype, toks, [300])                       # many-token products, tcgen05 attention
    err = float(np.abs(whole - ref).max()) / scale
    tol = TOL_F32 if dtype == "float32" else R.TOL[dtype]
    assert err <= tol, f"whole prompt: {err:.3e}"
    cut = _logits(model, dtype, toks, [257, 2, 24, 1, 1, 1, 14])     # portions, then single tokens
    err = float(np.abs(cut - ref).max()) / scale
    assert err <= tol, f"portions: {err:.3e}"
    tol_between = 2e-6 if dtype == "float32" else R.TOL[dtype]
    assert float(np.abs(cut - whole).max()) / scale <= tol_between
    if dtype == "bfloat16":                                           # single tokens replayed from CUDA graphs
        tail = _logits(model, dtype, toks, [284] + [1] * 16, graphs=True)
        assert float(np.abs(tail - ref).max()) / scale <= R.TOL[dtype]
    from kestrel_llm_b200.csrc import ops
    assert ops.gemm_tc_error() == 0 and ops.attention_tc_error() == 0
