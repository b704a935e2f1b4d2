"""The engine against the plain implementation at the benchmark's context lengths: requests of
4,300 and 9,100 tokens on a narrow model with head size 128, page size 16, under the cuttings
that long contexts bring - a whole prompt, 2,048-token portions and then single tokens (captured
and launched one by one), 512-token portions far into the context (the prompt-portion kernel
then cuts its key range into slices), and long requests decoding beside a short one.  Every
wanted position is held against `plain_qwen3.forward_logits`; the plain implementation is run
once per token sequence (a prefix of a sequence shares its logits, the model being causal).
The reference's long-context path is its tiled float32 attention
(src/model/vllm_safetensors.c:9762-9859)."""
import numpy as np
import pytest

import replay_util as R

pytestmark = pytest.mark.gpu

LONG = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=128,
            num_attention_heads=2, num_key_value_heads=1, head_dim=128, intermediate_size=192, vocab_size=307,
            rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=False,
            max_position_embeddings=16384, hidden_act="silu")
N1, N2 = 4300, 9100


@pytest.fixture(scope="module")
def long_model(tmp_path_factory):
    """{dtype: folder} of the narrow model, the float32 folder holding the bfloat16 values widened."""
    import os
    import shutil
    import torch
    from kestrel_llm_b200.config import Qwen3Config
    from kestrel_llm_b200.weights import write_random_model
    from kestrel_llm_b200.weights.safetensors_io import ModelFolder, write_safetensors
    base = tmp_path_factory.mktemp("model_long")
    d16, d32 = str(base / "bf16"), str(base / "f32")
    write_random_model(Qwen3Config.from_dict(LONG), 21, d16, "bfloat16")
    os.makedirs(d32)
    shutil.copy(os.path.join(d16, "config.json"), os.path.join(d32, "config.json"))
    mf = ModelFolder(d16)
    write_safetensors(os.path.join(d32, "model.safetensors"), ((n, mf.tensor(n).to(torch.float32)) for n in mf.names()))
    mf.close()
    return {"bfloat16": d16, "float32": d32}


def _tokens():
    rng = np.random.default_rng(77)
    return rng.integers(0, LONG["vocab_size"], size=N1).tolist(), rng.integers(0, LONG["vocab_size"], size=N2).tolist()


def _wanted(n, lo=0):
    """A strided subset of the positions lo..n-1, and always the last 64."""
    return sorted(set(range(lo, n, 97)) | set(range(max(lo, n - 64), n)))


def _steps_in_portions(name, toks, portion, tail, want_from=0):
    """Portions of `portion` tokens, then the last `tail` tokens one by one; logits wanted at the
    strided subset (among the portions) and at every single token."""
    steps, pos = [], 0
    wanted = set(_wanted(len(toks), want_from))
    body = len(toks) - tail
    while pos < body:
        n = min(portion, body - pos)
        steps.append({"entries": [{"id": name, "tokens": toks[pos:pos + n], "want": [p - pos for p in range(pos, pos + n) if p in wanted]}],
                      "end": []})
        pos += n
    for i in range(body, len(toks)):
        steps.append({"entries": [{"id": name, "tokens": [toks[i]], "want": [0]}], "end": []})
    steps[-1]["end"] = [name]
    return steps


def _check(model_f32, toks, got, dtype, label, positions=None):
    ref = R.plain_logits(model_f32, toks)
    scale = float(np.abs(ref).max())
    worst = 0.0
    for p in sorted(got if positions is None else positions):
        row = got[p]
        assert np.isfinite(row).all(), f"{label}: position {p}: logits are not finite"
        err = float(np.abs(row - ref[p]).max()) / scale
        worst = max(worst, err)
        assert err <= R.TOL[dtype], f"{label}: first wrong position {p} of {len(toks)}: error {err:.3e}, allowed {R.TOL[dtype]:.1e}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_whole_prompt_of_4300_tokens(long_model, dtype):
    t1, _ = _tokens()
    steps = [{"entries": [{"id": "a", "tokens": t1, "want": _wanted(N1)}], "end": ["a"]}]
    got = R.run_trace(R.make_engine(long_model[dtype], dtype, R.ceil64(N1)), steps)
    worst = _check(long_model["float32"], t1, got["a"], dtype, f"whole/{dtype}")
    print(f"[long] whole prompt {dtype}: {len(got['a'])} positions, worst {worst:.3e}")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_2048_then_the_last_32_tokens_one_by_one(long_model, dtype, graphs):
    t1, _ = _tokens()
    steps = _steps_in_portions("a", t1, 2048, 32)
    engine = R.make_engine(long_model[dtype], dtype, R.ceil64(N1), graphs=graphs)
    got = R.run_trace(engine, steps)
    assert (engine.graph_launches > 0) == graphs
    _check(long_model["float32"], t1, got["a"], dtype, f"2048+32/{dtype}/graphs={graphs}")


def test_portions_of_512_far_into_9100_tokens(long_model):
    """bfloat16: the first 3,600 tokens in one step, then portions of 512 at contexts of 4,100 to
    9,100 keys, where the tcgen05 kernel's few row tiles cut their key ranges into slices; then
    the last 32 tokens one by one from captured graphs (the context class beyond 4,096)."""
    _, t2 = _tokens()
    head = 3600
    steps = [{"entries": [{"id": "x", "tokens": t2[:head], "want": []}], "end": []}]
    for st in _steps_in_portions("x", t2[head:], 512, 32):
        steps.append(st)
    # positions of the later steps are relative to the request, which run_trace tracks itself
    engine = R.make_engine(long_model["bfloat16"], "bfloat16", R.ceil64(N2), graphs=True)
    got = R.run_trace(engine, steps)["x"]
    assert min(got) >= head and max(got) == N2 - 1 and len(got) > 100
    worst = _check(long_model["float32"], t2, got, "bfloat16", "512 far into 9100")
    print(f"[long] 512-token portions up to {N2} keys: {len(got)} positions, worst {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_requests_decode_beside_a_short_one(long_model, dtype):
    """Three requests live at once: 4,300 tokens, a 4,200-token prefix of the 9,100-token
    sequence (in bfloat16 the whole 9,100), and a short one; their last 24 tokens are decoded in
    the same steps, after portions of changing size."""
    t1, t2 = _tokens()
    second = t2 if dtype == "bfloat16" else t2[:4200]
    short = np.random.default_rng(5).integers(0, LONG["vocab_size"], size=70).tolist()
    reqs = {"a": t1, "b": second, "s": short}
    tail = 24
    pos = {n: 0 for n in reqs}
    sizes = {"a": 1500, "b": 2048, "s": 23}
    wanted = {n: set(_wanted(len(t))) for n, t in reqs.items()}
    steps = []
    while any(pos[n] < len(reqs[n]) - tail for n in reqs):
        entries = []
        for n, t in reqs.items():
            left = len(t) - tail - pos[n]
            if left <= 0:
                continue
            k = min(sizes[n], left)
            entries.append({"id": n, "tokens": t[pos[n]:pos[n] + k], "want": [p - pos[n] for p in range(pos[n], pos[n] + k) if p in wanted[n]]})
            pos[n] += k
        steps.append({"entries": entries, "end": []})
    for i in range(tail):
        steps.append({"entries": [{"id": n, "tokens": [t[len(t) - tail + i]], "want": [0]} for n, t in reqs.items()], "end": []})
    steps[-1]["end"] = list(reqs)
    engine = R.make_engine(long_model[dtype], dtype, sum(R.ceil64(len(t)) for t in reqs.values()), graphs=(dtype == "bfloat16"))
    got = R.run_trace(engine, steps)
    _check(long_model["float32"], t1, got["a"], dtype, f"beside/{dtype}/a")
    _check(long_model["float32"], t2, got["b"], dtype, f"beside/{dtype}/b")          # a prefix shares the sequence's logits
    _check(long_model["float32"], short, got["s"], dtype, f"beside/{dtype}/s")


def test_keys_in_the_wrong_pages_are_noticed(long_model):
    """The comparison above can fail: after a 4,300-token prompt, two of the request's OWN pages
    trade their contents in one layer - what a wrong block-table column would read - and the
    next token's logits leave the tolerance.  Only valid memory is touched."""
    import torch
    t1, _ = _tokens()
    engine = R.make_engine(long_model["float32"], "float32", R.ceil64(N1))
    from kestrel_llm_b200.engine import Entry
    engine.step([Entry(0, t1[:-1], ())])
    table = engine.cache.block_table(0, 0)
    a, b = table[3], table[200]
    k = engine.cache.k[1]
    tmp = k[a].clone()
    k[a].copy_(k[b])
    k[b].copy_(tmp)
    row = engine.step([Entry(0, t1[-1:], (0,))])[0].cpu().numpy()
    engine.release(0)
    ref = R.plain_logits(long_model["float32"], t1)
    err = float(np.abs(row - ref[-1]).max()) / float(np.abs(ref).max())
    assert err > 20 * R.TOL["float32"], f"swapped pages moved the logits by {err:.3e} only"
