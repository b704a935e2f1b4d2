"""Each part alone against the plain function of the same part, and the claims about how
parts compose: a toy mixer with state of its own, a toy position encoding and a toy
feed-forward are defined HERE, registered, built and stepped without a change to the
package; the order of layers is data (a block runs twice, a layer reads another's cache) (GPU)."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P
import replay_util as R
import tiny_configs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 5e-6, "bfloat16": 2e-2}


def _step_tools(specs, dtype, tokens_per_req, page=16):
    """A cache manager and one batch holding whole requests, for driving a part directly."""
    from kestrel_llm_b200.cache import CacheManager
    from kestrel_llm_b200.engine import Entry, StepBatch
    total = sum(R.ceil64(len(t)) for t in tokens_per_req)
    cm = CacheManager(specs, DT[dtype], DEV, page, total // page, 4, 512)
    entries = []
    for i, toks in enumerate(tokens_per_req):
        cm.admit(i)
        cm.reserve(i, len(toks))
        entries.append(Entry(i, toks, ()))
    return cm, StepBatch(entries, cm, DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from kestrel_llm_b200.parts import RMSNorm
    n = RMSNorm(200, 3e-5, DEV, "w")
    assert [s.name for s in n.weight_slots()] == ["w"] and n.weight_slots()[0].init == "norm"
    w = torch.randn(200)
    n.weight.copy_(w)
    x = torch.randn((6, 200))
    res = x.to(DEV)
    out = n.add_forward(res, None, DT[dtype])
    ref = P.rms_norm(x.numpy(), w.numpy(), 3e-5)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=TOL[dtype] * 50, atol=TOL[dtype] * np.abs(ref).max())


def test_rotary_part_matches_the_plain_angles():
    from kestrel_llm_b200.parts import RotaryHalf
    r = RotaryHalf(48, 50000.0, DEV)
    spec = r.rotary()
    inv, rot = spec.inv_freq, spec.dim
    assert rot == 48 and inv.dtype == torch.float32 and spec.pairing == "half" and spec.scale == 1.0
    cos, sin = P.rope_angles([1], 48, 50000.0)
    np.testing.assert_array_equal(np.cos(inv.cpu().numpy().astype(np.float32)), cos[0])
    with pytest.raises(ValueError):
        RotaryHalf(48, 1e4, DEV, rotary_dim=50)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_attention_part(model_dirs, name, dtype):
    """The mixer of layer 1 alone: projections, per-head norm, rotation, cache write, attention,
    output projection, for two requests in one batch."""
    from kestrel_llm_b200.weights import load_model
    m = load_model(model_dirs[name][dtype], dtype, DEV)
    cfg, W = P.read_model(model_dirs[name]["float32"])
    mixer = m.blocks[1].mixer
    lens = (37, 90)
    xs = [torch.randn((n, cfg["hidden_size"]), generator=torch.Generator().manual_seed(n)).to(DT[dtype]) for n in lens]
    cm, batch = _step_tools([mixer.cache_spec()], dtype, [[0] * n for n in lens])
    out = mixer.forward(torch.cat(xs).to(DEV), batch, cm.layer(0)).reduce(torch.float32).cpu().numpy()
    off = 0
    for x, n in zip(xs, lens):
        ref = P.attention_block(x.float().numpy(), np.arange(n), W, cfg, 1, P.layer_window(cfg, 1))
        np.testing.assert_allclose(out[off:off + n], ref, rtol=0, atol=TOL[dtype] * 3 * np.abs(ref).max())
        off += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(model_dirs, dtype):
    from kestrel_llm_b200.weights import load_model
    m = load_model(model_dirs["B"][dtype], dtype, DEV)
    cfg, W = P.read_model(model_dirs["B"]["float32"])
    x = torch.randn((11, 96), generator=torch.Generator().manual_seed(0)).to(DT[dtype])
    out = m.blocks[2].ffn.forward(x.to(DEV), None).reduce(torch.float32).cpu().numpy()
    p = "model.layers.2.mlp."
    ref = P.gated_mlp(x.float().numpy(), W[p + "gate_proj.weight"], W[p + "up_proj.weight"], W[p + "down_proj.weight"])
    np.testing.assert_allclose(out, ref, rtol=0, atol=TOL[dtype] * 3 * np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_embedding_and_head(model_dirs, dtype):
    from kestrel_llm_b200.weights import load_model
    m = load_model(model_dirs["B"][dtype], dtype, DEV)
    cfg, W = P.read_model(model_dirs["B"]["float32"])
    toks = list(range(100, 150))
    cm, batch = _step_tools([m.blocks[0].cache_spec()], dtype, [toks])
    x = m.embedding.forward(batch.token_ids)
    ref = P.embedding(W["model.embed_tokens.weight"], toks)
    np.testing.assert_array_equal(x.cpu().numpy(), ref)
    res, pending = m.blocks[0].forward(x, None, batch, cm.layer(0))
    got = (res + pending.reduce(torch.float32)).cpu().numpy()
    ref = P.decoder_layer(ref, np.arange(len(toks)), W, cfg, 0)
    np.testing.assert_allclose(got, ref, rtol=0, atol=TOL[dtype] * 3 * np.abs(ref).max())
    n = torch.randn((3, 96)).to(DT[dtype])
    lg = m.lm_head.forward(n.to(DEV)).cpu().numpy()
    refl = P.linear(n.float().numpy(), W["lm_head.weight"])
    np.testing.assert_allclose(lg, refl, rtol=0, atol=TOL[dtype] * np.abs(refl).max() + 1e-6)


# ---- toy parts, defined in the tests (tests/toy_architecture.py) ------------------------------

def _toy_folder(tmp_path, seed=11):
    """The toy architecture written to a folder by the random-weights mode, from its own
    configuration class; returns (folder, config.json dict, tensors)."""
    import toy_architecture as toy
    from kestrel_llm_b200.weights import write_random_model
    cfg = toy.register().from_dict(dict(toy.RAW))
    d = write_random_model(cfg, seed, str(tmp_path / "toy"), "float32")
    pcfg, W = toy.read_folder(d)
    assert set(pcfg) >= {"width", "depth", "rotary_scale"} and "hidden_size" not in pcfg     # its own keys
    return d, pcfg, W


def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    """A mixer with state of its own, a feed-forward with routing, a learned position table and
    a rotation of another form (adjacent pairs, part of a head, scaled), with a configuration
    class of their own, none of them in the package: written to a folder by the random-weights
    mode, loaded by name through the registry, stepped whole, token by token and in portions with
    several requests interleaved; all agree with a numpy statement of the toy model.  The model
    has parts without a step program, so its steps walk the parts' forward methods."""
    import toy_architecture as toy
    d, pcfg, W = _toy_folder(tmp_path)
    reqs = R.random_requests(pcfg["vocab"], (40, 23, 64), seed=4)
    refs = {n: toy.reference_logits(W, pcfg, t) for n, t in reqs.items()}
    for family in (R.trace_whole, R.trace_tail_decode, R.trace_portions, R.trace_mixed):
        steps, max_tokens = family(reqs)
        engine = R.make_engine(d, "float32", max_tokens)
        assert engine.runner is None
        assert [type(s).__name__ for s in engine.model.cache_specs()] == ["FixedStateSpec", "PagedKVSpec"] * 2
        got = R.run_trace(engine, steps)
        for n, toks in reqs.items():
            for p in range(len(toks)):
                err = np.abs(got[n][p] - refs[n][p]).max() / np.abs(refs[n]).max()
                assert err < 2e-5, f"{family.__name__}: request {n} position {p}: {err:.2e}"


def test_toy_generation_reuses_state_slots_and_survives_preemption(tmp_path):
    """Through `LLM.generate`, where the native scheduler admits requests on its own: more
    requests than state slots, so slots are reused by later requests, and so few pages that
    requests are preempted and start again from position 0.  A slot that kept its last owner's
    running sum would change the tokens; they are those of the numpy model."""
    import toy_architecture as toy
    from kestrel_llm_b200 import LLM, SamplingParams
    d, pcfg, W = _toy_folder(tmp_path)
    prompts = list(R.random_requests(pcfg["vocab"], (21, 9, 30, 14, 25), seed=6).values())
    sp = SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True)
    want = [toy.greedy_continuation(W, pcfg, p, 14) for p in prompts]
    roomy = LLM(d, dtype="float32", page_size=16, batch_max=2, max_tokens=512)
    outs = roomy.generate(prompts, sp)
    assert [o.token_ids for o in outs] == want
    tight = LLM(d, dtype="float32", page_size=16, batch_max=3, num_pages=6)        # 96 tokens for up to 3 requests of up to 44
    outs = tight.generate(prompts, sp)
    assert tight.scheduler.num_preemptions > 0
    assert [o.token_ids for o in outs] == want
    tight.engine.cache.check()


def test_toy_architecture_through_the_command_line(tmp_path):
    """bin/kestrel in a process of its own: `--plugin` imports the module that registers the toy
    architecture, `--random-weights` writes its folder from a config.json with the toy's own
    keys, and the streaming harness prints the numpy model's greedy tokens."""
    import json
    import os
    import subprocess
    import sys
    import toy_architecture as toy
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "toy_config.json"
    cfg_file.write_text(json.dumps(toy.RAW))
    model_dir = tmp_path / "toy_cli"
    prompt = R.random_requests(toy.RAW["vocab"], (19,), seed=2)["r0"]
    env = dict(os.environ, PYTHONPATH=os.path.join(root, "tests") + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "kestrel"), "--plugin", "toy_architecture", "--model", str(model_dir),
                        "--config", str(cfg_file), "--random-weights", "5", "--dtype", "float32", "--stream-test", "--stream-n", "10",
                        "--prompt-ids", ",".join(str(t) for t in prompt), "--ignore-eos", "--max-tokens", "256", "--batch-max", "2"],
                       capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("[STREAM] TOKIDS:")]
    assert len(line) == 1
    pcfg, W = toy.read_folder(str(model_dir))
    # the folder stores bfloat16 (the command line's random-weights mode); the float32 engine widens it exactly
    assert [int(t) for t in line[0].split(":")[1].split()] == toy.greedy_continuation(W, pcfg, prompt, 10)
    assert any(l.startswith("[STREAM] metrics request=") for l in p.stdout.splitlines())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_order_is_data(model_dirs, dtype):
    """The same weights under another order: block 0, block 1, block 0 again (with a cache of
    its own), then block 2 reading block 1's cache instead of writing one."""
    from kestrel_llm_b200.models import LayerCall
    from kestrel_llm_b200.config import EngineOptions
    from kestrel_llm_b200.engine import Engine, Entry
    from kestrel_llm_b200.weights import load_model
    m = load_model(model_dirs["B"][dtype], dtype, DEV)
    order = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 1, writes_cache=False)]
    m2 = type(m)(m.config, m.dtype, m.device, m.embedding, m.position, m.blocks, order, m.final_norm, m.lm_head)
    assert len(m2.cache_specs()) == 3
    cfg, W = P.read_model(model_dirs["B"]["float32"])
    toks = R.random_requests(509, (45,), 9)["r0"]
    T = len(toks)
    pos = np.arange(T)

    def layer(x, i, kv_from=None, keep=None):
        pre = f"model.layers.{i}."
        n = P.rms_norm(x, W[pre + "input_layernorm.weight"], cfg["rms_norm_eps"])
        a = pre + "self_attn."
        nh, nkv, hd = 6, 2, 32
        q = P.linear(n, W[a + "q_proj.weight"], W[a + "q_proj.bias"]).reshape(T, nh, hd)
        q = P.head_rms_norm(q, W[a + "q_norm.weight"], cfg["rms_norm_eps"])
        cos, sin = P.rope_angles(pos, hd, cfg["rope_theta"])
        q = P.rope(q, cos, sin)
        if kv_from is None:
            k = P.linear(n, W[a + "k_proj.weight"], W[a + "k_proj.bias"]).reshape(T, nkv, hd)
            k = P.rope(P.head_rms_norm(k, W[a + "k_norm.weight"], cfg["rms_norm_eps"]), cos, sin)
            v = P.linear(n, W[a + "v_proj.weight"], W[a + "v_proj.bias"]).reshape(T, nkv, hd)
        else:
            k, v = kv_from
        if keep is not None:
            keep.extend([k, v])
        x = x + P.linear(P.causal_attention(q, k, v).reshape(T, nh * hd), W[a + "o_proj.weight"], W[a + "o_proj.bias"])
        n = P.rms_norm(x, W[pre + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        return x + P.gated_mlp(n, W[pre + "mlp.gate_proj.weight"], W[pre + "mlp.up_proj.weight"], W[pre + "mlp.down_proj.weight"])

    x = P.embedding(W["model.embed_tokens.weight"], toks)
    kv1 = []
    x = layer(x, 0)
    x = layer(x, 1, keep=kv1)
    x = layer(x, 0)
    x = layer(x, 2, kv_from=kv1)
    ref = P.linear(P.rms_norm(x, W["model.norm.weight"], cfg["rms_norm_eps"]), W["lm_head.weight"])
    eng = Engine(m2, EngineOptions(dtype=dtype, page_size=16, batch_max=2, num_pages=8, cuda_graphs=False))
    outs = []
    for b, e in ((0, 20), (20, 22), (22, 45)):            # in portions: the shared cache must persist
        outs.append(eng.step([Entry(0, toks[b:e], list(range(e - b)))]).cpu().numpy())
    got = np.concatenate(outs)
    assert np.abs(got - ref).max() <= TOL[dtype] * np.abs(ref).max()
    with pytest.raises(ValueError, match="read before it is written"):
        type(m)(m.config, m.dtype, m.device, m.embedding, m.position, m.blocks,
                [LayerCall(0, 0, writes_cache=False), LayerCall(1, 0)], m.final_norm, m.lm_head)
