"""Each part alone against the plain function of the same part, and the claims about how
parts compose: a toy mixer with state of its own, a toy position encoding and a toy
feed-forward are defined HERE, registered, built and stepped without a change to the
package; the order of layers is data (a block runs twice, a layer reads another's cache) (GPU)."""
import math
from dataclasses import dataclass

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


# ---- toy parts, defined in the test ----------------------------------------------------------

def _toy_parts():
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import FeedForward, FixedStateSpec, Mixer, PositionEncoding, WeightSlot

    class RunningMeanMixer(Mixer):
        """out[t] = W * mean(x[0..t]) of the request: needs a running sum per request, kept in a
        fixed-size state slot; no pages."""

        def __init__(self, width, dtype, device, prefix):
            self.width, self.dtype, self.prefix = width, dtype, prefix
            self.weight = torch.empty((width, width), dtype=dtype, device=device)

        def cache_spec(self):
            return FixedStateSpec((self.width,), torch.float32)

        def weight_slots(self):
            return [WeightSlot(self.prefix + "mix.weight", self.weight)]

        def forward(self, x, batch, cache):
            outs = []
            cu = batch.cu_seqlens_host
            for i in range(batch.num_seqs):
                b, e = cu[i], cu[i + 1]
                slot = batch.slots_host[i]
                cs = cache.state[slot] + torch.cumsum(x[b:e].float(), 0)
                cache.state[slot] = cs[-1]
                outs.append(cs / (batch.positions[b:e].float() + 1)[:, None])
            mean = torch.cat(outs).to(self.dtype)
            return ops.Partials(ops.linear(mean, self.weight))

    class LearnedPositions(PositionEncoding):
        """An absolute encoding: a table row per position, added to the embedded tokens."""

        def __init__(self, max_pos, width, device):
            self.table = torch.empty((max_pos, width), dtype=torch.float32, device=device)

        def weight_slots(self):
            return [WeightSlot("model.positions.weight", self.table)]

        def add_to_embedding(self, x, batch):
            x += self.table[batch.positions.long()]

    class RoutedFeedForward(FeedForward):
        """Two experts, each token goes to the one its router scores higher."""

        def __init__(self, width, inner, dtype, device, prefix):
            self.dtype, self.prefix = dtype, prefix
            self.router = torch.empty((2, width), dtype=dtype, device=device)
            self.up = [torch.empty((inner, width), dtype=dtype, device=device) for _ in range(2)]
            self.down = [torch.empty((width, inner), dtype=dtype, device=device) for _ in range(2)]

        def weight_slots(self):
            s = [WeightSlot(self.prefix + "router.weight", self.router)]
            for e in range(2):
                s += [WeightSlot(f"{self.prefix}experts.{e}.up.weight", self.up[e]),
                      WeightSlot(f"{self.prefix}experts.{e}.down.weight", self.down[e])]
            return s

        def forward(self, x, batch):
            score = ops.linear(x, self.router).sum(0)
            pick = score.argmax(1)
            out = torch.zeros((x.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
            for e in range(2):
                idx = (pick == e).nonzero().flatten()
                if idx.numel():
                    h = torch.relu(ops.linear(x[idx].contiguous(), self.up[e]).sum(0)).to(self.dtype)
                    out[idx] = ops.linear(h, self.down[e]).sum(0)
            return ops.Partials(out)

    return RunningMeanMixer, LearnedPositions, RoutedFeedForward


@dataclass(frozen=True)
class _ToyConfigBase:
    pass


def _register_toy():
    from kestrel_llm_b200.config import Qwen3Config, register_architecture
    from kestrel_llm_b200.models import DecoderModel, LayerCall
    from kestrel_llm_b200.parts import (GatedMLP, GroupedQueryAttention, LMHead, PreNormBlock, RMSNorm,
                                        TokenEmbedding)
    Mean, Learned, Routed = _toy_parts()

    def build(c, dtype, device):
        emb = TokenEmbedding(c.vocab_size, c.hidden_size, dtype, device, "model.embed_tokens.weight")
        pos = Learned(c.max_position_embeddings, c.hidden_size, device)
        blocks = []
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            if i % 2 == 0:
                mixer = Mean(c.hidden_size, dtype, device, p)
                ffn = Routed(c.hidden_size, c.intermediate_size, dtype, device, p + "moe.")
            else:        # attention without rotation: positions come from the learned table
                mixer = GroupedQueryAttention(c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
                                              c.head_dim, dtype, device, p + "self_attn.", None, None)
                ffn = GatedMLP(c.hidden_size, c.intermediate_size, dtype, device, p + "mlp.")
            blocks.append(PreNormBlock(RMSNorm(c.hidden_size, c.rms_norm_eps, device, p + "n1.weight"), mixer,
                                       RMSNorm(c.hidden_size, c.rms_norm_eps, device, p + "n2.weight"), ffn, dtype))
        order = [LayerCall(i, i) for i in range(c.num_hidden_layers)]
        return DecoderModel(c, dtype, device, emb, pos, blocks, order,
                            RMSNorm(c.hidden_size, c.rms_norm_eps, device, "model.norm.weight"),
                            LMHead(c.vocab_size, c.hidden_size, dtype, device, "lm_head.weight"))

    register_architecture("ToyStateForCausalLM", Qwen3Config, build)


def _toy_reference(W, cfg, toks):
    """The toy model, whole sequence, in numpy."""
    T = len(toks)
    pos = np.arange(T)
    x = W["model.embed_tokens.weight"][toks] + W["model.positions.weight"][pos]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        n = P.rms_norm(x, W[p + "n1.weight"], cfg["rms_norm_eps"])
        if i % 2 == 0:
            mean = np.cumsum(n, 0) / (pos + 1)[:, None].astype(np.float32)
            x = x + P.linear(mean.astype(np.float32), W[p + "mix.weight"])
            n = P.rms_norm(x, W[p + "n2.weight"], cfg["rms_norm_eps"])
            pick = P.linear(n, W[p + "moe.router.weight"]).argmax(1)
            y = np.zeros_like(x)
            for e in range(2):
                h = np.maximum(P.linear(n, W[f"{p}moe.experts.{e}.up.weight"]), 0)
                y[pick == e] = P.linear(h, W[f"{p}moe.experts.{e}.down.weight"])[pick == e]
            x = x + y
        else:
            nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
            a = p + "self_attn."
            q = P.linear(n, W[a + "q_proj.weight"]).reshape(T, nh, hd)
            k = P.linear(n, W[a + "k_proj.weight"]).reshape(T, nkv, hd)
            v = P.linear(n, W[a + "v_proj.weight"]).reshape(T, nkv, hd)
            x = x + P.linear(P.causal_attention(q, k, v).reshape(T, nh * hd), W[a + "o_proj.weight"])
            n = P.rms_norm(x, W[p + "n2.weight"], cfg["rms_norm_eps"])
            x = x + P.gated_mlp(n, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, W["model.norm.weight"], cfg["rms_norm_eps"]), W["lm_head.weight"])


def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    """A mixer with state of its own, a feed-forward with routing and another position
    encoding, none of them in the package: written to a folder by the random-weights mode,
    loaded by name through the registry, stepped whole, token by token and in portions with
    two requests interleaved; all agree with a numpy statement of the toy model."""
    from kestrel_llm_b200.config import Qwen3Config
    from kestrel_llm_b200.weights import write_random_model
    _register_toy()
    raw = dict(tiny_configs.B, architectures=["ToyStateForCausalLM"], num_hidden_layers=4, attention_bias=False,
               max_position_embeddings=128)
    cfg = Qwen3Config.from_dict(raw)
    d = write_random_model(cfg, 11, str(tmp_path / "toy"), "float32")
    pcfg, W = P.read_model(d)
    reqs = R.random_requests(cfg.vocab_size, (40, 23, 64), seed=4)
    refs = {n: _toy_reference(W, pcfg, t) for n, t in reqs.items()}
    for family in (R.trace_whole, R.trace_tail_decode, R.trace_portions, R.trace_mixed):
        steps, max_tokens = family(reqs)
        engine = R.make_engine(d, "float32", max_tokens)
        assert [type(s).__name__ for s in engine.model.cache_specs()] == ["FixedStateSpec", "PagedKVSpec"] * 2
        got = R.run_trace(engine, steps)
        for n, toks in reqs.items():
            for p in range(len(toks)):
                err = np.abs(got[n][p] - refs[n][p]).max() / np.abs(refs[n]).max()
                assert err < 2e-5, f"{family.__name__}: request {n} position {p}: {err:.2e}"


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
