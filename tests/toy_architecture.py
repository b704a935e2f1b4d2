"""A toy architecture made of parts that the package does not have, defined in the tests:
a configuration class of its own (its own config.json keys), a mixer with state of its own (a
running mean kept in a fixed-size state slot), a feed-forward with routing (two experts), a
learned absolute position table, and a rotary encoding of another form (adjacent pairing, only
part of a head, cos and sin scaled).  `register()` adds it to the registry; nothing in the
package is changed.  It is no model of the reference's or of anyone's.

Importable by name (``--plugin toy_architecture`` of the command line, with this folder on the
path), so that the command line can run it in a process of its own.  `reference_logits` is its
numpy statement, whole sequences, no cache.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict

import numpy as np
import torch

import plain_qwen3 as P

NAME = "ToyStateForCausalLM"
RAW = {"architectures": [NAME], "width": 96, "depth": 4, "vocab": 509, "positions": 160, "heads": 6, "kv_heads": 2,
       "head_size": 32, "rotary_size": 16, "rotary_scale": 0.9, "theta": 5000.0, "inner": 200, "eps": 1e-5}


def config_class():
    from kestrel_llm_b200.config.model_config import ConfigError, ModelConfig

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        """Keys of its own: width, depth, vocab, positions, heads, kv_heads, head_size,
        rotary_size, rotary_scale, theta, inner, eps."""
        heads: int = 0
        kv_heads: int = 0
        head_size: int = 0
        rotary_size: int = 0
        rotary_scale: float = 1.0
        theta: float = 10000.0
        inner: int = 0
        eps: float = 1e-5

        @classmethod
        def from_dict(cls, raw: Dict[str, Any]) -> "ToyConfig":
            for k in ("width", "depth", "vocab", "positions", "heads", "kv_heads", "head_size", "inner"):
                if not isinstance(raw.get(k), int) or raw[k] <= 0:
                    raise ConfigError(f"config.json: '{k}' must be a positive integer")
            return cls(architecture=raw["architectures"][0], vocab_size=raw["vocab"], hidden_size=raw["width"],
                       num_hidden_layers=raw["depth"], max_position_embeddings=raw["positions"], bos_token_id=None,
                       eos_token_ids=tuple(raw.get("eos", ())), heads=raw["heads"], kv_heads=raw["kv_heads"],
                       head_size=raw["head_size"], rotary_size=int(raw.get("rotary_size", raw["head_size"])),
                       rotary_scale=float(raw.get("rotary_scale", 1.0)), theta=float(raw.get("theta", 10000.0)),
                       inner=raw["inner"], eps=float(raw.get("eps", 1e-5)))

        def to_json_dict(self) -> Dict[str, Any]:
            return {"architectures": [self.architecture], "width": self.hidden_size, "depth": self.num_hidden_layers,
                    "vocab": self.vocab_size, "positions": self.max_position_embeddings, "heads": self.heads,
                    "kv_heads": self.kv_heads, "head_size": self.head_size, "rotary_size": self.rotary_size,
                    "rotary_scale": self.rotary_scale, "theta": self.theta, "inner": self.inner, "eps": self.eps,
                    "eos": list(self.eos_token_ids)}

    return ToyConfig


def parts():
    from kestrel_llm_b200.csrc import ops
    from kestrel_llm_b200.parts import FeedForward, FixedStateSpec, Mixer, PositionEncoding, Rotation, WeightSlot

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
        """An absolute encoding (a table row per position, added to the embedded tokens) that also
        hands mixers a rotation of another form than the package's: adjacent pairs, the first
        `rotary_size` dimensions of a head only, cos and sin scaled."""

        def __init__(self, max_pos, width, device, rotary_size, theta, scale):
            self.table = torch.empty((max_pos, width), dtype=torch.float32, device=device)
            half = rotary_size // 2
            inv = (1.0 / np.power(np.float32(theta), np.arange(half, dtype=np.float32) / np.float32(half), dtype=np.float32))
            self.inv_freq = torch.from_numpy(inv.astype(np.float32)).to(device)
            self.rotary_size, self.scale = rotary_size, scale

        def weight_slots(self):
            return [WeightSlot("model.positions.weight", self.table)]

        def add_to_embedding(self, x, batch):
            x += self.table[batch.positions.long()]

        def rotary(self):
            return Rotation(self.inv_freq, self.rotary_size, "interleaved", self.scale)

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


def register():
    from kestrel_llm_b200.config import register_architecture
    from kestrel_llm_b200.models import DecoderModel, LayerCall
    from kestrel_llm_b200.parts import (GatedMLP, GroupedQueryAttention, LMHead, PreNormBlock, RMSNorm,
                                        TokenEmbedding)
    Mean, Learned, Routed = parts()
    ToyConfig = config_class()

    def build(c, dtype, device):
        emb = TokenEmbedding(c.vocab_size, c.hidden_size, dtype, device, "model.embed_tokens.weight")
        pos = Learned(c.max_position_embeddings, c.hidden_size, device, c.rotary_size, c.theta, c.rotary_scale)
        blocks = []
        for i in range(c.num_hidden_layers):
            p = f"model.layers.{i}."
            if i % 2 == 0:
                mixer = Mean(c.hidden_size, dtype, device, p)
                ffn = Routed(c.hidden_size, c.inner, dtype, device, p + "moe.")
            else:        # attention whose queries and keys are turned by the toy encoding's rotation
                mixer = GroupedQueryAttention(c.hidden_size, c.heads, c.kv_heads, c.head_size, dtype, device,
                                              p + "self_attn.", pos, None)
                ffn = GatedMLP(c.hidden_size, c.inner, dtype, device, p + "mlp.")
            blocks.append(PreNormBlock(RMSNorm(c.hidden_size, c.eps, device, p + "n1.weight"), mixer,
                                       RMSNorm(c.hidden_size, c.eps, device, p + "n2.weight"), ffn, dtype))
        order = [LayerCall(i, i) for i in range(c.num_hidden_layers)]
        return DecoderModel(c, dtype, device, emb, pos, blocks, order,
                            RMSNorm(c.hidden_size, c.eps, device, "model.norm.weight"),
                            LMHead(c.vocab_size, c.hidden_size, dtype, device, "lm_head.weight"))

    register_architecture(NAME, ToyConfig, build)
    return ToyConfig


def rope_interleaved(x: np.ndarray, positions, rot: int, theta: float, scale: float) -> np.ndarray:
    """Pairs (2j, 2j+1) of the first `rot` dimensions turned by pos * theta^(-j/(rot/2)), cos and
    sin multiplied by `scale`; x [T, heads, hd]."""
    half = rot // 2
    freq = (np.float32(1.0) / np.power(np.float32(theta), np.arange(half, dtype=np.float32) / np.float32(half), dtype=np.float32))
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    c = (np.cos(ang) * np.float32(scale)).astype(np.float32)[:, None, :]
    s = (np.sin(ang) * np.float32(scale)).astype(np.float32)[:, None, :]
    out = x.astype(np.float32).copy()
    a, b = x[..., 0:rot:2], x[..., 1:rot:2]
    out[..., 0:rot:2] = a * c - b * s
    out[..., 1:rot:2] = b * c + a * s
    return out


def reference_logits(W: dict, cfg: dict, toks) -> np.ndarray:
    """The toy model, whole sequence, in numpy; `cfg` is the folder's config.json."""
    T = len(toks)
    pos = np.arange(T)
    x = W["model.embed_tokens.weight"][toks] + W["model.positions.weight"][pos]
    for i in range(cfg["depth"]):
        p = f"model.layers.{i}."
        n = P.rms_norm(x, W[p + "n1.weight"], cfg["eps"])
        if i % 2 == 0:
            mean = np.cumsum(n, 0) / (pos + 1)[:, None].astype(np.float32)
            x = x + P.linear(mean.astype(np.float32), W[p + "mix.weight"])
            n = P.rms_norm(x, W[p + "n2.weight"], cfg["eps"])
            pick = P.linear(n, W[p + "moe.router.weight"]).argmax(1)
            y = np.zeros_like(x)
            for e in range(2):
                h = np.maximum(P.linear(n, W[f"{p}moe.experts.{e}.up.weight"]), 0)
                y[pick == e] = P.linear(h, W[f"{p}moe.experts.{e}.down.weight"])[pick == e]
            x = x + y
        else:
            nh, nkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_size"]
            a = p + "self_attn."
            q = P.linear(n, W[a + "q_proj.weight"]).reshape(T, nh, hd)
            k = P.linear(n, W[a + "k_proj.weight"]).reshape(T, nkv, hd)
            v = P.linear(n, W[a + "v_proj.weight"]).reshape(T, nkv, hd)
            q = rope_interleaved(q, pos, cfg["rotary_size"], cfg["theta"], cfg["rotary_scale"])
            k = rope_interleaved(k, pos, cfg["rotary_size"], cfg["theta"], cfg["rotary_scale"])
            x = x + P.linear(P.causal_attention(q, k, v).reshape(T, nh * hd), W[a + "o_proj.weight"])
            n = P.rms_norm(x, W[p + "n2.weight"], cfg["eps"])
            x = x + P.gated_mlp(n, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, W["model.norm.weight"], cfg["eps"]), W["lm_head.weight"])


def read_folder(model_dir: str):
    """(config.json as a dict, tensors) with the plain implementation's own readers."""
    import os
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, P.read_safetensors(os.path.join(model_dir, "model.safetensors"))


def greedy_continuation(W, cfg, prompt, n):
    toks = list(prompt)
    out = []
    for _ in range(n):
        t = P.greedy(reference_logits(W, cfg, toks)[-1])
        out.append(t)
        toks.append(t)
    return out


register()
