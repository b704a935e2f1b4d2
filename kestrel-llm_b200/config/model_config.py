"""Typed model configuration read from an architecture's own ``config.json`` keys.

The reference reads the same keys with a substring search
(vqf_convert/src/model_cfgio.c:246-296) into ``STModelConfig``
(include/model/vllm_safetensors.h:59-113) and checks almost nothing; here every key is
typed, defaulted or required explicitly, and validated, and an unknown architecture is an
error rather than a guess.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model this engine runs."""


def _need(d: Dict[str, Any], key: str, typ):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    return _typed(d, key, typ)


def _typed(d: Dict[str, Any], key: str, typ):
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                return int(v)
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
        return v
    return v


def _opt(d: Dict[str, Any], key: str, typ, default):
    if key not in d or d[key] is None:
        return default
    return _typed(d, key, typ)


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration offers the engine."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    bos_token_id: Optional[int]
    eos_token_ids: tuple

    def to_json_dict(self) -> Dict[str, Any]:  # pragma: no cover - overridden
        raise NotImplementedError


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder.  Field names are the config.json keys."""

    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    qk_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    hidden_act: str = "silu"
    sliding_window: int = 0
    layer_types: tuple = field(default_factory=tuple)   # "full_attention" | "sliding_attention" per layer
    torch_dtype: str = "bfloat16"

    # derived sizes -------------------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> int:
        """Number of keys a layer attends to, 0 meaning all of them."""
        if self.layer_types and self.layer_types[layer] == "sliding_attention":
            return self.sliding_window
        return 0

    # parsing -------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "Qwen3Config":
        d = dict(raw)
        # A multimodal checkpoint nests the decoder's keys (the reference finds them there by
        # the order of its substring search, model_cfgio.c:20-28); take them explicitly.
        if "hidden_size" not in d and isinstance(d.get("text_config"), dict):
            nested = dict(d["text_config"])
            for k in ("architectures", "tie_word_embeddings"):
                if k in d and k not in nested:
                    nested[k] = d[k]
            d = nested
        archs = d.get("architectures") or []
        arch = archs[0] if archs else "Qwen3ForCausalLM"
        hidden = _need(d, "hidden_size", int)
        layers = _need(d, "num_hidden_layers", int)
        heads = _need(d, "num_attention_heads", int)
        kv_heads = _opt(d, "num_key_value_heads", int, heads)
        ff = _need(d, "intermediate_size", int)
        vocab = _need(d, "vocab_size", int)
        # head_dim: explicit, else hidden/heads (model_cfgio.c:285-291, without its last
        # resort of guessing 128).
        head_dim = _opt(d, "head_dim", int, 0)
        for name, v in (("hidden_size", hidden), ("num_hidden_layers", layers),
                        ("num_attention_heads", heads), ("num_key_value_heads", kv_heads),
                        ("intermediate_size", ff), ("vocab_size", vocab)):
            if v <= 0:
                raise ConfigError(f"config.json: '{name}' must be positive, got {v}")
        if head_dim <= 0:
            if hidden % heads:
                raise ConfigError("config.json: no 'head_dim' and hidden_size is not a multiple of "
                                  "num_attention_heads")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"config.json: num_attention_heads ({heads}) must be a multiple of "
                              f"num_key_value_heads ({kv_heads})")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({head_dim}) must be even for rotate-half RoPE")
        act = d.get("hidden_act", "silu") or "silu"
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (only 'silu')")
        if d.get("rope_scaling") not in (None, {}):
            rs = d["rope_scaling"]
            rtype = rs.get("rope_type", rs.get("type")) if isinstance(rs, dict) else rs
            if rtype not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling {rs!r} is not supported")
        eps = _opt(d, "rms_norm_eps", float, 1e-6)
        theta = _opt(d, "rope_theta", float, 10000.0)
        if theta <= 0 or eps <= 0:
            raise ConfigError("config.json: rope_theta and rms_norm_eps must be positive")
        max_pos = _opt(d, "max_position_embeddings", int, 32768)
        if max_pos <= 0:
            raise ConfigError("config.json: max_position_embeddings must be positive")

        # sliding window: per-layer list if given, else the max_window_layers rule
        sw = _opt(d, "sliding_window", int, 0)
        use_sw = _opt(d, "use_sliding_window", bool, False)
        lt = d.get("layer_types")
        if lt is not None:
            if not isinstance(lt, list) or len(lt) != layers:
                raise ConfigError(f"config.json: layer_types must list {layers} layers")
            for t in lt:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"config.json: unknown layer type '{t}'")
            layer_types = tuple(lt)
        elif use_sw and sw > 0:
            first = _opt(d, "max_window_layers", int, 0)
            layer_types = tuple("sliding_attention" if i >= first else "full_attention"
                                for i in range(layers))
        else:
            layer_types = tuple("full_attention" for _ in range(layers))
        if "sliding_attention" in layer_types and sw <= 0:
            raise ConfigError("config.json: sliding_attention layers need a positive 'sliding_window'")
        if "sliding_attention" not in layer_types:
            sw = 0

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, list):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (_typed(d, "eos_token_id", int),)
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: eos_token_id {e} outside the vocabulary")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16")) or "bfloat16"
        return cls(
            architecture=arch, vocab_size=vocab, hidden_size=hidden, num_hidden_layers=layers,
            max_position_embeddings=max_pos, bos_token_id=_opt(d, "bos_token_id", int, None),
            eos_token_ids=eos_ids, num_attention_heads=heads, num_key_value_heads=kv_heads,
            head_dim=head_dim, intermediate_size=ff, rope_theta=theta, rms_norm_eps=eps,
            qk_norm_eps=_opt(d, "qk_norm_eps", float, eps),
            tie_word_embeddings=_opt(d, "tie_word_embeddings", bool, False),
            attention_bias=_opt(d, "attention_bias", bool, False), hidden_act=act,
            sliding_window=sw, layer_types=layer_types, torch_dtype=str(dtype))

    def to_json_dict(self) -> Dict[str, Any]:
        """The config.json that parses back to this configuration."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "rms_norm_eps": self.rms_norm_eps,
            "hidden_act": self.hidden_act,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "torch_dtype": self.torch_dtype,
        }
        if self.qk_norm_eps != self.rms_norm_eps:
            out["qk_norm_eps"] = self.qk_norm_eps
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            out["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 \
                else list(self.eos_token_ids)
        if self.sliding_window:
            out["sliding_window"] = self.sliding_window
            out["use_sliding_window"] = True
            out["layer_types"] = list(self.layer_types)
        return out


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw
