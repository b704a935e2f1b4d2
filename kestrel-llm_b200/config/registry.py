"""One registry from an architecture's name (``architectures[0]`` of config.json) to its
configuration class and model builder.

The reference has no registry: it switches on substrings of config.json
(vqf_convert/src/model_cfgio.c:293-296, 303, 350).  Here an unknown name is an error that
lists the known ones.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Type

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Type[ModelConfig]
    build: Callable[..., Any]            # build(config, dtype, device) -> model (weights unset)


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type[ModelConfig], build: Callable[..., Any]) -> None:
    """Add an architecture.  Registering a name twice replaces the earlier entry, so a test
    can register a toy model without touching the package."""
    _ARCHITECTURES[name] = Architecture(name, config_class, build)


def known_architectures() -> List[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def resolve_architecture(name: str) -> Architecture:
    _load_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not registered; known: "
                          f"{', '.join(sorted(_ARCHITECTURES))}")
    return _ARCHITECTURES[name]


def architecture_of(raw: Dict[str, Any]) -> str:
    archs = raw.get("architectures")
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must name the model class, e.g. "
                          "[\"Qwen3ForCausalLM\"]")
    return archs[0]


def load_config(model_dir: str) -> ModelConfig:
    """Parse ``model_dir/config.json`` with the class its architecture registers."""
    raw = read_config_json(model_dir)
    arch = resolve_architecture(architecture_of(raw))
    return arch.config_class.from_dict(raw)


def _load_builtin() -> None:
    # The built-in models register themselves on import.
    from .. import models  # noqa: F401
