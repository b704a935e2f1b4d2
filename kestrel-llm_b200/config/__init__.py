from .model_config import ConfigError, ModelConfig, Qwen3Config, read_config_json
from .registry import (Architecture, architecture_of, known_architectures, load_config,
                       register_architecture, resolve_architecture)
from .engine_options import EngineOptions

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "read_config_json", "Architecture",
           "architecture_of", "known_architectures", "load_config", "register_architecture",
           "resolve_architecture", "EngineOptions"]
