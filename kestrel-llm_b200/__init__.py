"""kestrel-llm_b200: a single-GPU inference engine for the Qwen3 dense decoder on NVIDIA B200.

Typed configuration and an architecture registry (`config`), safetensors weights by tensor
name and a random-weights mode (`weights`), layers assembled from parts (`parts`, `models`),
a paged cache manager (`cache`), one step function, a scheduler and the generation loop
(`engine`), sampling (`sampling`), and hand-written sm_100a kernels with their native host
runtime (`csrc`).  Import as ``kestrel_llm_b200``.
"""
__version__ = "0.1.0"

_LAZY = {
    "LLM": ("engine.llm", "LLM"),
    "SamplingParams": ("sampling.params", "SamplingParams"),
    "EngineOptions": ("config.engine_options", "EngineOptions"),
    "load_config": ("config.registry", "load_config"),
    "register_architecture": ("config.registry", "register_architecture"),
    "load_model": ("weights.loader", "load_model"),
    "write_random_model": ("weights.random_init", "write_random_model"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
