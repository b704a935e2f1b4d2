from .decoder import DecoderModel, LayerCall
from . import qwen3  # registers "Qwen3ForCausalLM"

__all__ = ["DecoderModel", "LayerCall", "qwen3"]
