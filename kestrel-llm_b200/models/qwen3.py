"""Qwen3 dense decoder assembled from parts.

Per layer (reference: src/model/vllm_safetensors.c:16404-16812, float32 branches): RMSNorm,
grouped-query attention with per-head QK RMSNorm and rotate-half RoPE, residual; RMSNorm,
SwiGLU MLP, residual; then a final RMSNorm and the output head.  Checkpoint tensor names are
the ones the reference's converter binds (vqf_convert/src/model_layers.c:150-166, 296-301;
vqf_convert/src/conv_main.c:588-614).  Whether a layer attends to all keys or to a window is
read per layer from the configuration.
"""
from __future__ import annotations

import torch

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..csrc import ops
from ..parts import (GatedMLP, GroupedQueryAttention, LMHead, PreNormBlock, RMSNorm, RotaryHalf,
                     TokenEmbedding)
from .decoder import DecoderModel, LayerCall


def build_qwen3(config: Qwen3Config, dtype: torch.dtype, device) -> DecoderModel:
    c = config
    emb = TokenEmbedding(c.vocab_size, c.hidden_size, dtype, device, "model.embed_tokens.weight")
    rope = RotaryHalf(c.head_dim, c.rope_theta, device)
    planner = ops.AttentionPlanner() if dtype == torch.bfloat16 and torch.device(device).type == "cuda" else None
    blocks = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = GroupedQueryAttention(c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
                                      c.head_dim, dtype, device, p + "self_attn.", rope,
                                      qk_norm_eps=c.qk_norm_eps, bias=c.attention_bias,
                                      window=c.layer_window(i), planner=planner)
        ffn = GatedMLP(c.hidden_size, c.intermediate_size, dtype, device, p + "mlp.", c.hidden_act)
        blocks.append(PreNormBlock(RMSNorm(c.hidden_size, c.rms_norm_eps, device, p + "input_layernorm.weight"),
                                   mixer,
                                   RMSNorm(c.hidden_size, c.rms_norm_eps, device, p + "post_attention_layernorm.weight"),
                                   ffn, dtype))
    order = [LayerCall(block=i, cache=i) for i in range(c.num_hidden_layers)]
    final_norm = RMSNorm(c.hidden_size, c.rms_norm_eps, device, "model.norm.weight")
    head = LMHead(c.vocab_size, c.hidden_size, dtype, device, "lm_head.weight",
                  tied_to=emb if c.tie_word_embeddings else None)
    optional = ("lm_head.weight",) if c.tie_word_embeddings else ()
    return DecoderModel(c, dtype, device, emb, rope, blocks, order, final_norm, head, optional)


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3)
