"""Tiny configurations of the Qwen3 dense decoder for tests.  A and B differ in every size and
option (layers, width, heads and groups, head size, feed-forward width, vocabulary, rope
theta, the norms' eps, tied or separate head, attention bias, context limit); C adds windowed
layers between full ones, so two cache groups exist and pages fall out of the window.  No
size is a power of two in B and C where it need not be.  D and E have the head sizes 128 and 64,
for which the bfloat16 path has kernels of its own (tcgen05 attention of prompt portions, the
decode attention with the TMA loader): D with grouped heads and a windowed layer between full
ones, E with six query heads on one kv head.  F has eighteen query heads on one kv head: more
rows a token than the 16-row tiles of the decode kernels and of a captured step hold."""

A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
         num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
         rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False,
         max_position_embeddings=256, hidden_act="silu")

B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
         num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=200, vocab_size=509,
         rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=True,
         max_position_embeddings=512, hidden_act="silu")

C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
         num_attention_heads=5, num_key_value_heads=5, head_dim=48, intermediate_size=136, vocab_size=301,
         rope_theta=50000.0, rms_norm_eps=3e-6, qk_norm_eps=2e-5, tie_word_embeddings=False,
         attention_bias=False, max_position_embeddings=384, hidden_act="silu", sliding_window=40,
         use_sliding_window=True,
         layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"])

D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=192,
         num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=328, vocab_size=333,
         rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False,
         max_position_embeddings=512, hidden_act="silu", sliding_window=70, use_sliding_window=True,
         layer_types=["full_attention", "sliding_attention", "full_attention"])

E = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=136,
         num_attention_heads=6, num_key_value_heads=1, head_dim=64, intermediate_size=200, vocab_size=277,
         rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=True,
         max_position_embeddings=512, hidden_act="silu")

F = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=88,
         num_attention_heads=18, num_key_value_heads=1, head_dim=128, intermediate_size=120, vocab_size=211,
         rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, attention_bias=False,
         max_position_embeddings=512, hidden_act="silu")

CONFIGS = {"A": (A, 0), "B": (B, 2), "C": (C, 5), "D": (D, 7), "E": (E, 9), "F": (F, 11)}
