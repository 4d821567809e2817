"""The tiny Qwen3 configurations of the tests.  They differ in every size and option: layers, width,
head counts and group size, head_dim (16 / 32 / 48), heads * head_dim equal to the width or not,
intermediate size, an even or odd vocabulary that is no power of two, rope_theta, the norms' eps,
tied or untied head, and no window / a window on some layers."""

TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
              intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=2048,
              hidden_act="silu", attention_bias=False, use_sliding_window=False)

TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=509, hidden_size=96,
              intermediate_size=224, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=2048,
              hidden_act="silu", attention_bias=False, use_sliding_window=False)

TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=301, hidden_size=80,
              intermediate_size=176, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
              rope_theta=500000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=4096,
              hidden_act="silu", attention_bias=False, sliding_window=24,
              layer_types=["sliding_attention", "full_attention", "sliding_attention"])

# head_dim 64: the size from which the bfloat16 path runs its tensor-core attention kernels
TINY_D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=400, hidden_size=128,
              intermediate_size=192, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
              rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
              hidden_act="silu", attention_bias=False, sliding_window=70,
              layer_types=["full_attention", "sliding_attention"])

# head_dim 128 with groups of 4: the sizes from which prompts run the tcgen05 attention kernel
TINY_E = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=333, hidden_size=192,
              intermediate_size=320, num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
              rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096,
              hidden_act="silu", attention_bias=False, sliding_window=150,
              layer_types=["sliding_attention", "full_attention"])

# name -> (config.json dict, weight seed)
TINY = {"a": (TINY_A, 0), "b": (TINY_B, 1), "c": (TINY_C, 2), "d": (TINY_D, 3), "e": (TINY_E, 4)}
