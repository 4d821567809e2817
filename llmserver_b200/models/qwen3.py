"""Qwen3 dense: from its typed configuration to the architecture-neutral model specification.

This is the only place that knows how Qwen3 arranges its parts and names its tensors
(utils/model.py:7-54 and utils/attention.py:33-39, utils/layers.py:188-191 for the names):
pre-norm layers, grouped-query attention with per-head Q/K RMSNorm and rotary positions, a SwiGLU
feed-forward, RMSNorm everywhere, an output head that may be tied to the embedding.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def qwen3_spec(config: Qwen3Config) -> ModelSpec:
    norm = PartSpec.of("rmsnorm", width=config.hidden_size, eps=config.rms_norm_eps)
    block = PartSpec.of("pre_norm", mixer_prefix="self_attn.", feed_forward_prefix="mlp.",
                        mixer_norm_prefix="input_layernorm.", feed_forward_norm_prefix="post_attention_layernorm.")
    feed_forward = PartSpec.of("swiglu", hidden=config.hidden_size, intermediate=config.intermediate_size)
    layers = []
    for index in range(config.num_hidden_layers):
        mixer = PartSpec.of("gqa_attention", hidden=config.hidden_size, heads=config.num_attention_heads,
                            kv_heads=config.num_key_value_heads, head_dim=config.head_dim,
                            scale=config.attention_scale, qk_norm=True, eps=config.rms_norm_eps,
                            window=config.window_of(index))
        layers.append(LayerSpec(prefix=f"model.layers.{index}.", block=block, mixer=mixer, feed_forward=feed_forward,
                                mixer_norm=norm, feed_forward_norm=norm, position="rotary"))
    return ModelSpec(
        architecture=config.architecture, vocab_size=config.vocab_size, hidden_size=config.hidden_size,
        layers=layers, schedule=[ScheduleEntry(index) for index in range(config.num_hidden_layers)],
        positions={"rotary": PartSpec.of("rotary", head_dim=config.head_dim, theta=config.rope_theta)},
        final_norm=norm, tie_head=config.tie_word_embeddings, max_positions=config.max_position_embeddings,
        eos_token_ids=config.eos_token_id,
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_spec)
