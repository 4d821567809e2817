"""Configuration and registry (no GPU)."""
import json

import pytest

from llmserver_b200.config import (ARCHITECTURES, Qwen3Config, UnsupportedModelError, architecture_of, read_config)
from llmserver_b200.config.spec import ModelSpec, PartSpec, ScheduleEntry
import llmserver_b200.models  # noqa: F401
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_config_json():
    config = Qwen3Config.from_dict(TINY_B)
    assert (config.vocab_size, config.hidden_size, config.intermediate_size) == (509, 96, 224)
    assert (config.num_hidden_layers, config.num_attention_heads, config.num_key_value_heads, config.head_dim) == (3, 6, 1, 32)
    assert config.rope_theta == 1e6 and config.rms_norm_eps == 1e-5 and not config.tie_word_embeddings
    assert config.attention_scale == 32 ** -0.5 and config.group_size == 6
    assert config.layer_types == ("full_attention",) * 3 and config.sliding_window is None


def test_defaults_follow_the_reference():
    raw = dict(TINY_A)
    del raw["head_dim"], raw["rope_theta"]
    config = Qwen3Config.from_dict(raw)
    assert config.head_dim == 64 // 4              # hidden_size // num_attention_heads
    assert config.rope_theta == 10000.0
    raw["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    assert Qwen3Config.from_dict(raw).rope_theta == 12345.0


def test_window_layers():
    config = Qwen3Config.from_dict(TINY_C)
    assert [config.window_of(i) for i in range(3)] == [24, None, 24]
    raw = dict(TINY_B, use_sliding_window=True, sliding_window=10, max_window_layers=2)
    assert [Qwen3Config.from_dict(raw).window_of(i) for i in range(3)] == [None, None, 10]
    # a window that no layer uses is not kept
    assert Qwen3Config.from_dict(dict(TINY_A, sliding_window=4096)).sliding_window is None


@pytest.mark.parametrize("change,words", [
    ({"num_key_value_heads": 3}, "multiple of num_key_value_heads"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "RoPE type 'yarn'"),
    ({"partial_rotary_factor": 0.5}, "partial rotary"),
    ({"attn_logit_softcapping": 50.0}, "attn_logit_softcapping"),
    ({"attention_bias": True}, "biases"),
    ({"hidden_act": "gelu"}, "activation 'gelu'"),
    ({"layer_types": ["full_attention"]}, "layer_types has 1 entries"),
    ({"layer_types": ["sliding_attention", "full_attention"], "sliding_window": None}, "positive sliding_window"),
    ({"vocab_size": None}, "lacks required keys: vocab_size"),
    ({"rms_norm_eps": None}, "rms_norm_eps"),
])
def test_refusals_say_what_is_different(change, words):
    with pytest.raises(UnsupportedModelError) as error:
        Qwen3Config.from_dict(dict(TINY_A, **change))
    assert words in str(error.value)


def test_round_trip_through_config_json(tmp_path):
    for raw in (TINY_A, TINY_B, TINY_C):
        config = Qwen3Config.from_dict(raw)
        (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
        again, architecture = read_config(str(tmp_path))
        assert again == config and architecture.name == "Qwen3ForCausalLM"


def test_registry_chooses_by_architecture_name():
    assert "Qwen3ForCausalLM" in ARCHITECTURES
    with pytest.raises(UnsupportedModelError) as error:
        architecture_of({"architectures": ["GemmaForCausalLM"]})
    assert "GemmaForCausalLM" in str(error.value) and "Qwen3ForCausalLM" in str(error.value)
    with pytest.raises(UnsupportedModelError):
        architecture_of({})


def test_spec_carries_sizes_layer_by_layer():
    spec = ARCHITECTURES["Qwen3ForCausalLM"].build_spec(Qwen3Config.from_dict(TINY_C))
    assert [layer.mixer.get("window") for layer in spec.layers] == [24, None, 24]
    assert spec.layers[0].mixer.get("head_dim") == 48 and spec.layers[0].feed_forward.get("intermediate") == 176
    assert spec.layers[0].mixer_norm.get("eps") == 3e-6 and spec.positions["rotary"].get("theta") == 500000.0
    assert [entry.layer for entry in spec.schedule] == [0, 1, 2]
    spec.validate()


def test_schedule_validation():
    spec = ARCHITECTURES["Qwen3ForCausalLM"].build_spec(Qwen3Config.from_dict(TINY_A))
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_from=1), ScheduleEntry(0)]
    spec.validate()
    spec.schedule = [ScheduleEntry(0, cache_from=0)]
    with pytest.raises(ValueError):
        spec.validate()
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1, cache_from=0), ScheduleEntry(1, cache_from=1)]
    with pytest.raises(ValueError):
        spec.validate()
    spec.schedule = [ScheduleEntry(5)]
    with pytest.raises(ValueError):
        spec.validate()


def test_a_published_qwen3_config_json_parses():
    """The keys of a published Qwen3-8B config.json, nulls and unused keys included."""
    raw = {"architectures": ["Qwen3ForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 151643,
           "eos_token_id": 151645, "head_dim": 128, "hidden_act": "silu", "hidden_size": 4096, "initializer_range": 0.02,
           "intermediate_size": 12288, "max_position_embeddings": 40960, "max_window_layers": 36, "model_type": "qwen3",
           "num_attention_heads": 32, "num_hidden_layers": 36, "num_key_value_heads": 8, "rms_norm_eps": 1e-06,
           "rope_scaling": None, "rope_theta": 1000000, "sliding_window": None, "tie_word_embeddings": False,
           "torch_dtype": "bfloat16", "transformers_version": "4.51.0", "use_cache": True, "use_sliding_window": False,
           "vocab_size": 151936}
    config = Qwen3Config.from_dict(raw)
    assert config.layer_types == ("full_attention",) * 36 and config.sliding_window is None
    assert config.eos_token_id == (151645,) and config.rope_theta == 1e6 and config.head_dim == 128
    spec = ARCHITECTURES["Qwen3ForCausalLM"].build_spec(config)
    assert len(spec.layers) == 36 and spec.max_positions == 40960 and not spec.tie_head


def test_generation_config_overrides_eos(tmp_path):
    from llmserver_b200.models.loading import generation_eos_ids
    assert generation_eos_ids(str(tmp_path)) is None
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [151645, 151643], "temperature": 0.6}))
    assert generation_eos_ids(str(tmp_path)) == (151645, 151643)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 7}))
    assert generation_eos_ids(str(tmp_path)) == (7,)
