"""Weights by tensor name: the random-weights mode, dtypes, and the one error that lists everything (no GPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from llmserver_b200.config import ARCHITECTURES, Qwen3Config, WeightLoadError
from llmserver_b200.weights import CheckpointReader, CheckpointSource, RandomSource, declared_weights, write_model_folder
import llmserver_b200.models  # noqa: F401
from tiny_configs import TINY_A, TINY_B


def spec_of(raw):
    return ARCHITECTURES["Qwen3ForCausalLM"].build_spec(Qwen3Config.from_dict(raw))


def test_declared_names_are_the_checkpoint_names():
    names = set(declared_weights(spec_of(TINY_B)))
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names and "lm_head.weight" in names
    for part in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "self_attn.q_norm",
                 "self_attn.k_norm", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj", "input_layernorm",
                 "post_attention_layernorm"):
        assert f"model.layers.2.{part}.weight" in names
    assert len(names) == 3 + 3 * 11
    assert "lm_head.weight" not in declared_weights(spec_of(TINY_A))   # tied


def test_random_mode_writes_a_loadable_folder(tmp_path):
    folder = write_model_folder(Qwen3Config.from_dict(TINY_B), str(tmp_path / "m"), seed=1)
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["Qwen3ForCausalLM"]
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    assert all(tensor.dtype == torch.bfloat16 for tensor in tensors.values())
    assert tensors["model.layers.0.self_attn.q_proj.weight"].shape == (6 * 32, 96)
    matrix = tensors["model.layers.1.mlp.down_proj.weight"].float()
    norm = tensors["model.layers.1.input_layernorm.weight"].float()
    assert abs(matrix.std().item() - 0.02) < 0.002 and abs(matrix.mean().item()) < 0.002
    assert abs(norm.mean().item() - 1.0) < 0.05 and 0.05 < norm.std().item() < 0.15
    # same seed, same values; another seed, other values; a tensor does not depend on the others
    again = load_file(os.path.join(write_model_folder(Qwen3Config.from_dict(TINY_B), str(tmp_path / "n"), seed=1), "model.safetensors"))
    other = load_file(os.path.join(write_model_folder(Qwen3Config.from_dict(TINY_B), str(tmp_path / "o"), seed=2), "model.safetensors"))
    assert all(torch.equal(tensors[name], again[name]) for name in tensors)
    assert not torch.equal(tensors["model.norm.weight"], other["model.norm.weight"])
    fewer = dict(TINY_B, num_hidden_layers=1)
    small = load_file(os.path.join(write_model_folder(Qwen3Config.from_dict(fewer), str(tmp_path / "p"), seed=1), "model.safetensors"))
    assert torch.equal(small["model.layers.0.mlp.up_proj.weight"], tensors["model.layers.0.mlp.up_proj.weight"])


def test_loading_keeps_bfloat16_and_does_not_narrow_32_bit_tensors(tmp_path):
    folder = write_model_folder(Qwen3Config.from_dict(TINY_A), str(tmp_path / "m"), seed=0)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float() + 1e-4   # stored in 32-bit
    save_file(tensors, path)
    source = CheckpointSource(folder, spec_of(TINY_A), torch.bfloat16, "cpu")
    assert source.get("model.layers.0.mlp.up_proj.weight").dtype == torch.bfloat16
    assert source.get("model.layers.0.input_layernorm.weight").dtype == torch.bfloat16
    kept = source.get("model.norm.weight")
    assert kept.dtype == torch.float32 and torch.equal(kept, tensors["model.norm.weight"])
    wide = CheckpointSource(folder, spec_of(TINY_A), torch.float32, "cpu")
    assert wide.get("model.layers.0.mlp.up_proj.weight").dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_tensors(tmp_path):
    folder = write_model_folder(Qwen3Config.from_dict(TINY_B), str(tmp_path / "m"), seed=1)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    del tensors["model.layers.1.self_attn.k_norm.weight"]
    del tensors["model.layers.2.mlp.gate_proj.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(96, 100, dtype=torch.bfloat16)
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    save_file(tensors, path)
    with pytest.raises(WeightLoadError) as error:
        CheckpointSource(folder, spec_of(TINY_B), torch.bfloat16, "cpu")
    message = str(error.value)
    assert "missing tensors (2)" in message and "model.layers.1.self_attn.k_norm.weight" in message
    assert "model.layers.2.mlp.gate_proj.weight" in message
    assert "unexpected tensors (1)" in message and "rotary_emb.inv_freq" in message
    assert "model.layers.0.mlp.down_proj.weight: shape [96, 100] where [96, 224] is expected" in message
    assert "model.norm.weight: dtype" in message


def test_a_checkpoint_without_a_head_is_tied(tmp_path):
    folder = write_model_folder(Qwen3Config.from_dict(TINY_B), str(tmp_path / "m"), seed=1)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    del tensors["lm_head.weight"]
    save_file(tensors, path)
    spec = spec_of(TINY_B)
    CheckpointSource(folder, spec, torch.bfloat16, "cpu")
    assert spec.tie_head
    # and a tied configuration may carry a copy of the head, which is ignored
    folder = write_model_folder(Qwen3Config.from_dict(TINY_A), str(tmp_path / "t"), seed=0)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, path)
    CheckpointSource(folder, spec_of(TINY_A), torch.bfloat16, "cpu")


def test_sharded_checkpoints_are_found_through_the_index(tmp_path):
    folder = write_model_folder(Qwen3Config.from_dict(TINY_A), str(tmp_path / "m"), seed=0)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    save_file({name: tensors[name] for name in names[:half]}, os.path.join(folder, "model-00001-of-00002.safetensors"))
    save_file({name: tensors[name] for name in names[half:]}, os.path.join(folder, "model-00002-of-00002.safetensors"))
    os.remove(os.path.join(folder, "model.safetensors"))
    weight_map = {name: ("model-00001-of-00002.safetensors" if index < half else "model-00002-of-00002.safetensors")
                  for index, name in enumerate(names)}
    json.dump({"weight_map": weight_map}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    reader = CheckpointReader(folder)
    assert reader.names() == names and torch.equal(reader.get(names[-1]), tensors[names[-1]])
    with pytest.raises(FileNotFoundError):
        CheckpointReader(str(tmp_path))


def test_random_source_matches_the_written_folder(tmp_path):
    folder = write_model_folder(Qwen3Config.from_dict(TINY_A), str(tmp_path / "m"), seed=7)
    tensors = load_file(os.path.join(folder, "model.safetensors"))
    source = RandomSource(spec_of(TINY_A), 7, torch.bfloat16, "cpu")
    assert torch.equal(source.get("model.layers.1.self_attn.o_proj.weight"), tensors["model.layers.1.self_attn.o_proj.weight"])
