"""The Qwen3-8B layer sizes (width 4096, 32 / 8 heads of 128, intermediate 12288, vocabulary 151936, theta 1e6)
with two layers and seeded random bfloat16 weights, against the plain implementation run on the same GPU in
float32: the sizes at which the serving path uses its tcgen05 / TMA kernels.  Each request whole, with its
tail decoded token by token, in portions, and mixed with others in a small pool."""
import numpy as np
import pytest
import torch

import plain_model
import traces
from helpers import tokens_for

pytestmark = pytest.mark.gpu

CONFIG = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
              intermediate_size=12288, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
              rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960,
              hidden_act="silu", attention_bias=False, use_sliding_window=False)
# float32 against a float32 oracle: sums of up to 12288 products on both sides; bfloat16 as everywhere
TOLERANCE = {"float32": 2e-4, "bfloat16": 3e-2}


class KeptSource:
    """Random tensors made on the GPU, kept so that the plain side sees the same values."""

    def __init__(self, spec, seed, dtype):
        from llmserver_b200.weights import RandomSource
        self.inner = RandomSource(spec, seed, torch.bfloat16, "cuda:0")
        self.dtype, self.seen = dtype, {}

    def get(self, name):
        tensor = self.inner.get(name)
        self.seen[name] = tensor
        return tensor.to(self.dtype)


@pytest.fixture(scope="module")
def shaped():
    from llmserver_b200.config import ARCHITECTURES, Qwen3Config
    import llmserver_b200.models  # noqa: F401
    config = Qwen3Config.from_dict(CONFIG)
    spec = ARCHITECTURES["Qwen3ForCausalLM"].build_spec(config)
    return config, spec


def plain_rows(weights, tokens):
    with torch.no_grad():
        return plain_model.forward(CONFIG, weights, tokens).float().cpu().numpy()


def close(got, want, dtype, what):
    scale = np.abs(want).max(axis=-1, keepdims=True)
    error = (np.abs(got - want).max(axis=-1, keepdims=True) / scale).max()
    assert np.isfinite(got).all() and error <= TOLERANCE[dtype], f"{what}: relative error {error:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_8b_sized_layers_under_every_cut(shaped, dtype):
    from llmserver_b200.cache import CacheManager
    from llmserver_b200.engine.step import StepFunction
    from llmserver_b200.models import DecoderModel
    from llmserver_b200.models.loading import as_dtype
    from llmserver_b200.parts import Runtime

    config, spec = shaped
    torch.manual_seed(0)
    source = KeptSource(spec, 11, as_dtype(dtype))
    model = DecoderModel(spec, source, Runtime(as_dtype(dtype), torch.device("cuda:0")))
    model.config = config
    # the plain functions patch torch.arange-based masks on the CPU; run them on the GPU tensors in float32
    weights = {name: tensor.float() for name, tensor in source.seen.items()}
    requests = {"a": tokens_for(151936, 300, 1), "b": tokens_for(151936, 97, 2), "c": tokens_for(151936, 190, 3)}
    default = torch.get_default_device() if hasattr(torch, "get_default_device") else None
    torch.set_default_device("cuda:0")
    try:
        expected = {name: plain_rows(weights, tokens) for name, tokens in requests.items()}
    finally:
        torch.set_default_device(default or "cpu")
    del weights
    torch.cuda.empty_cache()

    def replay(records, max_tokens):
        cache = CacheManager(model.cache_needs(), 16, max(1, max_tokens // 16), num_slots=4, prefix_sharing=False)
        cache.materialize(model.runtime.device, model.runtime.dtype)
        step = StepFunction(model, cache)
        live, out = set(), {}
        for record in records:
            entries = []
            for entry in record["entries"]:
                if entry["id"] not in live:
                    step.admit(entry["id"])
                    live.add(entry["id"])
                entries.append((entry["id"], entry["tokens"], entry["want"]))
            logits = step.run(entries)
            if logits.shape[0]:
                out[record["step"]] = logits.cpu().numpy()
            for name in record["end"]:
                step.release(name)
                live.discard(name)
        step.check_errors()
        cache.check_invariants()
        return out

    def compare(records, got, what):
        want = traces.expected_rows(records, requests, lambda name: expected[name])
        assert set(got) == set(want)
        for step_index in want:
            close(got[step_index], want[step_index], dtype, f"{what}, step {step_index}")

    records = traces.whole("a", requests["a"])
    compare(records, replay(records, 320), "whole")
    records = traces.tail_decoded("c", requests["c"], 32)
    compare(records, replay(records, 192), "tail decoded")
    records = traces.portions("a", requests["a"], [7, 2, 130, 3, 64, 2, 33])
    compare(records, replay(records, 320), "portions")
    records, peak = traces.mixed(requests, seed=4, max_live=3)
    compare(records, replay(records, peak), "mixed")
