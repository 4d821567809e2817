"""The plain implementation itself (no GPU): it reproduces the reference model's logits recorded under
tests/golden/ (see make_golden.py), and its generalisations behave as documented."""
import math
import os

import numpy as np
import pytest
import torch

import plain_model
from tiny_configs import TINY

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["a", "b"])
def test_reproduces_the_reference_models_logits(tiny_folders, name):
    golden = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
    config, weights = plain_model.read_model_folder(tiny_folders[name], torch.float32)
    for row in range(golden["tokens"].shape[0]):
        ours = plain_model.forward(config, weights, golden["tokens"][row].tolist()).numpy()
        assert np.abs(ours - golden["logits"][row]).max() < 2e-5
    # and in float64 it stays within float32 rounding of the same numbers
    config, weights = plain_model.read_model_folder(tiny_folders[name], torch.float64)
    ours = plain_model.forward(config, weights, golden["tokens"][0].tolist()).numpy()
    assert np.abs(ours - golden["logits"][0]).max() < 2e-5


def test_causality_and_prefix_property(tiny_folders):
    config, weights = plain_model.read_model_folder(tiny_folders["c"], torch.float64)
    tokens = torch.randint(0, config["vocab_size"], (60,), generator=torch.Generator().manual_seed(0)).tolist()
    whole = plain_model.forward(config, weights, tokens)
    assert torch.allclose(plain_model.forward(config, weights, tokens[:37]), whole[:37], atol=1e-12)


def test_window_semantics():
    torch.manual_seed(0)
    q, k, v = torch.randn(9, 2, 4, dtype=torch.float64), torch.randn(9, 1, 4, dtype=torch.float64), torch.randn(9, 1, 4, dtype=torch.float64)
    full = plain_model.causal_attention(q, k, v, 0.5)
    assert torch.allclose(plain_model.causal_attention(q, k, v, 0.5, window=9), full)
    one = plain_model.causal_attention(q, k, v, 0.5, window=1)        # each query sees itself only
    assert torch.allclose(one.view(9, 2, 4), v.expand(9, 2, 4))
    three = plain_model.causal_attention(q, k, v, 0.5, window=3)
    assert torch.allclose(three[:3], full[:3]) and not torch.allclose(three[3:], full[3:])
    by_hand = plain_model.causal_attention(q[4:7], k[4:7], v[4:7], 0.5)[-1]     # query 6 sees keys 4, 5, 6
    assert torch.allclose(three[6], by_hand)


def test_order_may_repeat_layers_and_share_keys_and_values(tiny_folders):
    config, weights = plain_model.read_model_folder(tiny_folders["a"], torch.float64)
    tokens = list(range(3, 20))
    default = plain_model.forward(config, weights, tokens)
    assert torch.equal(plain_model.forward(config, weights, tokens, order=[(0, None), (1, None)]), default)
    twice = plain_model.forward(config, weights, tokens, order=[(0, None), (1, None), (1, None)])
    shared = plain_model.forward(config, weights, tokens, order=[(0, None), (1, None), (1, 1)])
    assert not torch.allclose(twice, default) and not torch.allclose(shared, twice)


def test_rope_matches_complex_rotation():
    positions = torch.tensor([0, 1, 7, 300])
    cosine, sine = plain_model.rope_tables(positions, 8, 10000.0, torch.float64)
    x = torch.randn(4, 1, 8, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    rotated = plain_model.apply_rope(x, cosine, sine)
    for row, position in enumerate(positions.tolist()):
        for i in range(4):
            angle = float(torch.tensor(position, dtype=torch.float32) * (1.0 / (torch.tensor(10000.0) ** (torch.tensor(2.0 * i) / 8))))
            pair = complex(x[row, 0, i], x[row, 0, i + 4]) * complex(math.cos(angle), math.sin(angle))
            assert abs(rotated[row, 0, i] - pair.real) < 1e-9 and abs(rotated[row, 0, i + 4] - pair.imag) < 1e-9


def test_counter_based_uniforms_and_gumbel_choice():
    values = [plain_model.uniform_for(3, step, index) for step in range(20) for index in range(50)]
    assert all(0.0 < value < 1.0 for value in values) and len(set(values)) > 990
    assert abs(sum(values) / len(values) - 0.5) < 0.03
    assert plain_model.uniform_for(3, 1, 2) == plain_model.uniform_for(3, 1, 2) != plain_model.uniform_for(4, 1, 2)
    logits = torch.tensor([0.0, 5.0, -2.0])
    picks = [int(torch.argmax(plain_model.gumbel_scores(logits, 0.5, 11, step))) for step in range(200)]
    assert picks.count(1) > 190           # softmax(logits / 0.5) puts 0.99995 on token 1
    assert plain_model.greedy(torch.tensor([1.0, 3.0, 3.0])) == 1
