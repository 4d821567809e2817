"""Compares the plain implementation (tests/plain_model.py) once with AshvinSehgal/LLMServer's own
model code on two tiny random models, on the CPU in float32, and writes the small outputs that
tests/test_plain_model.py checks against.

    python tests/golden/make_golden.py /path/to/LLMServer

The reference's ``utils.model.Model`` is imported from the given checkout, filled with the tensors of a
model folder written by this engine's random-weights mode (same names; the tied configuration sets
``lm_head.weight`` to the embedding), and run on whole sequences.  Only configurations the reference
runs are used (it refuses sliding windows).  Outputs: ``tests/golden/tiny_<name>.npz`` with the token
ids, the reference's logits and the largest difference seen when this script ran.
"""
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def main(reference_root):
    sys.path.insert(0, reference_root)
    from utils.model import Model  # the reference's model (utils/model.py:43)

    import plain_model
    from tiny_configs import TINY
    from llmserver_b200.config import Qwen3Config
    from llmserver_b200.weights import write_model_folder
    import llmserver_b200.models  # noqa: F401

    for name in ("a", "b"):
        raw, seed = TINY[name]
        with tempfile.TemporaryDirectory() as folder:
            write_model_folder(Qwen3Config.from_dict(raw), folder, seed, torch.bfloat16)
            config, weights = plain_model.read_model_folder(folder, torch.float32)
        head_dim = plain_model.head_dim_of(config)
        model = Model(vocab_size=config["vocab_size"], hidden_size=config["hidden_size"],
                      intermediate_size=config["intermediate_size"], n_hidden_layers=config["num_hidden_layers"],
                      head_dim=head_dim, rope_theta=plain_model.rope_theta_of(config),
                      n_query_heads=config["num_attention_heads"], n_kv_heads=config["num_key_value_heads"], bias=False,
                      attention_scaling=head_dim ** -0.5, rms_norm_eps=config["rms_norm_eps"])
        state = {key[len("model."):] if key.startswith("model.") else key: value for key, value in weights.items()}
        if "lm_head.weight" not in state:
            state["lm_head.weight"] = state["embed_tokens.weight"]
        model.load_state_dict(state, strict=True)
        model.eval()
        generator = torch.Generator().manual_seed(1234 + seed)
        tokens = torch.randint(0, config["vocab_size"], (2, 23), generator=generator)
        with torch.inference_mode():
            reference = model(tokens).float()
        worst = 0.0
        for row in range(tokens.shape[0]):
            ours = plain_model.forward(config, weights, tokens[row].tolist())
            worst = max(worst, (ours - reference[row]).abs().max().item())
        print(f"tiny {name}: max |plain - reference| = {worst:.3e} (largest logit {reference.abs().max().item():.3f})")
        assert worst < 2e-5
        np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), tokens=tokens.numpy().astype(np.int32),
                            logits=reference.numpy().astype(np.float32), worst_difference=np.float32(worst))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/LLMServer")
    main(sys.argv[1])
