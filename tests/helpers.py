"""Shared helpers of the GPU tests: token streams, the plain oracle's logits and the comparison rule."""
import functools

import numpy as np
import torch

import plain_model

# Largest allowed |engine - plain| as a fraction of the largest |plain logit| of the same row.
# float32: sums of a few hundred to a few thousand float32 products against a float64 oracle.
# bfloat16: activations are rounded to 8 significant bits between kernels (about 4e-3 each time).
TOLERANCE = {"float32": 2e-5, "bfloat16": 3e-2}


def tokens_for(vocab, length, seed):
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


_PLAIN_CACHE = {}


def plain_folder(folder):
    if folder not in _PLAIN_CACHE:
        _PLAIN_CACHE[folder] = plain_model.read_model_folder(folder, torch.float64)
    return _PLAIN_CACHE[folder]


_LOGIT_CACHE = {}


def plain_logits(folder, tokens):
    """float64 logits [T, V] of the whole sequence from the plain implementation (cached)."""
    key = (folder, tuple(tokens))
    if key not in _LOGIT_CACHE:
        config, weights = plain_folder(folder)
        _LOGIT_CACHE[key] = plain_model.forward(config, weights, list(tokens)).numpy()
    return _LOGIT_CACHE[key]


def assert_close(got, want, dtype, what=""):
    """Row by row: max |got - want| <= TOLERANCE * max |want row|; reports the first bad row."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = np.abs(want).max(axis=-1, keepdims=True)
    error = np.abs(got - want).max(axis=-1, keepdims=True) / scale
    bad = np.nonzero(error.reshape(-1) > TOLERANCE[dtype])[0]
    if bad.size:
        raise AssertionError(f"{what}: {bad.size} of {error.size} rows differ; first bad row {int(bad[0])} "
                             f"(relative error {float(error.reshape(-1)[bad[0]]):.3e}, allowed {TOLERANCE[dtype]:.1e}); "
                             f"worst {float(error.max()):.3e}")
    return float(error.max())
