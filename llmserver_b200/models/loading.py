"""From a model folder, or from a configuration and a seed, to a model on the device."""
from __future__ import annotations

import json
import os

import torch

from ..config.registry import ARCHITECTURES, read_config
from ..parts import Runtime
from ..weights import CheckpointSource, RandomSource
from .decoder import DecoderModel

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def as_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {dtype}")
        return dtype
    if dtype not in DTYPES:
        raise ValueError(f"unknown dtype {dtype!r} (known: {', '.join(sorted(DTYPES))})")
    return DTYPES[dtype]


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> DecoderModel:
    """Reads config.json, chooses the model by its architecture name and loads model.safetensors.
    The reference's ``model_loader`` (utils/model_loader.py:18-86) does the same through a Hugging
    Face module tree; only local folders are read here."""
    config, architecture = read_config(model_dir)
    spec = architecture.build_spec(config)
    runtime = Runtime(as_dtype(dtype), torch.device(device))
    eos = generation_eos_ids(model_dir)
    if eos is not None:
        spec.eos_token_ids = eos
    model = DecoderModel(spec, CheckpointSource(model_dir, spec, runtime.dtype, runtime.device), runtime)
    model.config = config
    return model


def generation_eos_ids(model_dir: str):
    """End-of-sequence ids of generation_config.json when the folder has one; they take precedence over
    config.json's, as in the reference (utils/engine.py:107-117)."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return None
    with open(path) as handle:
        eos = json.load(handle).get("eos_token_id")
    if eos is None:
        return None
    return (int(eos),) if isinstance(eos, int) else tuple(int(token) for token in eos)


def random_model(config, seed: int, dtype="bfloat16", device="cuda:0", spec=None) -> DecoderModel:
    """A model with seeded random weights made on the device (nothing is written or read)."""
    if spec is None:
        spec = ARCHITECTURES[config.architecture].build_spec(config)
    runtime = Runtime(as_dtype(dtype), torch.device(device))
    model = DecoderModel(spec, RandomSource(spec, seed, runtime.dtype, runtime.device), runtime)
    model.config = config
    return model
