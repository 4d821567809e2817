"""Random-weights mode: tensors from a configuration and a seed, in memory or as a model folder.

Every matrix is N(0, 0.02) and every norm weight 1 + N(0, 0.1).  Each tensor is drawn from its own
generator, seeded by (seed, tensor name), so a tensor's values do not depend on which other tensors
exist or in which order they are made.  The reference has no such mode in its library; its tests
fill a bare model with ``normal_`` (tests/test_fused_ops.py:27-31, tests/test_architectures.py:30-36).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from .declare import MATRIX, NORM, TABLE, WeightDecl, declared_weights


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, declaration: WeightDecl, seed: int, device="cpu") -> torch.Tensor:
    """float32 values (int32 for tables) on ``device``; CPU and CUDA generators give different
    streams, so a model made on one device is not reproduced on the other."""
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    if declaration.kind == TABLE:
        return torch.randint(0, 2 ** 15, declaration.shape, generator=generator, dtype=torch.int32, device=device)
    values = torch.randn(declaration.shape, generator=generator, dtype=torch.float32, device=device)
    if declaration.kind == NORM:
        return values.mul_(0.1).add_(1.0)
    return values.mul_(0.02)


class RandomSource:
    """Tensor source that makes each tensor when it is asked for (nothing is written to disk)."""

    def __init__(self, spec, seed: int, dtype: torch.dtype, device):
        self.wanted: Dict[str, WeightDecl] = declared_weights(spec)
        self.seed, self.dtype, self.device = seed, dtype, device

    def get(self, name: str) -> torch.Tensor:
        declaration = self.wanted[name]
        tensor = random_tensor(name, declaration, self.seed, self.device)
        return tensor if declaration.kind == TABLE else tensor.to(self.dtype)


def write_model_folder(config, folder: str, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for the typed ``config`` (any registered
    architecture's configuration class).  Values are drawn in float32 on the CPU and stored as ``dtype``."""
    from safetensors.torch import save_file

    from ..config.registry import architecture_of

    raw = config.to_dict()
    spec = architecture_of(raw).build_spec(config)
    tensors = {}
    for name, declaration in declared_weights(spec).items():
        tensor = random_tensor(name, declaration, seed, "cpu")
        tensors[name] = tensor if declaration.kind == TABLE else tensor.to(dtype).contiguous()
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(raw, handle, indent=2)
    save_file(tensors, os.path.join(folder, "model.safetensors"))
    return folder
