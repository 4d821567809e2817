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


def write_model_folder(config, folder: str, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu",
                       shard_bytes: int = 4 << 30) -> str:
    """Writes ``config.json`` and the weights for the typed ``config`` (any registered architecture's configuration
    class): ``model.safetensors``, or, when the tensors exceed ``shard_bytes``, numbered shards with a
    ``model.safetensors.index.json`` (so a large model never sits in host memory whole).  Values are drawn in float32
    on ``device`` (the CPU by default; a GPU draws other values from the same seed, much faster) and stored as ``dtype``."""
    from safetensors.torch import save_file

    from ..config.registry import architecture_of

    raw = config.to_dict()
    spec = architecture_of(raw).build_spec(config)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(raw, handle, indent=2)
    wanted = declared_weights(spec)
    sizes = {name: int(torch.tensor(declaration.shape).prod()) * (4 if declaration.kind == TABLE else torch.empty(0, dtype=dtype).element_size())
             for name, declaration in wanted.items()}
    shards, current, held = [], [], 0
    for name in wanted:
        if current and held + sizes[name] > shard_bytes:
            shards.append(current)
            current, held = [], 0
        current.append(name)
        held += sizes[name]
    shards.append(current)
    weight_map = {}
    for index, names in enumerate(shards):
        tensors = {}
        for name in names:
            tensor = random_tensor(name, wanted[name], seed, device)
            tensors[name] = (tensor if wanted[name].kind == TABLE else tensor.to(dtype)).cpu().contiguous()
        file_name = "model.safetensors" if len(shards) == 1 else f"model-{index + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(tensors, os.path.join(folder, file_name))
        weight_map.update({name: file_name for name in names})
    if len(shards) > 1:
        with open(os.path.join(folder, "model.safetensors.index.json"), "w") as handle:
            json.dump({"metadata": {"total_size": sum(sizes.values())}, "weight_map": weight_map}, handle)
    return folder
