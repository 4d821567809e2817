"""Loads a model's tensors by name, checks them against what the specification declares, and
hands them out in the model's dtype.

Dtypes: matrices are kept in the compute dtype asked for (bfloat16 for serving, float32 for the
32-bit path); a small tensor (a norm weight, say) that the checkpoint stores in 32-bit stays 32-bit,
the kernels read it as such; integer tables become int32.  One ``WeightLoadError`` lists every missing tensor, every
unexpected tensor and every wrong shape or dtype family; nothing is loaded partially.

The reference loads module by module with ``load_state_dict(strict=True)`` (utils/model_loader.py:49-52),
which reports one module's mismatch at a time, and ties the head when the config says so or the
checkpoint has no ``lm_head.weight`` (utils/model_loader.py:56-59).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.errors import WeightLoadError
from .declare import MATRIX, TABLE, WeightDecl, declared_weights
from .reader import CheckpointReader

_FLOAT_FAMILY = {"F64", "F32", "F16", "BF16"}
_INT_FAMILY = {"I64", "I32", "I16", "I8", "U8"}


def check_checkpoint(reader: CheckpointReader, wanted: Dict[str, WeightDecl], optional=()) -> None:
    missing, unexpected, wrong = [], [], []
    present = set(reader.names())
    for name, declaration in sorted(wanted.items()):
        if name not in present:
            missing.append(name)
            continue
        shape, dtype = reader.shape_and_dtype(name)
        if tuple(shape) != tuple(declaration.shape):
            wrong.append(f"{name}: shape {list(shape)} where {list(declaration.shape)} is expected")
        family = _INT_FAMILY if declaration.kind == TABLE else _FLOAT_FAMILY
        if dtype.upper() not in family:
            wrong.append(f"{name}: dtype {dtype} where {'an integer' if declaration.kind == TABLE else 'a floating'} type is expected")
    for name in sorted(present - set(wanted) - set(optional)):
        unexpected.append(name)
    if missing or unexpected or wrong:
        lines = [f"model.safetensors in {reader.folder!r} does not match the configuration:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        raise WeightLoadError("\n".join(lines))


class CheckpointSource:
    """Tensor source backed by a model folder."""

    def __init__(self, folder: str, spec, dtype: torch.dtype, device):
        self.reader = CheckpointReader(folder)
        self.dtype, self.device = dtype, device
        wanted = declared_weights(spec)
        optional = set()
        if spec.tie_head:
            # a tied checkpoint may still carry a copy of the head; it is not read
            optional.add(spec.head_name)
        elif not self.reader.has(spec.head_name):
            # no head in the checkpoint means tied (utils/model_loader.py:56)
            spec.tie_head = True
            wanted.pop(spec.head_name, None)
        check_checkpoint(self.reader, wanted, optional)
        self.wanted = wanted

    def get(self, name: str) -> torch.Tensor:
        declaration = self.wanted[name]
        tensor = self.reader.get(name)
        if declaration.kind == TABLE:
            return tensor.to(torch.int32).to(self.device)
        if declaration.kind != MATRIX and tensor.dtype == torch.float32:
            return tensor.to(self.device)  # a small tensor stored in 32-bit is not narrowed
        return tensor.to(self.dtype).to(self.device)
