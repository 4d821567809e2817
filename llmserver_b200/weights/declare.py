"""What tensors a model needs: collected from the parts its specification names."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

MATRIX = "matrix"   # random mode: N(0, 0.02)
NORM = "norm"       # random mode: 1 + N(0, 0.1)
TABLE = "table"     # integer table (kept as int32)


@dataclass(frozen=True)
class WeightDecl:
    shape: Tuple[int, ...]
    kind: str = MATRIX


def declared_weights(spec) -> Dict[str, WeightDecl]:
    """Full tensor name -> declaration, for every tensor the model reads from a checkpoint."""
    from ..parts import registry as parts

    wanted: Dict[str, WeightDecl] = {spec.embedding_name: WeightDecl((spec.vocab_size, spec.hidden_size))}
    for layer in spec.layers:
        for _, part_spec, part_cls, prefix in parts.parts_of_layer(layer):
            for local, declaration in part_cls.declare_weights(part_spec.as_dict()).items():
                wanted[prefix + local] = declaration
    for local, declaration in parts.NORMS.get(spec.final_norm.kind).declare_weights(spec.final_norm.as_dict()).items():
        wanted[spec.final_norm_prefix + local] = declaration
    for name, position in spec.positions.items():
        for local, declaration in parts.POSITION_ENCODINGS.get(position.kind).declare_weights(position.as_dict()).items():
            wanted[f"model.positions.{name}.{local}"] = declaration
    if not spec.tie_head:
        wanted[spec.head_name] = WeightDecl((spec.vocab_size, spec.hidden_size))
    return wanted
