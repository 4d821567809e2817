"""The architecture-neutral description of a model: which parts, with which sizes, in which order.

A configuration class (one per architecture) is translated into a ``ModelSpec`` by the
architecture's builder; everything below the builder (weights, cache groups, the generic
decoder, the step function) sees only this description.  Parts are named by registry keys
and carry their sizes and constants as parameters, layer by layer, so one model may use
different mixers and feed-forwards in different layers.  The order in which layers run is a
list (``schedule``): it may name a layer twice, and an entry may read the cache that an
earlier entry wrote instead of keeping its own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its kind (a key of the matching registry in ``llmserver_b200.parts``) and its
    sizes and constants."""
    kind: str
    params: Tuple[Tuple[str, object], ...] = ()

    @staticmethod
    def of(kind: str, **params) -> "PartSpec":
        return PartSpec(kind, tuple(sorted(params.items())))

    def get(self, key, default=None):
        return dict(self.params).get(key, default)

    def as_dict(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges.

    Which parts a block has is the block's business: its class names its *roles* (``Block.roles``), each filled by
    a part of some registry (a mixer, a feed-forward, a norm).  The usual four roles have fields of their own here;
    a block with further roles (more norms, say) finds them in ``extra`` under the role's name.  ``prefix`` is the
    layer's tensor-name prefix in the checkpoint; each part's tensors live under ``prefix + <sub-prefix the block
    gives the role>``."""
    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    position: Optional[str] = None  # key of ModelSpec.positions used by the mixer
    extra: Tuple[Tuple[str, PartSpec], ...] = ()

    def part(self, role: str) -> PartSpec:
        """The part that fills ``role`` in this layer."""
        found = dict(self.extra).get(role)
        if found is None and role in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm"):
            found = getattr(self, role)
        if found is None:
            raise KeyError(f"layer {self.prefix!r}: its block wants a part in the role {role!r}, the layer names none")
        return found


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  ``cache_from`` names an earlier entry (by its index in the
    schedule) whose cache this entry reads; None means the entry keeps a cache of its own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    positions: Dict[str, PartSpec]
    final_norm: PartSpec
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    tie_head: bool = False
    max_positions: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    notes: dict = field(default_factory=dict)

    def validate(self):
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {index} names layer {entry.layer}; the model has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(f"schedule entry {index} reads the cache of entry {entry.cache_from}, which does not run before it")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {index} reads the cache of entry {entry.cache_from}, which has none of its own")
        for layer in self.layers:
            if layer.position is not None and layer.position not in self.positions:
                raise ValueError(f"layer {layer.prefix!r} uses position encoding {layer.position!r}, which the model does not define")
