"""Registries of part kinds.  A model specification names parts by these keys; registering a new
class under a new key is all it takes to make a new mixer, feed-forward, norm, position encoding
or block arrangement available to any architecture (tests register toy parts this way)."""
from __future__ import annotations

from typing import Dict


class PartRegistry:
    def __init__(self, what: str):
        self.what = what
        self.kinds: Dict[str, type] = {}

    def register(self, kind: str, cls: type = None):
        """Usable as ``registry.register("name", Class)`` or as a class decorator."""
        if cls is None:
            def decorate(inner):
                self.kinds[kind] = inner
                return inner
            return decorate
        self.kinds[kind] = cls
        return cls

    def get(self, kind: str) -> type:
        if kind not in self.kinds:
            raise KeyError(f"unknown {self.what} {kind!r} (registered: {', '.join(sorted(self.kinds)) or 'none'})")
        return self.kinds[kind]

    def __contains__(self, kind: str) -> bool:
        return kind in self.kinds


MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
NORMS = PartRegistry("norm")
POSITION_ENCODINGS = PartRegistry("position encoding")
BLOCKS = PartRegistry("block")

REGISTRIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}


def parts_of_layer(layer):
    """What a layer is made of, as its block says: a list of (role, part specification, part class, tensor-name
    prefix).  The model builder and the weight declarations both go by this list."""
    block_cls = BLOCKS.get(layer.block.kind)
    block_params = layer.block.as_dict()
    block_cls.check_params(block_params)
    found = []
    for role, registry in block_cls.roles(block_params).items():
        if registry not in REGISTRIES:
            raise KeyError(f"block {layer.block.kind!r}: role {role!r} names the unknown registry {registry!r}")
        spec = layer.part(role)
        REGISTRIES[registry].get(spec.kind).check_params(spec.as_dict())
        found.append((role, spec, REGISTRIES[registry].get(spec.kind), layer.prefix + block_cls.prefix_of(block_params, role)))
    return found
