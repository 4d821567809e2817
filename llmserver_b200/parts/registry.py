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
