"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream."""
from __future__ import annotations

from .base import Block
from .registry import BLOCKS


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """h += mixer(norm1(h)); h += feed_forward(norm2(h))  (utils/model.py:16-35).

    Each add is fused with the norm that follows it, as the reference's fused dataflow does
    (utils/model.py:87-96): the block receives the stream and the previous sub-layer's output that has
    not been added yet, and returns the stream and its feed-forward's output, still to be added.
    Parameters: the tensor-name prefixes of its four parts (``mixer_prefix`` ...)."""

    KNOWN_PARAMS = ("mixer_prefix", "feed_forward_prefix", "mixer_norm_prefix", "feed_forward_norm_prefix")

    def forward(self, residual, delta, batch, cache):
        normed = self.mixer_norm.add_norm(residual, delta)
        mixed = self.mixer.forward(normed, batch, cache)
        normed = self.feed_forward_norm.add_norm(residual, mixed)
        return residual, self.feed_forward.forward(normed)
