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

    passes_stream = True

    def entry(self):
        return self.mixer_norm, self.mixer

    def forward(self, residual, delta, batch, cache, after=None):
        # With few rows, parts that can do so add their results to the stream themselves and prepare the next norm's
        # input (``sink``), and take a norm's output before its division (``unscaled``); see ``ops.stream``.  Parts
        # and norms that cannot are called as ever.
        normed = _add_norm(self.mixer_norm, residual, delta, self.mixer)
        sink = self.feed_forward_norm.sink(residual, self.feed_forward) if self.mixer.feeds_stream else None
        mixed = self.mixer.forward(normed, batch, cache, sink=sink) if sink is not None else self.mixer.forward(normed, batch, cache)
        normed = _add_norm(self.feed_forward_norm, residual, sink if sink is not None and sink.added else mixed, self.feed_forward)
        sink = after[0].sink(residual, after[1]) if after is not None and self.feed_forward.feeds_stream else None
        out = self.feed_forward.forward(normed, sink=sink) if sink is not None else self.feed_forward.forward(normed)
        return residual, (sink if sink is not None and sink.added else out)


def _add_norm(norm, residual, delta, consumer):
    if getattr(consumer, "takes_unscaled", False) and norm.sink(residual, consumer) is not None:
        return norm.add_norm(residual, delta, unscaled=True)
    return norm.add_norm(residual, delta)
