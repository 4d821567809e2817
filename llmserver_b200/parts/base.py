"""Interfaces of the parts a layer is put together from.

Every part is built from ``(params, weights, runtime)``: ``params`` are its sizes and constants
(the dict form of its ``PartSpec``), ``weights`` the tensors it declared, already on the device,
and ``runtime`` says in which dtype and on which device it runs.  No part knows which model it is in.

    Mixer        forward(x [N, H], batch, cache) -> [N, H_out]   reads/writes its cache view
    FeedForward  forward(x [N, H]) -> [N, H]
    Norm         add_norm(residual f32 [N, H], delta or None, rows=None) -> normed [*, H]
    PositionEncoding   holds what mixers need to encode positions (for rotary: inverse frequencies)
    Block        forward(residual, delta, batch, cache) -> (residual, delta): the arrangement of
                 norms, mixer and feed-forward around the residual stream; ``delta`` is the output of
                 the previous sub-layer that has not been added to the stream yet, so that the add
                 fuses with the next norm.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..weights.declare import WeightDecl


@dataclass
class Runtime:
    dtype: torch.dtype
    device: torch.device


class Part:
    # Names of the parameters the part understands (None: anything goes).  A specification that gives a part a
    # parameter it does not know is refused: a "bias=True" that is silently dropped would compute another model.
    KNOWN_PARAMS = None

    @classmethod
    def check_params(cls, params: dict) -> None:
        """Raises ``ValueError`` for a parameter the part does not know or a value it cannot honour."""
        if cls.KNOWN_PARAMS is not None:
            unknown = sorted(set(params) - set(cls.KNOWN_PARAMS))
            if unknown:
                raise ValueError(f"{cls.__name__} does not know the parameter(s) {', '.join(unknown)} "
                                 f"(it takes: {', '.join(sorted(cls.KNOWN_PARAMS))})")

    @classmethod
    def declare_weights(cls, params: dict) -> Dict[str, WeightDecl]:
        """Local tensor name -> declaration."""
        return {}

    def __init__(self, params: dict, weights: Dict[str, torch.Tensor], runtime: Runtime):
        self.check_params(params)
        self.params, self.runtime = params, runtime


class Mixer(Part):
    # Whether ``forward`` can be captured in a CUDA graph and replayed: it must launch the same kernels whatever the
    # batch holds and read nothing of the batch on the host.  A mixer that walks its rows in Python says False; decode
    # steps of a model that has one run eagerly.
    capturable = True
    # Two optional abilities, with which a step of few rows runs without stand-alone residual-add + norm kernels (see
    # ``ops.stream``).  ``takes_unscaled``: ``forward`` accepts an ``ops.RowScaled`` in place of the normalised rows.
    # ``feeds_stream``: ``forward`` takes a keyword ``sink`` (an ``ops.StreamSink``), may add its result to the sink's
    # stream itself (it then returns None and the sink says ``added``) and otherwise ignores it.  A part that leaves
    # both False is called exactly as before.
    takes_unscaled = False
    feeds_stream = False

    @classmethod
    def cache_need(cls, params: dict):
        """``KVPagesNeed``, ``StateNeed`` or None: what one execution of this mixer keeps per request."""
        return None

    def attach(self, position) -> None:
        """Receives the position encoding the layer names (or None)."""

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    takes_unscaled = False      # as for a mixer
    feeds_stream = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor],
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual += delta (when delta is given), then the normalised stream in the activation type."""
        raise NotImplementedError

    def sink(self, residual: torch.Tensor, consumer):
        """An ``ops.StreamSink`` through which the part in front may add its result to ``residual`` and prepare this
        norm's input for ``consumer`` (the part that reads the norm's output; None: nobody needs it prepared, the
        result is only added), or None when this norm cannot work that way.  A norm that gives out sinks accepts a
        used one as ``delta`` of ``add_norm``, and a keyword ``unscaled`` there (leave the division to the consumer)."""
        return None

    def norm(self, x: torch.Tensor) -> torch.Tensor:
        """Normalises activations that are not the stream (a sub-layer's output, in blocks that do so)."""
        raise NotImplementedError


class PositionEncoding(Part):
    def on_embedding(self, residual: torch.Tensor, batch) -> None:
        """Hook for encodings that act on the embedded tokens (absolute tables); default: nothing."""


class Block(Part):
    """An arrangement of parts around the residual stream.  The class says which parts it arranges: ``roles`` maps
    each role's name to the registry its part comes from ("mixer", "feed_forward" or "norm").  The model builds one
    part per role from the layer's specification and hands them over by name; they become attributes of the block.
    Exactly one role comes from the mixer registry: it is the part that owns the layer's cache."""

    @classmethod
    def roles(cls, params: dict) -> Dict[str, str]:
        return {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    @classmethod
    def prefix_of(cls, params: dict, role: str) -> str:
        """Tensor-name prefix (inside the layer) of the part in ``role``."""
        return params.get(f"{role}_prefix", role + ".")

    @classmethod
    def mixer_role(cls, params: dict) -> str:
        mixers = [role for role, registry in cls.roles(params).items() if registry == "mixer"]
        if len(mixers) != 1:
            raise ValueError(f"{cls.__name__} must arrange exactly one mixer, it names {len(mixers)}")
        return mixers[0]

    def __init__(self, params, parts: Dict[str, Part]):
        self.check_params(params)
        self.params, self.parts = params, dict(parts)
        for role, part in parts.items():
            setattr(self, role, part)

    def entry(self):
        """(norm, consumer): the norm that this block applies to the stream first and the part that reads its output,
        for a block in front that can prepare that norm's input; None when the block does not start that way."""
        return None

    # True: ``forward`` takes a keyword ``after``, the ``entry()`` of what runs next (the next block, or the final
    # norm with no consumer), and may return a used ``ops.StreamSink`` in place of its not yet added output.
    passes_stream = False

    def forward(self, residual, delta, batch, cache):
        raise NotImplementedError


@dataclass
class EntryCache:
    """What one schedule entry sees of the cache manager's storage.

    ``k_pages`` / ``v_pages``: [page, kv_head, slot, head_dim] (None for mixers without pages);
    ``group``: which block table of the batch goes with these pages; ``writes``: False when the
    entry reads the cache another entry wrote; ``state``: [slot, ...] tensor of per-request state."""
    k_pages: Optional[torch.Tensor] = None
    v_pages: Optional[torch.Tensor] = None
    group: int = 0
    writes: bool = True
    state: Optional[torch.Tensor] = None
