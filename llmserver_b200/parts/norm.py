"""RMSNorm over the residual stream."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.declare import NORM, WeightDecl
from .base import Norm
from .registry import NORMS


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y = weight * x / sqrt(mean(x^2) + eps) (utils/layers.py:123-138): weight multiplies, it is not
    (1 + weight); no bias.  Parameters: ``width``, ``eps``.  Fused with the residual add that precedes
    it, as the reference's add_rms_norm (utils/fused_ops.py:145-155)."""

    KNOWN_PARAMS = ("width", "eps")

    @classmethod
    def declare_weights(cls, params):
        return {"weight": WeightDecl((params["width"],), NORM)}

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.weight = weights["weight"].contiguous()
        self.eps = float(params["eps"])

    def add_norm(self, residual, delta, rows=None, unscaled=False):
        if isinstance(delta, ops.StreamSink):
            # the part in front added its result to the stream itself and, if asked, prepared this norm's input
            if delta.owner is not self or not delta.added:
                raise RuntimeError("a stream sink reached a norm that did not make it, or was never used")
            if delta.scaled is not None and rows is None:
                return delta.scaled
            delta = None
        unscaled = unscaled and rows is None and self._few_rows(residual)
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, rows=rows, act_dtype=self.runtime.dtype,
                               unscaled=unscaled)

    def _few_rows(self, residual) -> bool:
        return self.runtime.dtype == torch.bfloat16 and residual.shape[0] <= ops.STREAM_ROWS

    def sink(self, residual, consumer):
        if not self._few_rows(residual) or (consumer is not None and not getattr(consumer, "takes_unscaled", False)):
            return None
        if consumer is None:
            return ops.StreamSink(residual, owner=self)
        return ops.StreamSink(residual, self.weight, self.eps, owner=self)

    def norm(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)
