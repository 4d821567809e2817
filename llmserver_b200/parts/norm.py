"""RMSNorm over the residual stream."""
from __future__ import annotations

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

    def add_norm(self, residual, delta, rows=None):
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, rows=rows, act_dtype=self.runtime.dtype)

    def norm(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)
