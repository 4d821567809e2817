"""SwiGLU feed-forward."""
from __future__ import annotations

import functools

import torch

from .. import ops
from ..weights.declare import WeightDecl
from .base import FeedForward
from .registry import FEED_FORWARDS


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)) without biases (utils/layers.py:182-218).  gate and up are
    concatenated once at load into one [2 I, H] matrix, gate rows first, as the reference's
    ``fuse_projections`` (utils/layers.py:194-203).  Parameters: ``hidden``, ``intermediate``; ``bias`` must be off
    and ``activation``, if given, "silu"."""

    KNOWN_PARAMS = ("hidden", "intermediate", "bias", "activation")

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        if params.get("bias"):
            raise ValueError("swiglu has no biases (bias must be absent or false)")
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"swiglu gates with SiLU, not {params['activation']!r}")

    @classmethod
    def declare_weights(cls, params):
        hidden, intermediate = params["hidden"], params["intermediate"]
        return {"gate_proj.weight": WeightDecl((intermediate, hidden)),
                "up_proj.weight": WeightDecl((intermediate, hidden)),
                "down_proj.weight": WeightDecl((hidden, intermediate))}

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        gate, up = weights["gate_proj.weight"], weights["up_proj.weight"]
        # bfloat16: gate and up rows interleaved in groups of 64, the layout in which the product kernel for few rows
        # can apply the gate itself; the 32-bit path keeps gate rows first
        self.group = ops.GATE_UP_GROUP if gate.dtype == torch.bfloat16 and gate.shape[0] % ops.GATE_UP_GROUP == 0 else 0
        self.gate_up = ops.interleave_gate_up(gate, up) if self.group else torch.cat([gate, up], dim=0).contiguous()
        self.down = weights["down_proj.weight"].contiguous()

    feeds_stream = True

    @functools.cached_property
    def takes_unscaled(self):
        return ops.unscaled_rows_supported(self.gate_up)

    def forward(self, x, sink=None):
        return ops.linear(ops.gate_up_silu(x, self.gate_up, self.group), self.down, sink=sink)
