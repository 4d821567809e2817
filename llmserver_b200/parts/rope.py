"""Rotary position encoding (NeoX half-split form)."""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import POSITION_ENCODINGS


@POSITION_ENCODINGS.register("rotary")
class RotaryPosition(PositionEncoding):
    """inv_freq[i] = theta ** (-2i / D), i = 0 .. D/2 - 1, built in float32 exactly as the reference does
    (utils/layers.py:147,157); angle = position * inv_freq is formed in the kernel that rotates Q and
    K.  Parameters: ``head_dim``, ``theta``.  Attention factor 1 (default schedule)."""

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        head_dim, theta = int(params["head_dim"]), float(params["theta"])
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {head_dim}")
        dim_indices = torch.arange(0, head_dim, 2, dtype=torch.long)
        inverse = 1.0 / (theta ** (dim_indices.to(torch.float32) / head_dim))
        self.head_dim = head_dim
        self.inv_freq = inverse.to(torch.float32).to(runtime.device).contiguous()
