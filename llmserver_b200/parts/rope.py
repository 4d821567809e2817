"""Rotary position encoding (NeoX half-split form)."""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import POSITION_ENCODINGS


@POSITION_ENCODINGS.register("rotary")
class RotaryPosition(PositionEncoding):
    """inv_freq[i] = theta ** (-2i / R), i = 0 .. R/2 - 1, built in float32 exactly as the reference does
    (utils/layers.py:147,157) with R = ``rotary_dim``; angle = position * inv_freq is formed in the kernel that
    rotates Q and K.  Parameters: ``head_dim``, ``theta``; optional ``rotary_dim`` (default head_dim: the whole
    head rotates, as in the reference), ``pairing`` ("halves", the reference's NeoX form, or "interleaved") and
    ``attention_factor`` (1: the default schedule; mixers may refuse anything else)."""

    KNOWN_PARAMS = ("head_dim", "theta", "rotary_dim", "pairing", "attention_factor")

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        head_dim, theta = int(params["head_dim"]), float(params["theta"])
        rotary_dim = int(params.get("rotary_dim") or head_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary encoding needs an even rotary_dim of at most head_dim {head_dim}, got {rotary_dim}")
        dim_indices = torch.arange(0, rotary_dim, 2, dtype=torch.long)
        inverse = 1.0 / (theta ** (dim_indices.to(torch.float32) / rotary_dim))
        self.head_dim, self.rotary_dim = head_dim, rotary_dim
        self.pairing = params.get("pairing") or "halves"
        self.attention_factor = float(params.get("attention_factor") or 1.0)
        self.inv_freq = inverse.to(torch.float32).to(runtime.device).contiguous()
