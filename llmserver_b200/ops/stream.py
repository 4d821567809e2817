"""Two small types with which a step of few rows does without stand-alone residual-add + RMSNorm kernels.

A product whose result belongs on the residual stream adds it there in its own epilogue (``StreamSink``) and leaves,
for the RMSNorm that follows, the stream times the norm's weight (bfloat16) and partial sums of squares of the
updated rows (``RowScaled``).  The product that consumes the norm's output multiplies its 32-bit accumulators row by
row with 1 / rms: W (s w x) = s W (w x) for one scalar s per row.  Statistics, scale and the residual sum stay 32-bit;
only the place where bfloat16 rounding happens moves (before the division instead of after it).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

# Up to this many rows a step runs this way: 16, the rows up to which this package's product kernel is always used
# (LLMSERVER_B200_STREAM_ROWS changes it, up to the kernel's 64 rows; beyond 16 rows the library's products win most
# measurements and the stand-alone kernels run beside them).  LLMSERVER_B200_STREAM_EPILOGUES=0 switches it off: the
# stand-alone add + norm kernel then runs at every row count.
STREAM_ROWS = (min(max(int(os.environ.get("LLMSERVER_B200_STREAM_ROWS", "16")), 0), 64)
               if os.environ.get("LLMSERVER_B200_STREAM_EPILOGUES", "1") != "0" else 0)
NO_SCALE = (0, 0, 0, 0.0)


class RowScaled:
    """``x`` [N, H] bfloat16 = stream * norm weight; ``parts`` float32 [n_parts, >= N]: the sum over i of parts[i, n] is
    the sum of squares of stream row n.  Stands for x[n] / sqrt(sum / H + eps)."""

    __slots__ = ("x", "parts", "eps")

    def __init__(self, x: torch.Tensor, parts: torch.Tensor, eps: float):
        self.x, self.parts, self.eps = x, parts, float(eps)

    @property
    def shape(self):
        return self.x.shape

    @property
    def dtype(self):
        return self.x.dtype

    @property
    def device(self):
        return self.x.device

    def scale_args(self) -> tuple:
        """(parts pointer, number of parts, row capacity, eps) as the launchers take them."""
        return self.parts.data_ptr(), self.parts.shape[0], self.parts.shape[1], self.eps


def scale_args_of(x) -> tuple:
    return x.scale_args() if isinstance(x, RowScaled) else NO_SCALE


def rows_of(x) -> torch.Tensor:
    return x.x if isinstance(x, RowScaled) else x


class StreamSink:
    """Where a product may add its result: the 32-bit stream ``residual`` [N, H].  With ``norm_weight`` (and ``eps``)
    the product also prepares the input of the RMSNorm that follows (``scaled``, a ``RowScaled``).  ``owner`` is
    whoever made the sink (the norm it prepares for); ``added`` says whether a product took it."""

    __slots__ = ("residual", "norm_weight", "eps", "owner", "added", "scaled")

    def __init__(self, residual: torch.Tensor, norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, owner=None):
        self.residual, self.norm_weight, self.eps, self.owner = residual, norm_weight, float(eps), owner
        self.added = False
        self.scaled: Optional[RowScaled] = None
