"""Sampling: one token per row of logits, greedy or at a temperature.

The reference samples greedily only (``torch.argmax``, utils/engine.py:295-297; README.md:125).
Here one kernel serves both: a row with temperature 0 takes the argmax (lowest index on ties); a row
with temperature T > 0 takes argmax_i(logit_i / T + g_i) with Gumbel noise g_i from a counter-based
generator keyed by (the request's seed, the index of the token being generated, i).  That draws from
softmax(logits / T) and keeps no state, so a request's tokens do not depend on which other requests
share its steps, nor on preemption and recomputation.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

from .. import ops


@dataclass
class SamplingRow:
    temperature: float = 0.0
    seed: int = 0
    step: int = 0     # how many tokens the request has generated before this one


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def __call__(self, logits: torch.Tensor, rows: Sequence[SamplingRow]) -> List[int]:
        """``logits``: float32 [R, V] on the device.  Returns R token ids on the host (the step's one
        device-to-host read)."""
        if logits.shape[0] != len(rows):
            raise ValueError(f"{logits.shape[0]} rows of logits for {len(rows)} requests")
        return self.sample_on_device(logits, rows).tolist()

    def from_batch(self, logits: torch.Tensor, batch) -> torch.Tensor:
        """Samples with the per-row inputs that crossed to the device inside the step's batch; the tokens
        stay on the device (the step function reads them back together with its error flags)."""
        return ops.sample(logits, batch.temperatures, batch.seeds, batch.sample_steps)

    def sample_on_device(self, logits: torch.Tensor, rows: Sequence[SamplingRow]) -> torch.Tensor:
        if any(row.temperature > 0 for row in rows):
            temperatures = torch.tensor([row.temperature for row in rows], dtype=torch.float32)
            seeds = torch.tensor([row.seed & 0x7FFFFFFFFFFFFFFF for row in rows], dtype=torch.int64)
            steps = torch.tensor([row.step for row in rows], dtype=torch.int32)
            return ops.sample(logits, temperatures.to(self.device, non_blocking=True),
                              seeds.to(self.device, non_blocking=True), steps.to(self.device, non_blocking=True))
        return ops.sample(logits)
