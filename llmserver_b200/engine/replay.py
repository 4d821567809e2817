"""Trace replay: feeds given token ids through the engine step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same model,
step function, cache manager and kernels that generation uses.  ``bin/trace_run`` is its command line.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Iterable, TextIO

import numpy as np
import torch

from ..cache import CacheManager
from ..models import load_model
from .step import StepFunction

ROUND_TO = 64   # each live request's token count is rounded up to this for the pool size


class TraceReplayer:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, device: str = "cuda:0",
                 max_live: int = 4):
        self.model = load_model(model_dir, dtype, device)
        if ROUND_TO % page_size:
            raise ValueError(f"page_size {page_size} must divide {ROUND_TO}")
        num_pages = max(1, -(-max_tokens // page_size))
        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, num_slots=max_live,
                                  prefix_sharing=False)
        self.cache.materialize(self.model.runtime.device, self.model.runtime.dtype)
        self.step_function = StepFunction(self.model, self.cache)
        self.live = set()

    def run_step(self, record: dict):
        """Runs one trace record; returns the logits as a float32 array [wanted, vocab] or None."""
        entries = []
        for entry in record.get("entries", []):
            request_id = entry["id"]
            if request_id not in self.live:
                self.step_function.admit(request_id)
                self.live.add(request_id)
            entries.append((request_id, entry["tokens"], entry.get("want", [])))
        logits = None
        if entries:
            result = self.step_function.run(entries)
            if result.shape[0]:
                logits = result.to("cpu", torch.float32).numpy()
            self.step_function.check_errors()
        for request_id in record.get("end", []):
            if request_id in self.live:
                self.step_function.release(request_id)
                self.live.discard(request_id)
        return logits


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines: Iterable[str], done: TextIO = sys.stdout,
           page_size: int = 16) -> int:
    os.makedirs(out_dir, exist_ok=True)
    replayer = TraceReplayer(model_dir, dtype, max_tokens, page_size)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = replayer.run_step(record)
        if logits is not None:
            np.ascontiguousarray(logits, dtype="<f4").tofile(os.path.join(out_dir, f"{record['step']}.f32"))
        done.write(f"done {record['step']}\n")
        done.flush()
    return 0
