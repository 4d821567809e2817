"""The flat token batch of one step.

A step is a list of (request, its next tokens, where logits are wanted).  Portions of prompts and
single decoded tokens lie side by side on one token axis of length N; nothing is padded.  For the
kernels the batch carries, on the device as int32:

    token_ids[N], positions[N] (absolute), seq_of_token[N] (row of the block tables),
    q_start[S + 1] (first token of each sequence on the token axis), context_len[S] (tokens the
    sequence holds after this step), block_tables[group][S, width], state_slots[S],
    logit_rows[R] (indices into the token axis),
    and per wanted row the sampling inputs: temperatures[R] (float32), seeds[R] (int64), sample_steps[R].

Everything is packed into ONE pinned host buffer and crosses to the device in a single copy; the
``BatchLayout`` says where each section lies.  A layout depends only on (N, S, R, table widths), so a
decode step of a given batch size always has the same layout: that is what lets a CUDA graph replay it
from a fixed device buffer.

The reference builds either a padded [B, T] prefill batch or a [B, 1] decode batch with an additive
mask (utils/batch.py:4-81) and never mixes the two in one forward (utils/engine.py:437-443).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class SequenceSlice:
    """One request's share of a step."""
    request_id: object
    tokens: Sequence[int]
    start: int                       # tokens of this request already in the cache
    want: Sequence[int] = ()         # places among ``tokens`` whose logits are asked for
    tables: Sequence[Sequence[int]] = ()   # one block table per cache group
    state_slot: int = 0


def _align(count: int, to: int = 4) -> int:
    return -(-max(count, 1) // to) * to


@dataclass(frozen=True)
class BatchLayout:
    """Offsets (in int32 words) of the sections of the packed buffer."""
    n_tokens: int
    n_seqs: int
    n_logits: int
    widths: Tuple[int, ...]

    def __post_init__(self):
        offsets, total = {}, 0
        for name, count in (("token_ids", self.n_tokens), ("positions", self.n_tokens), ("seq_of_token", self.n_tokens),
                            ("q_start", self.n_seqs + 1), ("context_len", self.n_seqs), ("state_slots", self.n_seqs),
                            ("logit_rows", self.n_logits), ("temperatures", self.n_logits), ("seeds", 2 * self.n_logits),
                            ("sample_steps", self.n_logits), ("error_flag", 1)):
            offsets[name] = total
            total += _align(count)
        tables = []
        for width in self.widths:
            tables.append(total)
            total += _align(self.n_seqs * width)
        object.__setattr__(self, "offsets", offsets)
        object.__setattr__(self, "table_offsets", tuple(tables))
        object.__setattr__(self, "total", total)


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    n_logits: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    q_start: torch.Tensor
    context_len: torch.Tensor
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    temperatures: torch.Tensor
    seeds: torch.Tensor
    sample_steps: torch.Tensor
    block_tables: List[torch.Tensor]
    error_flag: torch.Tensor
    # host-side copies that kernels' launch logic needs
    q_lens: List[int] = field(default_factory=list)
    context_lens: List[int] = field(default_factory=list)
    max_q_len: int = 0
    max_context: int = 0
    decode_only: bool = False
    host_bytes: int = 0
    scratch: dict = field(default_factory=dict)   # per-step data kernels' wrappers derive once
    # A request's tokens before this step's were cached by earlier steps, and this step begins with the copy of its
    # batch to the device, behind which those steps are complete: kernels may read such keys without waiting for the
    # kernel launched just before them.  True for every batch packed here; a hand-made batch that fills the cache and
    # reads it in the same breath must say False.
    keys_settled: bool = True


def layout_of(slices: List[SequenceSlice], n_groups: int, min_table_width: int = 1) -> BatchLayout:
    n_tokens = sum(len(piece.tokens) for piece in slices)
    n_logits = sum(len(piece.want) for piece in slices)
    widths = tuple(max(min_table_width, max(len(piece.tables[group]) for piece in slices)) for group in range(n_groups))
    return BatchLayout(n_tokens, len(slices), n_logits, widths)


def pack(slices: List[SequenceSlice], layout: BatchLayout, host: np.ndarray, vocab_size: Optional[int] = None,
         sampling: Optional[Sequence] = None) -> None:
    """Fills ``host`` (int32 [layout.total]) with the step.  ``sampling``: per wanted row, in order, an
    object with ``temperature``, ``seed`` and ``step`` (absent: greedy)."""
    if not slices:
        raise ValueError("a step needs at least one request")
    off = layout.offsets
    host[:] = 0
    at, row_at = 0, 0
    q_start = [0]
    for row, piece in enumerate(slices):
        count = len(piece.tokens)
        if count == 0:
            raise ValueError(f"request {piece.request_id!r} brings no tokens to the step")
        tokens = np.asarray(piece.tokens, dtype=np.int64)
        if vocab_size is not None and (tokens.min() < 0 or tokens.max() >= vocab_size):
            raise ValueError(f"request {piece.request_id!r}: a token id is outside the vocabulary of {vocab_size}")
        host[off["token_ids"] + at:off["token_ids"] + at + count] = tokens
        host[off["positions"] + at:off["positions"] + at + count] = np.arange(piece.start, piece.start + count)
        host[off["seq_of_token"] + at:off["seq_of_token"] + at + count] = row
        host[off["context_len"] + row] = piece.start + count
        host[off["state_slots"] + row] = piece.state_slot
        for place in piece.want:
            if not 0 <= place < count:
                raise ValueError(f"request {piece.request_id!r}: logits wanted at place {place} of {count} tokens")
            host[off["logit_rows"] + row_at] = at + place
            row_at += 1
        at += count
        q_start.append(at)
        for group, (width, table_offset) in enumerate(zip(layout.widths, layout.table_offsets)):
            pages = np.asarray(piece.tables[group], dtype=np.int32)
            if pages.size > width:
                raise ValueError(f"request {piece.request_id!r} holds {pages.size} pages; the batch has room for {width}")
            begin = table_offset + row * width
            # pages a window has given back (negative entries) become page 0 on the device: the attention kernels
            # still load the tile such an entry lies in when the window starts inside it, and mask those keys
            host[begin:begin + pages.size] = np.maximum(pages, 0)
    host[off["q_start"]:off["q_start"] + len(q_start)] = q_start
    if sampling is not None:
        if len(sampling) != layout.n_logits:
            raise ValueError(f"{len(sampling)} sampling rows for {layout.n_logits} wanted logits")
        if layout.n_logits:
            host[off["temperatures"]:off["temperatures"] + layout.n_logits] = np.asarray(
                [row.temperature for row in sampling], dtype=np.float32).view(np.int32)
            host[off["seeds"]:off["seeds"] + 2 * layout.n_logits] = np.asarray(
                [row.seed & 0x7FFFFFFFFFFFFFFF for row in sampling], dtype=np.int64).view(np.int32)
            host[off["sample_steps"]:off["sample_steps"] + layout.n_logits] = [row.step for row in sampling]


def views(buffer: torch.Tensor, layout: BatchLayout, slices: List[SequenceSlice]) -> StepBatch:
    """A StepBatch whose tensors are views of the device copy of the packed buffer."""
    off = layout.offsets

    def section(name: str, length: int) -> torch.Tensor:
        return buffer[off[name]:off[name] + length]

    n, s, r = layout.n_tokens, layout.n_seqs, layout.n_logits
    q_lens = [len(piece.tokens) for piece in slices]
    context_lens = [piece.start + len(piece.tokens) for piece in slices]
    return StepBatch(
        n_tokens=n, n_seqs=s, n_logits=r,
        token_ids=section("token_ids", n), positions=section("positions", n), seq_of_token=section("seq_of_token", n),
        q_start=section("q_start", s + 1), context_len=section("context_len", s), state_slots=section("state_slots", s),
        logit_rows=section("logit_rows", r), temperatures=section("temperatures", r).view(torch.float32),
        seeds=section("seeds", 2 * r).view(torch.int64), sample_steps=section("sample_steps", r),
        block_tables=[buffer[offset:offset + s * width].view(s, width)
                      for width, offset in zip(layout.widths, layout.table_offsets)],
        error_flag=section("error_flag", 1),
        q_lens=q_lens, context_lens=context_lens, max_q_len=max(q_lens), max_context=max(context_lens),
        decode_only=all(length == 1 for length in q_lens), host_bytes=layout.total * 4,
    )


def build_batch(slices: List[SequenceSlice], n_groups: int, device, vocab_size: Optional[int] = None,
                min_table_width: int = 1, sampling: Optional[Sequence] = None) -> StepBatch:
    """Packs the step on the host (pinned when the device is a GPU) and copies it over in one go."""
    if not slices:
        raise ValueError("a step needs at least one request")
    layout = layout_of(slices, n_groups, min_table_width)
    on_gpu = torch.device(device).type == "cuda"
    host = torch.empty(layout.total, dtype=torch.int32, pin_memory=on_gpu)
    pack(slices, layout, host.numpy(), vocab_size, sampling)
    return views(host.to(device, non_blocking=True), layout, slices)
