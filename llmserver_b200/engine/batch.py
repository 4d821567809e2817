"""The flat token batch of one step.

A step is a list of (request, its next tokens, where logits are wanted).  Portions of prompts and
single decoded tokens lie side by side on one token axis of length N; nothing is padded.  For the
kernels the batch carries, on the device as int32:

    token_ids[N], positions[N] (absolute), seq_of_token[N] (row of the block tables),
    q_start[S + 1] (first token of each sequence on the token axis), context_len[S] (tokens the
    sequence holds after this step), block_tables[group][S, max_blocks], state_slots[S],
    logit_rows[R] (indices into the token axis).

Everything is packed into one pinned host buffer and crosses to the device in a single copy.
The reference builds either a padded [B, T] prefill batch or a [B, 1] decode batch with an additive
mask (utils/batch.py:4-81) and never mixes the two in one forward (utils/engine.py:437-443).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

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


def _align(count: int, to: int = 4) -> int:
    return -(-count // to) * to


def build_batch(slices: List[SequenceSlice], n_groups: int, device, vocab_size: int = None,
                min_table_width: int = 1) -> StepBatch:
    if not slices:
        raise ValueError("a step needs at least one request")
    n_seqs = len(slices)
    tokens: List[int] = []
    positions: List[int] = []
    seq_of_token: List[int] = []
    q_start = [0]
    context_len: List[int] = []
    logit_rows: List[int] = []
    for row, piece in enumerate(slices):
        count = len(piece.tokens)
        if count == 0:
            raise ValueError(f"request {piece.request_id!r} brings no tokens to the step")
        if vocab_size is not None:
            for token in piece.tokens:
                if not 0 <= int(token) < vocab_size:
                    raise ValueError(f"request {piece.request_id!r}: token id {token} is outside the vocabulary of {vocab_size}")
        base = len(tokens)
        tokens.extend(int(t) for t in piece.tokens)
        positions.extend(range(piece.start, piece.start + count))
        seq_of_token.extend([row] * count)
        q_start.append(base + count)
        context_len.append(piece.start + count)
        for place in piece.want:
            if not 0 <= place < count:
                raise ValueError(f"request {piece.request_id!r}: logits wanted at place {place} of {count} tokens")
            logit_rows.append(base + place)
    n_tokens, n_logits = len(tokens), len(logit_rows)
    widths = []
    for group in range(n_groups):
        width = max(min_table_width, max(len(piece.tables[group]) for piece in slices))
        widths.append(width)
    sections = [tokens, positions, seq_of_token, q_start, context_len, [piece.state_slot for piece in slices], logit_rows]
    offsets, total = [], 0
    for section in sections:
        offsets.append(total)
        total += _align(max(len(section), 1))
    table_offsets = []
    for width in widths:
        table_offsets.append(total)
        total += _align(n_seqs * width)
    flag_offset = total
    total += 4
    host = torch.zeros(total, dtype=torch.int32)
    for section, offset in zip(sections, offsets):
        if section:
            host[offset:offset + len(section)] = torch.tensor(section, dtype=torch.int32)
    for group, (width, offset) in enumerate(zip(widths, table_offsets)):
        table = torch.zeros((n_seqs, width), dtype=torch.int32)
        for row, piece in enumerate(slices):
            pages = [page if page >= 0 else 0 for page in piece.tables[group]]  # released pages are never read
            if pages:
                table[row, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        host[offset:offset + n_seqs * width] = table.view(-1)
    if torch.device(device).type == "cuda":
        host = host.pin_memory()
    buffer = host.to(device, non_blocking=True)

    def view(index: int, length: int) -> torch.Tensor:
        return buffer[offsets[index]:offsets[index] + length]

    q_lens = [len(piece.tokens) for piece in slices]
    return StepBatch(
        n_tokens=n_tokens, n_seqs=n_seqs, n_logits=n_logits,
        token_ids=view(0, n_tokens), positions=view(1, n_tokens), seq_of_token=view(2, n_tokens),
        q_start=view(3, n_seqs + 1), context_len=view(4, n_seqs), state_slots=view(5, n_seqs),
        logit_rows=view(6, n_logits),
        block_tables=[buffer[offset:offset + n_seqs * width].view(n_seqs, width)
                      for width, offset in zip(widths, table_offsets)],
        error_flag=buffer[flag_offset:flag_offset + 1],
        q_lens=q_lens, context_lens=context_len, max_q_len=max(q_lens), max_context=max(context_len),
        decode_only=all(length == 1 for length in q_lens), host_bytes=total * 4,
    )
