"""The cache manager: paged keys and values per group of layers, block tables per request, and
slots of fixed-size per-request state.

What a mixer needs is declared by its class (``KVPagesNeed`` or ``StateNeed``); the manager knows
nothing about models.  Schedule entries with the same page shape and the same window form one
*group* with a page pool, a storage tensor and per-request block tables of its own, so a group
that keeps every key and a group that keeps only a window can grow and shrink independently.
Pages are given back when a request ends and, in windowed groups, as soon as the window has
passed them; they are reused by later allocations.

The reference has one cache shape for all layers (utils/engine.py:77-85, utils/kv_cache.py:84-89)
and no per-request state in its paged path; groups and state slots are this engine's own.  Storage
layout per group: [entry, k|v, page, kv_head, slot, head_dim].
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from .pool import KVCacheExhaustedError, KVCacheStateError, PagePool

RELEASED = -1  # block-table entry of a page the window has passed


@dataclass(frozen=True)
class KVPagesNeed:
    """Keys and values of ``kv_heads`` heads of ``head_dim``; ``window`` None keeps all tokens,
    else only the last ``window`` tokens are ever read."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A tensor of fixed ``shape`` per request (zeroed when the request is admitted)."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


class CacheGroup:
    def __init__(self, index: int, need: KVPagesNeed, entries: List[int], num_pages: int, page_size: int):
        self.index = index
        self.need = need
        self.entries = entries            # schedule entries that own a cache in this group
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.tables: Dict[object, List[int]] = {}
        self.released_upto: Dict[object, int] = {}   # per request: pages [0, n) were given back
        self.storage = None               # torch tensor once materialised

    @property
    def window(self) -> Optional[int]:
        return self.need.window

    def pages_for(self, request_id, total_tokens: int) -> int:
        """Pages to allocate so that positions < total_tokens have a slot."""
        table = self.tables[request_id]
        return max(0, -(-total_tokens // self.page_size) - len(table))

    def passed_pages(self, num_computed: int) -> int:
        """Number of leading pages no later query can read when ``num_computed`` tokens are done."""
        if self.window is None:
            return 0
        first_needed = num_computed - self.window + 1  # earliest key of the query at position num_computed
        return max(0, first_needed // self.page_size)


class StateSlots:
    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self.free: List[int] = list(range(num_slots - 1, -1, -1))
        self.slot_of: Dict[object, int] = {}
        self.storage: Dict[int, object] = {}    # schedule entry -> tensor [num_slots, *shape]

    def take(self, request_id) -> int:
        if request_id in self.slot_of:
            raise KVCacheStateError(f"request {request_id!r} already holds a state slot")
        if not self.free:
            raise KVCacheExhaustedError("no state slot is free")
        slot = self.free.pop()
        self.slot_of[request_id] = slot
        for tensor in self.storage.values():
            tensor[slot].zero_()
        return slot

    def give_back(self, request_id) -> None:
        slot = self.slot_of.pop(request_id, None)
        if slot is None:
            raise KVCacheStateError(f"request {request_id!r} holds no state slot")
        self.free.append(slot)


class CacheManager:
    """``needs[i]`` is what schedule entry i keeps for itself: a ``KVPagesNeed``, a ``StateNeed`` or
    None (nothing, or it reads another entry's cache)."""

    def __init__(self, needs: Sequence[object], page_size: int, num_pages: int, num_slots: int = 64,
                 prefix_sharing: bool = True, model_identity: str = "model"):
        if page_size <= 0:
            raise ValueError(f"page_size must be positive: {page_size}")
        self.page_size = page_size
        self.groups: List[CacheGroup] = []
        self.group_of_entry: Dict[int, Tuple[int, int]] = {}  # entry -> (group index, index inside the group)
        self.state_entries: Dict[int, StateNeed] = {}
        by_need: Dict[KVPagesNeed, CacheGroup] = {}
        for entry, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, StateNeed):
                self.state_entries[entry] = need
            elif isinstance(need, KVPagesNeed):
                group = by_need.get(need)
                if group is None:
                    group = CacheGroup(len(self.groups), need, [], num_pages, page_size)
                    by_need[need] = group
                    self.groups.append(group)
                self.group_of_entry[entry] = (group.index, len(group.entries))
                group.entries.append(entry)
            else:
                raise TypeError(f"schedule entry {entry}: unknown cache need {need!r}")
        self.slots = StateSlots(num_slots)
        self.requests: Dict[object, int] = {}   # request -> tokens that have a slot in every group
        self.has_windows = any(group.window is not None for group in self.groups)
        # A prefix can be skipped only if every layer's cache of it is at hand.  Groups that keep every key qualify:
        # what their pages hold is a function of the prefix alone, and each keeps a digest chain of its own.  A
        # windowed group gives pages back and per-request state is not kept in pages at all, so a model with
        # either recomputes its prompts.
        only_full = not self.has_windows and not self.state_entries
        self.prefix_sharing = bool(prefix_sharing and only_full and self.groups)
        self.model_identity = model_identity
        self.device = None
        self.dtype = None

    # ------------------------------------------------------------------ storage
    def materialize(self, device, dtype) -> None:
        """Allocates the device tensors (pages zero-initialised as utils/kv_cache.py:87-89)."""
        import torch

        self.device, self.dtype = device, dtype
        for group in self.groups:
            need = group.need
            group.storage = torch.zeros((len(group.entries), 2, group.pool.num_pages, need.kv_heads, self.page_size,
                                         need.head_dim), dtype=dtype, device=device)
        for entry, need in self.state_entries.items():
            self.slots.storage[entry] = torch.zeros((self.slots.num_slots,) + tuple(need.shape),
                                                    dtype=getattr(torch, need.dtype), device=device)

    def pages_of_entry(self, entry: int):
        """(k_pages, v_pages, group index) of the schedule entry that owns a paged cache."""
        group_index, inside = self.group_of_entry[entry]
        storage = self.groups[group_index].storage
        return storage[inside, 0], storage[inside, 1], group_index

    def state_of_entry(self, entry: int):
        return self.slots.storage[entry]

    def storage_bytes(self) -> int:
        total = 0
        for group in self.groups:
            if group.storage is not None:
                total += group.storage.numel() * group.storage.element_size()
        return total

    # ------------------------------------------------------------------ requests
    def admit(self, request_id) -> int:
        """Registers a request: empty block tables in every group and a zeroed state slot."""
        if request_id in self.requests:
            raise KVCacheStateError(f"request {request_id!r} is already admitted")
        slot = self.slots.take(request_id)
        self.requests[request_id] = 0
        for group in self.groups:
            group.tables[request_id] = []
            group.released_upto[request_id] = 0
        return slot

    def is_admitted(self, request_id) -> bool:
        return request_id in self.requests

    def slot_of(self, request_id) -> int:
        return self.slots.slot_of[request_id]

    def table(self, request_id, group: int = 0) -> List[int]:
        return self.groups[group].tables[request_id]

    def pages_needed(self, request_id, total_tokens: int) -> List[int]:
        """Per group, the pages that ``ensure(request_id, total_tokens)`` would allocate."""
        if request_id not in self.requests:
            return [-(-total_tokens // self.page_size) for _ in self.groups]
        return [group.pages_for(request_id, total_tokens) for group in self.groups]

    def reserve_null_pages(self) -> List[int]:
        """Sets one page per group aside for good and returns their ids: rows that only pad a batch to a
        fixed size point there, so what they write and read touches no request's pages."""
        for group in self.groups:
            if getattr(group, "null_page", None) is None:
                group.null_page = group.pool.allocate()
        return [group.null_page for group in self.groups]

    def capacity(self) -> List[int]:
        """Pages per group that requests can hold (the pool minus a page set aside for padding rows)."""
        return [group.pool.num_pages - (1 if getattr(group, "null_page", None) is not None else 0) for group in self.groups]

    def has_room(self, request_id, total_tokens: int) -> bool:
        """True when positions < total_tokens already have a slot in every group (no page to allocate)."""
        limit = total_tokens
        for group in self.groups:
            if len(group.tables[request_id]) * self.page_size < limit:
                return False
        return True

    def available(self) -> List[int]:
        return [group.pool.num_available for group in self.groups]

    def ensure(self, request_id, total_tokens: int) -> None:
        """Gives positions < total_tokens a slot in every group, or raises ``KVCacheExhaustedError``
        and allocates nothing."""
        if request_id not in self.requests:
            raise KVCacheStateError(f"request {request_id!r} is not admitted")
        needed = self.pages_needed(request_id, total_tokens)
        for group, count in zip(self.groups, needed):
            if count > group.pool.num_available:
                raise KVCacheExhaustedError(
                    f"request {request_id!r} needs {count} pages in cache group {group.index}, {group.pool.num_available} are available")
        for group, count in zip(self.groups, needed):
            table = group.tables[request_id]
            for _ in range(count):
                table.append(group.pool.allocate())
        self.requests[request_id] = max(self.requests[request_id], total_tokens)

    def advance(self, request_id, num_computed: int) -> int:
        """Called after a step: gives back the pages of windowed groups that no later query of this
        request can read.  Returns how many pages were released."""
        if not self.has_windows:
            return 0
        released = 0
        for group in self.groups:
            upto = min(group.passed_pages(num_computed), len(group.tables[request_id]))
            table = group.tables[request_id]
            for index in range(group.released_upto[request_id], upto):
                if table[index] != RELEASED:
                    group.pool.release(table[index])
                    table[index] = RELEASED
                    released += 1
            group.released_upto[request_id] = max(group.released_upto[request_id], upto)
        return released

    def free(self, request_id) -> None:
        """Gives back everything the request holds.  The tables are validated first, so a corrupt
        table frees nothing (utils/kv_cache.py:164-176)."""
        if request_id not in self.requests:
            raise KVCacheStateError(f"request {request_id!r} is not admitted (freed twice?)")
        for group in self.groups:
            table = group.tables[request_id]
            live = [page for page in table if page != RELEASED]
            if len(set(live)) != len(live):
                raise KVCacheStateError(f"request {request_id!r}: a page appears twice in its block table")
            for page in live:
                if page not in group.pool.references:
                    raise KVCacheStateError(f"request {request_id!r}: page {page} of its block table is not allocated")
        for group in self.groups:
            for page in group.tables.pop(request_id):
                if page != RELEASED:
                    group.pool.release(page)
            del group.released_upto[request_id]
        self.slots.give_back(request_id)
        del self.requests[request_id]

    # ------------------------------------------------------------------ shared prefixes
    def block_digest(self, parent: str, tokens: Sequence[int]) -> str:
        """Chain digest of one complete block: sha256 over [parent digest, tokens, model identity,
        adapter] as utils/engine.py:193-195 builds it."""
        payload = json.dumps([parent, list(tokens), self.model_identity, "none"], separators=(",", ":")).encode("utf-8")
        return hashlib.sha256(payload).hexdigest()

    def _prompt_digests(self, prompt: Sequence[int]):
        """Chain digests of the prompt's complete blocks that may be shared: all but the block holding the last
        token, so that at least one token is left to compute (utils/engine.py:197-208)."""
        parent = "root"
        for block in range((len(prompt) - 1) // self.page_size):
            parent = self.block_digest(parent, prompt[block * self.page_size:(block + 1) * self.page_size])
            yield parent

    def share_prefix(self, request_id, prompt: Sequence[int]) -> int:
        """Takes over cached pages for the longest prefix of complete blocks that EVERY group still holds.  Returns the
        number of tokens covered."""
        if not self.prefix_sharing:
            return 0
        tables = [group.tables[request_id] for group in self.groups]
        if any(tables):
            raise KVCacheStateError("shared prefixes are looked up before anything is allocated")
        covered = 0
        for digest in self._prompt_digests(prompt):
            if any(group.pool.lookup(digest) is None for group in self.groups):
                break
            for group, table in zip(self.groups, tables):
                group.pool.share(digest, table)
            covered += self.page_size
        self.requests[request_id] = covered
        return covered

    def probe_prefix(self, prompt: Sequence[int]):
        """What ``share_prefix`` would do, without doing it: (tokens covered, how many of the pages taken are idle
        now and would stop counting as available; with several groups, the most in any of them)."""
        if not self.prefix_sharing:
            return 0, 0
        covered, idle = 0, [0] * len(self.groups)
        for digest in self._prompt_digests(prompt):
            pages = [group.pool.lookup(digest) for group in self.groups]
            if any(page is None for page in pages):
                break
            for index, (group, page) in enumerate(zip(self.groups, pages)):
                idle[index] += page in group.pool.idle
            covered += self.page_size
        return covered, max(idle)

    def register_prefix(self, request_id, prompt: Sequence[int], old_computed: int, new_computed: int) -> None:
        """Hashes, in every group, the prompt blocks completed by the step that moved the request from
        ``old_computed`` to ``new_computed`` tokens (utils/engine.py:382-401)."""
        if not self.prefix_sharing:
            return
        first = min(old_computed, len(prompt)) // self.page_size
        last = min(new_computed, len(prompt)) // self.page_size
        for group in self.groups:
            table = group.tables[request_id]
            for block in range(first, last):
                parent = "root" if block == 0 else group.pool.digest_of.get(table[block - 1])
                if parent is None:
                    break
                digest = self.block_digest(parent, prompt[block * self.page_size:(block + 1) * self.page_size])
                group.pool.register_digest(table[block], digest)

    # ------------------------------------------------------------------ checks
    def check_invariants(self) -> None:
        for group in self.groups:
            group.pool.check_invariants()
            counts: Dict[int, int] = {}
            for table in group.tables.values():
                for page in table:
                    if page != RELEASED:
                        counts[page] = counts.get(page, 0) + 1
            if getattr(group, "null_page", None) is not None:
                counts[group.null_page] = counts.get(group.null_page, 0) + 1
            if counts != group.pool.references:
                raise AssertionError(f"group {group.index}: block tables and reference counts disagree")
        held = set(self.slots.slot_of.values())
        if len(held) != len(self.slots.slot_of) or held & set(self.slots.free):
            raise AssertionError("a state slot is held twice or is both held and free")
        if len(held) + len(self.slots.free) != self.slots.num_slots:
            raise AssertionError("a state slot was lost")
