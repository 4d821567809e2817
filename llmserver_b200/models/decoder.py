"""The generic decoder: embedding, the scheduled layers, final norm, output head.

Built from a ``ModelSpec`` alone; which architecture the specification came from does not matter
here.  ``step`` is the model half of the engine's step function: it runs exactly the tokens of the
batch, against the cache, and returns float32 logits at the rows the batch asks for.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..config.spec import ModelSpec
from ..parts import BLOCKS, MIXERS, NORMS, POSITION_ENCODINGS, EntryCache, Runtime
from ..parts.registry import parts_of_layer
from ..parts.base import Block


class DecoderModel:
    def __init__(self, spec: ModelSpec, source, runtime: Runtime):
        """``source.get(full tensor name)`` returns the tensor on the device in the right dtype."""
        spec.validate()
        self.spec, self.runtime = spec, runtime
        self.positions = {}
        for name, part in spec.positions.items():
            cls = POSITION_ENCODINGS.get(part.kind)
            weights = {local: source.get(f"model.positions.{name}.{local}") for local in cls.declare_weights(part.as_dict())}
            self.positions[name] = cls(part.as_dict(), weights, runtime)
        self.embedding = source.get(spec.embedding_name).contiguous()
        self.layers: List[Block] = []
        for layer in spec.layers:
            block_cls = BLOCKS.get(layer.block.kind)
            block_params = layer.block.as_dict()
            built = {}
            for role, part, cls, prefix in parts_of_layer(layer):
                weights = {local: source.get(prefix + local) for local in cls.declare_weights(part.as_dict())}
                built[role] = cls(part.as_dict(), weights, runtime)
            built[block_cls.mixer_role(block_params)].attach(self.positions.get(layer.position) if layer.position else None)
            self.layers.append(block_cls(block_params, built))
        norm_cls = NORMS.get(spec.final_norm.kind)
        self.final_norm = norm_cls(spec.final_norm.as_dict(),
                                   {local: source.get(spec.final_norm_prefix + local)
                                    for local in norm_cls.declare_weights(spec.final_norm.as_dict())}, runtime)
        # tied head: the same tensor as the embedding (utils/model_loader.py:56-57)
        self.head = self.embedding if spec.tie_head else source.get(spec.head_name).contiguous()
        self.entry_caches: Optional[List[EntryCache]] = None

    # ------------------------------------------------------------------ cache
    def cache_needs(self) -> list:
        """Per schedule entry, what it keeps for itself (None when it reads another entry's cache)."""
        needs = []
        for entry in self.spec.schedule:
            layer = self.spec.layers[entry.layer]
            block_cls = BLOCKS.get(layer.block.kind)
            mixer = layer.part(block_cls.mixer_role(layer.block.as_dict()))
            need = MIXERS.get(mixer.kind).cache_need(mixer.as_dict())
            needs.append(None if entry.cache_from is not None else need)
        return needs

    def bind_cache(self, cache) -> None:
        """Resolves every schedule entry's view of the cache manager's storage."""
        views = []
        for index, entry in enumerate(self.spec.schedule):
            owner = index if entry.cache_from is None else entry.cache_from
            view = EntryCache(writes=entry.cache_from is None)
            if owner in cache.group_of_entry:
                view.k_pages, view.v_pages, view.group = cache.pages_of_entry(owner)
            if owner in cache.state_entries:
                view.state = cache.state_of_entry(owner)
            views.append(view)
        self.entry_caches = views

    # ------------------------------------------------------------------ the step
    def step(self, batch) -> torch.Tensor:
        if self.entry_caches is None:
            raise RuntimeError("bind_cache() has to be called before the first step")
        residual = ops.embedding(self.embedding, batch.token_ids)
        for position in self.positions.values():
            position.on_embedding(residual, batch)
        delta = None
        schedule = self.spec.schedule
        for index, entry in enumerate(schedule):
            block = self.layers[entry.layer]
            if block.passes_stream:
                # what runs next, for a block whose last part can prepare that norm's input
                after = self.layers[schedule[index + 1].layer].entry() if index + 1 < len(schedule) else (self.final_norm, None)
                residual, delta = block.forward(residual, delta, batch, self.entry_caches[index], after=after)
            else:
                residual, delta = block.forward(residual, delta, batch, self.entry_caches[index])
        if batch.n_logits == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        # final norm only where logits are wanted (utils/model.py:147-157)
        normed = self.final_norm.add_norm(residual, delta, rows=batch.logit_rows)
        return ops.linear(normed, self.head, out_dtype=torch.float32)
