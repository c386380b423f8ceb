"""The step function: a model, its cache, and one call that runs the tokens
it is given against what earlier steps left in the cache.

Reference: ``run_full_model_with_cache_state``
(``src/backend/bindless/pipeline/inference.rs:342-353``), which steps one
sequence and returns the last token's logits; here a step carries a batch of
sequences of unequal lengths and returns logits at the wanted places.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import PoolError, SequenceCache
from .batch import StepBatch, StepEntry, build_batch
from .model import Model


class StepError(ValueError):
    """A step was malformed: unknown slot, mixed kinds, bad token or place."""


class Engine:
    """``max_tokens``: the most tokens that live sequences hold together (each
    sequence's count rounded up to whole cache pages).  ``max_context``: the
    longest single sequence (the model's own limit by default)."""

    def __init__(self, model: Model, max_tokens: int, max_context: Optional[int] = None,
                 max_sequences: Optional[int] = None):
        if not model.loaded:
            raise ValueError("the model has no weights yet")
        self.model = model
        self.device = model.ctx.device
        limit = model.spec.max_positions
        self.max_context = min(max_context, limit) if max_context else limit
        self.cache = SequenceCache(model.cache_needs(), max_tokens, self.max_context,
                                   dtype=model.ctx.compute_dtype, device=self.device,
                                   max_sequences=max_sequences)
        self.vocab_size = model.spec.vocab_size

    # ------------------------------------------------------------------ slots

    def take_slot(self) -> int:
        return self.cache.take_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------------ step

    def check(self, entries) -> list:
        """Validate a step; returns each sequence's length before it."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen = set()
        lens = []
        for e in entries:
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            try:
                lens.append(self.cache.length(e.slot))
            except PoolError as err:
                raise StepError(str(err)) from err
            if len(e.tokens) == 0:
                raise StepError(f"slot {e.slot}: a step needs at least one token per sequence")
            for t in e.tokens:
                if not 0 <= t < self.vocab_size:
                    raise StepError(f"slot {e.slot}: token id {t} outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"slot {e.slot}: wanted place {w} outside its {len(e.tokens)} tokens")
        starting = [n == 0 for n in lens]
        if any(starting) and not all(starting):
            raise StepError("the sequences of a step either all start or all go on")
        if not all(starting) and any(len(e.tokens) != 1 for e in entries):
            raise StepError("sequences that go on bring one token each")
        return lens

    def step(self, entries, pad_to: int = 0):
        """Run one step.  Returns float32 logits [wanted, vocab] on the device,
        in the order of the entries and of their ``want`` lists, or None when
        nothing is wanted."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        lens = self.check(entries)
        growth = {e.slot: n + len(e.tokens) for e, n in zip(entries, lens)}
        self.cache.reserve(growth)
        self.cache.flush()
        batch = build_batch(entries, lens, self.device, pad_to=pad_to)
        logits = self.model.forward(batch, self.cache)
        self.cache.commit(growth)
        return logits
