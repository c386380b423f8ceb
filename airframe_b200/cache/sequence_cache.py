"""The cache: a slot for each live sequence, keys and values for each cached
run of a layer, each sequence with its own length.

Storage is paged.  A *group* holds the runs of layers with the same need
(number of kv heads, head size, all keys or a window of them).  Each group
owns K and V pages ``[runs, pages, kv_heads, PAGE, head_dim]`` and a page
table ``[slots, pages per sequence]``.  A group with a window keeps rows
modulo ``ring_rows`` (the window rounded up to whole pages), so a sequence
never holds more than ``ring_rows`` rows there.  Pages are taken as a
sequence grows and given back, with the slot, when it ends; both are used
again by later sequences.

Beside the pages lies per-sequence state of fixed size for mixers that ask
for it: ``[runs, slots, *shape]``, zeroed when a slot is taken.

Reference: the single-sequence ``KVCache`` (``src/backend/bindless/kv_cache.rs:18-61``,
layout ``:106-108``, overflow error ``:284-293``, ``reset`` ``:259-262``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import transfers

from ..kernels_const import PAGE
from ..parts.base import KVNeed
from .pool import CacheFull, IndexPool, PoolError

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


class ContextOverflow(RuntimeError):
    """A sequence would grow beyond the longest context the cache was built for."""


def pages_for(rows: int) -> int:
    return (rows + PAGE - 1) // PAGE


class KVGroup:
    """Pages and page tables of the runs that share one :class:`KVNeed`."""

    def __init__(self, need: KVNeed, run_ids, n_slots: int, n_pages: int, max_context: int,
                 dtype, device):
        self.need = need
        self.run_ids = list(run_ids)
        self.index_of = {r: i for i, r in enumerate(self.run_ids)}
        self.ring_rows = pages_for(need.window) * PAGE if need.window else 0
        cap_rows = min(self.ring_rows, max_context) if self.ring_rows else max_context
        self.pages_per_seq = max(1, pages_for(cap_rows))
        self.n_pages = n_pages
        self.pages = IndexPool(n_pages, "cache page")
        self.held = [[] for _ in range(n_slots)]        # slot -> its pages, in row order
        self.table_host = torch.full((n_slots, self.pages_per_seq), -1, dtype=torch.int32)
        self.dirty = set()
        self.k = self.v = self.table = None
        if device is not None:
            shape = (len(self.run_ids), n_pages, need.num_kv_heads, PAGE, need.head_dim)
            self.k = torch.zeros(shape, dtype=dtype, device=device)
            self.v = torch.zeros(shape, dtype=dtype, device=device)
            self.table = torch.full((n_slots, self.pages_per_seq), -1, dtype=torch.int32, device=device)

    def rows_held(self, length: int) -> int:
        return min(length, self.ring_rows) if self.ring_rows else length

    def pages_missing(self, slot: int, new_len: int) -> int:
        return max(0, pages_for(self.rows_held(new_len)) - len(self.held[slot]))

    def room(self, slot: int) -> int:
        """Tokens the sequence may hold before this group needs another page."""
        held = len(self.held[slot])
        if self.ring_rows and held * PAGE >= self.ring_rows:
            return 1 << 62                  # the ring is complete: it never grows again
        return held * PAGE

    def grow(self, slot: int, new_len: int) -> None:
        n = self.pages_missing(slot, new_len)
        if n == 0:
            return
        have = len(self.held[slot])
        new = self.pages.take_many(n)
        self.held[slot].extend(new)
        for j, p in enumerate(new):
            self.table_host[slot, have + j] = p
        self.dirty.add(slot)

    def release(self, slot: int) -> None:
        for p in self.held[slot]:
            self.pages.give_back(p)
        if self.held[slot]:
            self.table_host[slot, : len(self.held[slot])] = -1
            self.dirty.add(slot)
        self.held[slot] = []

    def flush(self) -> None:
        """Bring the device's page table up to date (rows that changed).  The
        rows travel in a buffer of their own: the host table goes on changing
        while earlier copies may still wait in the stream."""
        if self.table is not None and self.dirty:
            slots = sorted(self.dirty)
            rows = torch.empty(len(slots), 1 + self.pages_per_seq, dtype=torch.int32).pin_memory()
            rows[:, 0] = torch.tensor(slots, dtype=torch.int32)
            rows[:, 1:] = self.table_host[slots]
            dev = rows.to(self.table.device, non_blocking=True)
            transfers.count_h2d(rows)
            self.table.index_copy_(0, dev[:, 0].long(), dev[:, 1:])
        self.dirty.clear()

    def bytes_per_token(self) -> int:
        el = 2 if self.k is None else self.k.element_size()
        return 2 * len(self.run_ids) * self.need.num_kv_heads * self.need.head_dim * el


@dataclass
class KVView:
    """What a mixer sees of its run's keys and values."""
    k: Optional[torch.Tensor]           # [pages, kv_heads, PAGE, head_dim]
    v: Optional[torch.Tensor]
    page_table: Optional[torch.Tensor]  # [slots, pages per sequence] int32
    ring_rows: int                      # 0: rows are positions; else rows are positions modulo this
    need: KVNeed


@dataclass
class LayerCacheView:
    """The cache as one run of a layer sees it."""
    cache_id: int                       # the schedule entry whose storage this is
    writes: bool                        # False: the run reads another run's keys and values
    keep_step_kv: bool                  # a later run reads this run's keys and values
    kv: Optional[KVView]
    state: Optional[torch.Tensor]       # [slots, *shape]


class SequenceCache:
    """Slots, pages and fixed-size state for all runs of a model.

    ``needs`` lists, per schedule entry, ``(KVNeed | None, StateNeed | None,
    cache_from | None)``.  ``max_tokens`` is the most tokens live sequences
    hold together, each rounded up to whole pages; ``max_context`` the longest
    single sequence.  With ``device=None`` only the bookkeeping exists.

    ``max_sequences`` bounds the slots.  A group with a window never holds
    more than its ring of a sequence, so it gets ``slots x ring`` pages when
    that is less than ``max_tokens``: the saving of memory that the ring is
    for shows only when the caller names the most sequences it will hold at a
    time (by default there are as many slots as pages, and no saving).
    """

    def __init__(self, needs, max_tokens: int, max_context: int, dtype=torch.bfloat16, device=None,
                 max_sequences: Optional[int] = None):
        if max_tokens < PAGE:
            max_tokens = PAGE
        self.max_context = int(max_context)
        self.total_pages = pages_for(max_tokens)
        self.n_slots = self.total_pages if max_sequences is None else min(max_sequences, self.total_pages)
        self.slots = IndexPool(self.n_slots, "cache slot")
        self.lens = [0] * self.n_slots
        self.room = [0] * self.n_slots       # tokens that fit into the pages a slot holds in every group
        self.device = device
        self.dtype = dtype
        self.groups: dict = {}
        self.states: dict = {}
        self.views: list = []
        by_need: dict = {}
        readers = {n[2] for n in needs if n[2] is not None}
        for run, (kv_need, state_need, cache_from) in enumerate(needs):
            if cache_from is None and kv_need is not None:
                by_need.setdefault(kv_need, []).append(run)
        for need, runs in by_need.items():
            n_pages = self.total_pages
            if need.window:
                ring_pages = pages_for(min(pages_for(need.window) * PAGE, self.max_context))
                n_pages = min(n_pages, self.n_slots * ring_pages)
            self.groups[need] = KVGroup(need, runs, self.n_slots, n_pages, self.max_context, dtype, device)
        for run, (kv_need, state_need, cache_from) in enumerate(needs):
            src = run if cache_from is None else cache_from
            kv_view = None
            src_need = needs[src][0]
            if kv_need is not None:
                if src_need is None:
                    raise ValueError(f"run {run} reads keys and values of run {src}, which keeps none")
                if (src_need.num_kv_heads, src_need.head_dim) != (kv_need.num_kv_heads, kv_need.head_dim):
                    raise ValueError(f"run {run} reads the cache of run {src} with other head sizes")
                g = self.groups[src_need]
                i = g.index_of[src]
                kv_view = KVView(g.k[i] if g.k is not None else None, g.v[i] if g.v is not None else None,
                                 g.table, g.ring_rows, src_need)
            state = None
            if state_need is not None:
                if device is not None:
                    state = torch.zeros((self.n_slots, *state_need.shape),
                                        dtype=_STATE_DTYPES[state_need.dtype], device=device)
                self.states[run] = state
            self.views.append(LayerCacheView(cache_id=src, writes=cache_from is None,
                                             keep_step_kv=run in readers, kv=kv_view, state=state))

    # ------------------------------------------------------------------ slots

    def take_slot(self) -> int:
        slot = self.slots.take()
        self.lens[slot] = 0
        self.room[slot] = 0
        for st in self.states.values():
            if st is not None:
                st[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise PoolError(f"cache slot {slot} is not held (freed twice or never taken)")
        for g in self.groups.values():
            g.release(slot)
        self.lens[slot] = 0
        self.room[slot] = 0
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise PoolError(f"cache slot {slot} is not held")
        return self.lens[slot]

    # ------------------------------------------------------------------ growth

    def reserve(self, growth: dict) -> None:
        """Make room for ``growth`` (slot -> new length) or raise without
        changing anything."""
        for slot, new_len in growth.items():
            if not self.slots.is_held(slot):
                raise PoolError(f"cache slot {slot} is not held")
            if new_len > self.max_context:
                raise ContextOverflow(f"sequence in slot {slot} would hold {new_len} tokens; "
                                      f"the cache is built for {self.max_context}")
        # most steps add a token that still fits into the pages held: nothing to take
        short = {s: n for s, n in growth.items() if n > self.room[s]}
        if not short:
            return
        for g in self.groups.values():
            want = sum(g.pages_missing(s, n) for s, n in short.items())
            if want > g.pages.n_free:
                raise CacheFull(f"{want} more cache pages wanted, {g.pages.n_free} of {g.n_pages} free "
                                f"(window {g.need.window})")
        for g in self.groups.values():
            for s, n in short.items():
                g.grow(s, n)
        for s in short:
            self.room[s] = min((g.room(s) for g in self.groups.values()), default=self.max_context)

    def commit(self, growth: dict) -> None:
        for slot, new_len in growth.items():
            self.lens[slot] = new_len

    def flush(self) -> None:
        for g in self.groups.values():
            g.flush()

    def fits(self, token_counts) -> bool:
        """Whether sequences that come to hold these many tokens fit together:
        a slot each, and in every group the pages they hold there (a group with
        a window holds at most its ring of a sequence)."""
        if len(token_counts) > self.n_slots:
            return False
        return all(sum(pages_for(g.rows_held(n)) for n in token_counts) <= g.n_pages for g in self.groups.values())

    # ------------------------------------------------------------------ figures

    def pages_held(self) -> dict:
        return {need: g.pages.n_held for need, g in self.groups.items()}

    def bytes_allocated(self) -> int:
        n = 0
        for g in self.groups.values():
            if g.k is not None:
                n += g.k.numel() * g.k.element_size() * 2
        return n
