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

from .. import transfers

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
                 max_sequences: Optional[int] = None, use_graphs: bool = True):
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
        # decode steps of models whose parts allow it are captured into CUDA graphs,
        # one per padded batch size
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda" and model.graph_safe
        self._graphs: dict = {}
        self.replayed_launches = 0      # kernels launched through graph replays

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

    fused_greedy = True     # step(..., greedy=True) and decode_rows(..., greedy=True) give tokens instead of logits

    def step(self, entries, pad_to: int = 0, borrow: bool = False, probe=None, greedy: bool = False):
        """Run one step.  Returns float32 logits [wanted, vocab] on the device,
        in the order of the entries and of their ``want`` lists, or None when
        nothing is wanted.  ``borrow``: the caller uses the logits before the
        next step and may get a buffer that the next step overwrites (saves a
        copy when the step ran as a CUDA graph).  ``probe``: a
        :class:`~airframe_b200.engine.probe.LayerProbe` that is shown the
        residual stream after every run (the step then runs kernel by kernel).
        ``greedy``: instead of logits, the arg-max token at every wanted place
        (int32 [wanted] on the device; the logits are not written where the
        head can find the best without them)."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        lens = self.check(entries)
        growth = {e.slot: n + len(e.tokens) for e, n in zip(entries, lens)}
        self.cache.reserve(growth)
        self.cache.flush()
        if probe is None and self.use_graphs and lens[0] > 0 and all(e.want == [0] for e in entries):
            logits = self._decode_graphed([e.slot for e in entries], lens, tokens=[e.tokens[0] for e in entries],
                                          greedy=greedy)
            if not borrow:
                logits = logits.clone()
        else:
            batch = build_batch(entries, lens, self.device, pad_to=pad_to)
            logits = self.model.forward(batch, self.cache, probe, greedy=greedy)
        self.cache.commit(growth)
        return logits

    # ------------------------------------------------------------------ captured decode steps

    @staticmethod
    def padded_batch(n: int) -> int:
        """Decode batches are padded (slot -1, token 0) to these sizes so that
        few graphs serve every batch size."""
        for b in (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256):
            if n <= b:
                return b
        return (n + 127) // 128 * 128

    def decode_rows(self, slots, tokens_dev, borrow: bool = True, greedy: bool = False):
        """One decode step whose tokens are already on the device (the sampler's
        output of the step before): row r carries the next token ``tokens_dev[r]``
        of the sequence in ``slots[r]``; a row with slot None is not used.  Rows keep
        their places from step to step, so the host can queue this step before it has
        read the tokens themselves.  Needs CUDA graphs (``use_graphs``).  Returns the
        logits of all rows [len(slots), vocab], or with ``greedy`` their arg-max
        tokens (int32 [len(slots)])."""
        if not self.use_graphs:
            raise StepError("decode_rows needs captured decode steps")
        live = [s for s in slots if s is not None]
        if not live or len(set(live)) != len(live):
            raise StepError("decode_rows needs at least one sequence, each slot once")
        try:
            lens = [self.cache.length(s) if s is not None else 0 for s in slots]
        except PoolError as err:
            raise StepError(str(err)) from err
        if any(s is not None and n == 0 for s, n in zip(slots, lens)):
            raise StepError("sequences that go on have tokens in the cache")
        if tokens_dev.dtype != torch.int32 or tokens_dev.numel() < len(slots) or not tokens_dev.is_cuda:
            raise StepError("decode_rows wants one int32 token per row on the device")
        growth = {s: n + 1 for s, n in zip(slots, lens) if s is not None}
        self.cache.reserve(growth)
        self.cache.flush()
        logits = self._decode_graphed([-1 if s is None else s for s in slots], lens, tokens_dev=tokens_dev,
                                      greedy=greedy)
        self.cache.commit(growth)
        return logits if borrow else logits.clone()

    def repeat_last_decode(self, n: int) -> None:
        """Runs the captured decode step of the last call ``n`` more times on
        the inputs it had: the same rows go into the cache again and the same
        results come out, nothing else changes.  For measurements (the device's
        clocks settle under the load of the step itself before it is timed)."""
        g = getattr(self, "_last_graph", None)
        if g is None:
            raise StepError("no captured decode step has run yet")
        for _ in range(n):
            g["graph"].replay()

    def _decode_graphed(self, slots, lens, tokens=None, tokens_dev=None, greedy: bool = False):
        """One decode step, every row wanting its token's logits, through a CUDA
        graph.  Rows with slot -1 are padding.  The tokens come from the host
        (``tokens``) or lie on the device already (``tokens_dev``).  The result is
        the graph's own output buffer: it is valid until the next step of the same
        padded size."""
        B = len(slots)
        Bp = self.padded_batch(B)
        key = (Bp, "greedy") if greedy else Bp
        g = self._graphs.get(key)
        if g is None:
            g = self._capture(Bp, greedy)
            self._graphs[key] = g
        # two pinned staging buffers in turn: one may still be in flight when the next step is laid out
        k = g["turn"] = g["turn"] ^ 1
        host, sent = g["host"][k], g["sent"][k]
        sent.synchronize()
        lay = g["host_np"][k]                 # [tokens | positions | slots | len_after], Bp each
        lay[:B] = tokens if tokens is not None else 0
        lay[Bp:Bp + B] = lens
        lay[2 * Bp:2 * Bp + B] = slots
        lay[3 * Bp:3 * Bp + B] = [n + 1 if s >= 0 else 0 for s, n in zip(slots, lens)]
        if B < Bp:
            lay[B:Bp] = 0
            lay[Bp + B:2 * Bp] = 0
            lay[2 * Bp + B:3 * Bp] = -1
            lay[3 * Bp + B:] = 0
        g["dynamic"].copy_(host, non_blocking=True)
        transfers.count_h2d(host)
        sent.record()
        if tokens_dev is not None:
            g["dynamic"][:B].copy_(tokens_dev[:B], non_blocking=True)
        g["graph"].replay()
        self.replayed_launches += g["launches"]
        self._last_graph = g
        return g["logits"][:B]

    def _capture(self, Bp: int, greedy: bool = False) -> dict:
        dev = self.device
        # [tokens | positions | slots | len_after] change every step; the rest is fixed
        dynamic = torch.zeros(4 * Bp, dtype=torch.int32, device=dev)
        dynamic[2 * Bp: 3 * Bp] = -1
        fixed = torch.cat([torch.arange(Bp, dtype=torch.int32), torch.arange(Bp + 1, dtype=torch.int32),
                           torch.arange(Bp, dtype=torch.int32)]).to(dev)
        batch = StepBatch(
            is_prefill=False, n_tokens=Bp, n_seqs=Bp, max_len=1, seq_lens=[1] * Bp,
            tokens=dynamic[:Bp], positions=dynamic[Bp: 2 * Bp], seq_of_token=fixed[:Bp],
            slots=dynamic[2 * Bp: 3 * Bp], len_after=dynamic[3 * Bp:], seq_starts=fixed[Bp: 2 * Bp + 1],
            want_rows=fixed[2 * Bp + 1:], n_want=Bp,
            max_len_after=self.max_context)          # kernels size their splits for the longest context
        # a run outside the graph first: kernels set their attributes and load lazily
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self.model.forward(batch, self.cache, greedy=greedy)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        from .. import kernels
        graph = torch.cuda.CUDAGraph()
        n0 = kernels.launch_count()
        with torch.cuda.graph(graph):
            logits = self.model.forward(batch, self.cache, greedy=greedy)
        return {"graph": graph, "dynamic": dynamic, "logits": logits, "batch": batch, "fixed": fixed,
                "launches": kernels.launch_count() - n0, "turn": 0,
                "host": (hosts := [torch.empty(4 * Bp, dtype=torch.int32).pin_memory() for _ in range(2)]),
                "host_np": [h.numpy() for h in hosts],
                "sent": [torch.cuda.Event() for _ in range(2)]}
