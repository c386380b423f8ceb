"""The generation loop above the step function: requests are served in
batches, one batch after another; a batch's prompts (of unequal lengths) run
in one step, then every live sequence gets one token per step; a sequence
ends at a stop token (not emitted), at ``max_tokens`` or at the context limit,
leaves the batch and gives its slot back at once.

Reference: rules 3-5 of the single-sequence loop
(``crates/airframe_observe/src/isf.rs:333-529``): halt on the end token or an
extra stop id (``:397-410,477-483``), on max_tokens (``:481-485``); the context
limit of ``src/bin/shimmy_server_gpu/server_inference.rs:1246-1253``.

The loop needs of its engine: ``take_slot()``, ``free_slot(slot)``,
``step(entries) -> logits``, ``max_context``, ``vocab_size`` and
``cache.total_pages`` / ``cache.n_slots``; of its sampler:
``new_state(params, index)`` and ``sample(logits, states, params) -> tokens``.

With an engine that has ``decode_rows`` (decode steps captured into CUDA
graphs) and a sampler that has ``sample_async``, and without a repetition
penalty (it needs the token before the next step), the loop keeps the device
one step ahead of the host: step k + 1 takes its tokens from the device, where
the sampler of step k left them, and is queued before the host has read them.
What the host knows without the tokens (max_tokens, the context limit) it
applies in time; a stop token it sees one step late: that sequence's next
step is already queued, its result is dropped and nothing of it is emitted.
The tokens are the same either way.

A ``logits_processor`` is the loop's control hook (reference: ``InferenceControl::intervene``
with its decisions Allow / ForceToken / EarlyExit / BlockAndTerminate, ``src/control.rs:29-52``,
applied per token at ``src/runtime/engine.rs:183-205``).  It is called for every live
sequence before its token is chosen, with the request's index, the generation step
(0 for the first new token), the sequence's row of logits on the device (which it may
change in place: then the sampler chooses among what it left) and the tokens so far.
It returns None (go on), a token id (that token is emitted instead of the sampler's
choice), or :data:`STOP` (the sequence ends cleanly, reason ``control``); raising
:class:`Blocked` ends the whole call.  With a processor the loop steps in lock-step
(the host must see every token before the next step is laid out).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

from ..kernels_const import PAGE
from .batch import StepEntry


STOP = "stop"


class Blocked(RuntimeError):
    """A logits processor refused to let generation go on."""


class RequestError(ValueError):
    """A request cannot be served: empty, too long, or a bad token id."""


@dataclass
class _Sequence:
    index: int                 # position among the requests
    prompt: list
    slot: int = -1
    state: object = None
    out: list = field(default_factory=list)
    length: int = 0            # tokens in the cache
    finish: Optional[str] = None


def _pages(n: int) -> int:
    return (n + PAGE - 1) // PAGE


class GenerationLoop:
    def __init__(self, engine, sampler, stop_token_ids=(), max_batch: Optional[int] = None):
        self.engine = engine
        self.sampler = sampler
        self.model_stop_ids = set(stop_token_ids)
        self.max_batch = max_batch
        self.pipelined = True          # keep the device a step ahead of the host where engine and sampler allow
        self.finish_reasons: list = []
        self.batches_run: list = []

    # ------------------------------------------------------------------ planning

    def check(self, prompts, params) -> None:
        params.check()
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise RequestError(f"request {i}: the prompt is empty")
            if len(p) > self.engine.max_context:
                raise RequestError(f"request {i}: the prompt has {len(p)} tokens, the context holds "
                                   f"{self.engine.max_context}")
            for t in p:
                if not isinstance(t, int) or not 0 <= t < self.engine.vocab_size:
                    raise RequestError(f"request {i}: token id {t!r} outside the vocabulary")

    def tokens_held(self, prompt_len: int, params) -> int:
        """The most tokens a request can come to hold."""
        return min(prompt_len + max(params.max_tokens - 1, 0), self.engine.max_context)

    def plan_batches(self, prompts, params) -> list:
        """Requests in order, as many to a batch as slots and cache pages allow."""
        total_pages = self.engine.cache.total_pages
        limit = self.engine.cache.n_slots
        if self.max_batch:
            limit = min(limit, self.max_batch)
        # a cache whose groups of layers have storage of their own answers for each of them
        fits = getattr(self.engine.cache, "fits", None)
        batches, cur, cur_pages = [], [], 0
        for i, p in enumerate(prompts):
            held = self.tokens_held(len(p), params)
            need = _pages(held)
            if need > total_pages or (fits is not None and not fits([held])):
                raise RequestError(f"request {i} needs {need} cache pages, the cache has {total_pages}")
            if cur and (len(cur) >= limit or cur_pages + need > total_pages
                        or (fits is not None and not fits([self.tokens_held(len(prompts[j]), params) for j in cur]
                                                          + [held]))):
                batches.append(cur)
                cur, cur_pages = [], 0
            cur.append(i)
            cur_pages += need
        if cur:
            batches.append(cur)
        return batches

    # ------------------------------------------------------------------ running

    def generate(self, prompts, params, on_token: Optional[Callable] = None,
                 logits_processor: Optional[Callable] = None) -> list:
        """New token ids per request, in request order.  ``on_token(request
        index, token id)`` is called for every emitted token;
        ``logits_processor(request index, step, logits row, tokens so far)``
        before every choice (see the module's text)."""
        self.check(prompts, params)
        results = [[] for _ in prompts]
        self.finish_reasons = [None] * len(prompts)
        self.batches_run = []
        if params.max_tokens == 0:
            self.finish_reasons = ["length"] * len(prompts)
            return results
        stops = set(params.stop_token_ids)
        if not params.ignore_eos:
            stops |= self.model_stop_ids
        for batch in self.plan_batches(prompts, params):
            self.batches_run.append(list(batch))
            seqs = [_Sequence(i, list(prompts[i])) for i in batch]
            try:
                for s in seqs:
                    s.slot = self.engine.take_slot()
                    s.state = self.sampler.new_state(params, s.index)
                self._run_batch(seqs, params, stops, on_token, logits_processor)
            finally:
                for s in seqs:
                    if s.slot >= 0:
                        self.engine.free_slot(s.slot)
                        s.slot = -1
            for s in seqs:
                results[s.index] = s.out
                self.finish_reasons[s.index] = s.finish
        return results

    def _end(self, s: _Sequence, reason: str) -> None:
        s.finish = reason
        self.engine.free_slot(s.slot)
        s.slot = -1

    def _run_batch(self, seqs, params, stops, on_token, processor=None) -> None:
        ahead = (self.pipelined and processor is None and params.repetition_penalty == 1.0
                 and hasattr(self.engine, "decode_rows")
                 and hasattr(self.sampler, "sample_async") and getattr(self.engine, "use_graphs", False))
        if ahead:
            self._run_batch_ahead(seqs, params, stops, on_token)
        else:
            self._run_batch_in_step(seqs, params, stops, on_token, processor)

    def _run_batch_in_step(self, seqs, params, stops, on_token, processor=None) -> None:
        """Every step waits for the tokens of the step before."""
        logits = self.engine.step([StepEntry(s.slot, s.prompt, [len(s.prompt) - 1]) for s in seqs])
        for s in seqs:
            s.length = len(s.prompt)
        active = list(seqs)
        while active:
            decisions = [None] * len(active)
            if processor is not None:
                for r, s in enumerate(active):
                    d = processor(s.index, len(s.out), logits[r], s.prompt + s.out)
                    if not (d is None or d == STOP or (isinstance(d, int) and not isinstance(d, bool)
                                                       and 0 <= d < self.engine.vocab_size)):
                        raise RequestError(f"request {s.index}: the logits processor returned {d!r} "
                                           f"(None, a token id or STOP)")
                    decisions[r] = d
            tokens = self.sampler.sample(logits, [s.state for s in active], params)
            going = []
            for s, t, d in zip(active, tokens, decisions):
                if d == STOP:
                    self._end(s, "control")
                    continue
                if d is not None:
                    # the sampler's choice is discarded (its draw is spent, as in the reference, where the
                    # candidate is sampled before the hook sees it); what sampling remembers is the forced token
                    fix = getattr(s.state, "replace_last", None)
                    if fix is not None:
                        fix(d)
                    t = d
                if t in stops:
                    self._end(s, "stop")
                    continue
                s.out.append(t)
                if on_token is not None:
                    on_token(s.index, t)
                if len(s.out) >= params.max_tokens:
                    self._end(s, "length")
                elif s.length + 1 > self.engine.max_context:
                    self._end(s, "context")
                else:
                    going.append(s)
            active = going
            if not active:
                break
            logits = self.engine.step([StepEntry(s.slot, [s.out[-1]], [0]) for s in active], borrow=True)
            for s in active:
                s.length += 1

    def _run_batch_ahead(self, seqs, params, stops, on_token) -> None:
        """The device one step ahead of the host.  Row r of every decode step
        belongs to seqs[r]; a sequence that has ended leaves its row unused."""
        eng, smp = self.engine, self.sampler
        # greedy decoding with an engine whose head finds the best token itself: the steps give tokens,
        # not logits, and the sampler only brings them to the host
        fused = bool(params.greedy and getattr(eng, "fused_greedy", False) and hasattr(smp, "adopt"))
        kw = {"greedy": True} if fused else {}
        logits = eng.step([StepEntry(s.slot, s.prompt, [len(s.prompt) - 1]) for s in seqs], **kw)
        for s in seqs:
            s.length = len(s.prompt)
        n = len(seqs)
        sampled = [1] * n                       # samples asked for per row, the one in flight included
        pend = (smp.adopt(logits, [s.state for s in seqs]) if fused
                else smp.sample_async(logits, [s.state for s in seqs], params))
        pend_rows = list(range(n))              # rows whose tokens `pend` carries
        while True:
            # rows that go on whatever their token in flight is, unless it is a stop token
            go = [r for r in pend_rows
                  if seqs[r].finish is None and sampled[r] < params.max_tokens
                  and seqs[r].length + 1 <= eng.max_context]
            nxt = None
            if go:
                on = set(go)
                logits = eng.decode_rows([seqs[r].slot if r in on else None for r in range(n)], pend.device, **kw)
                states = [seqs[r].state if r in on else None for r in range(n)]
                nxt = smp.adopt(logits, states) if fused else smp.sample_async(logits, states, params)
            # now the tokens in flight (the next step is queued behind them)
            tokens = pend.result()
            for r in pend_rows:
                s = seqs[r]
                if s.finish is not None:
                    continue
                t = tokens[r]
                if t in stops:
                    self._end(s, "stop")        # its row of the queued step is wasted
                    continue
                s.out.append(t)
                if on_token is not None:
                    on_token(s.index, t)
                if len(s.out) >= params.max_tokens:
                    self._end(s, "length")
                elif s.length + 1 > eng.max_context:
                    self._end(s, "context")
            if nxt is None:
                break
            for r in go:
                seqs[r].length += 1
                sampled[r] += 1
            pend, pend_rows = nxt, go
