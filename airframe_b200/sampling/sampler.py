"""The device sampler: per-sequence state on the host (recent tokens, the
deterministic generator), one kernel launch per step.

Reference: ``sample_token`` (``src/runtime/gpu.rs:880-962``), the window of 64
recent tokens (``crates/airframe_observe/src/isf.rs:395-396,505-506``).  Every
sequence has a generator of its own, seeded ``seed + index of the request``,
so a sequence's tokens do not depend on what else is in its batch.
"""
from __future__ import annotations

import torch

from .. import kernels, transfers
from .params import RECENT_WINDOW, SamplingParams
from .rng import XorShift64Star


class SequenceSamplingState:
    """What sampling remembers of one sequence."""

    def __init__(self, params: SamplingParams, request_index: int):
        self.rng = XorShift64Star(params.seed + request_index)
        self.recent: list = []

    def note(self, token: int) -> None:
        self.recent.append(token)
        if len(self.recent) > RECENT_WINDOW:
            del self.recent[0]

    def replace_last(self, token: int) -> None:
        """The token noted last was not emitted after all (a control hook put another in its place)."""
        if self.recent:
            self.recent[-1] = token


class PendingTokens:
    """Tokens that the sampling kernel has been asked for: on the device at once
    (``device``, int32 [R], in stream order), on the host after :meth:`result`."""

    def __init__(self, sampler, device_tokens, host, gave_up, event, states):
        self._sampler = sampler
        self.device = device_tokens
        self._host = host
        self._gave_up = gave_up
        self._event = event
        self._states = states
        self._tokens = None

    def result(self) -> list:
        """Waits for the step, checks the device's error word that came with the
        tokens, notes the tokens in the states they belong to (None: no state)."""
        if self._tokens is None:
            self._event.synchronize()
            if int(self._gave_up[0]) != 0:
                kernels.check_device_errors(self._sampler.device)      # clears the word and raises
            self._tokens = self._host.tolist()
            for st, t in zip(self._states, self._tokens):
                if st is not None:
                    st.note(t)
        return self._tokens


class Sampler:
    def __init__(self, vocab_size: int, device):
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self._host_out = [None, None]       # pinned buffers in turn: two samples may be in flight
        self._done = [None, None]
        self._turn = 0

    def new_state(self, params: SamplingParams, request_index: int) -> SequenceSamplingState:
        return SequenceSamplingState(params, request_index)

    def sample(self, logits, states, params: SamplingParams) -> list:
        """One token for each row of ``logits`` (float32 [R, V] on the device;
        changed in place by the penalty).  Advances each state's generator and
        recent-token window."""
        return self.sample_async(logits, states, params).result()

    def sample_async(self, logits, states, params: SamplingParams) -> PendingTokens:
        """As :meth:`sample`, without waiting: the kernel and the copy of its
        tokens to the host are queued.  A row whose state is None takes no draw
        from any generator and notes nothing (its token is not used)."""
        R = logits.shape[0]
        if R != len(states):
            raise ValueError("one sampling state per row of logits")
        use_penalty = params.repetition_penalty != 1.0
        dev = None
        if use_penalty or not params.greedy:
            # what the kernel needs from the host: the draw and the recent tokens of every row
            n_extra = (RECENT_WINDOW + 1) if use_penalty else 0
            host = torch.zeros(R, 1 + n_extra, dtype=torch.int32)
            hv = host.view(torch.float32)
            for r, st in enumerate(states):
                if st is None:
                    continue
                if not params.greedy:
                    hv[r, 0] = st.rng.next_f32()
                if use_penalty:
                    host[r, 1] = len(st.recent)
                    if st.recent:
                        host[r, 2:2 + len(st.recent)] = torch.tensor(st.recent, dtype=torch.int32)
            dev = host.pin_memory().to(self.device, non_blocking=True)
            transfers.count_h2d(host)
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        kernels.sample(logits, out, params.temperature, params.top_p, params.repetition_penalty,
                       uniform=dev.view(torch.float32)[:, 0] if not params.greedy else None,
                       recent=dev[:, 2:] if use_penalty else None,
                       n_recent=dev[:, 1] if use_penalty else None)
        return self.adopt(out, states)

    def adopt(self, out, states) -> PendingTokens:
        """Tokens that are on the device already (int32 [R], one per state; the
        step function's own greedy choice): queues their copy to the host like
        :meth:`sample_async` does for the tokens it draws."""
        R = len(states)
        if out.dtype != torch.int32 or out.numel() < R:
            raise ValueError("one int32 token per state")
        out = out[:R]
        # the tokens come back through pinned memory kept for the purpose
        k = self._turn = self._turn ^ 1
        if self._done[k] is not None:
            self._done[k].synchronize()                  # (its last user has long been read)
        if self._host_out[k] is None or self._host_out[k].numel() < R + 1:
            self._host_out[k] = torch.empty(max(R, 64) + 1, dtype=torch.int32).pin_memory()
            self._done[k] = torch.cuda.Event()
        back = self._host_out[k][:R]
        back.copy_(out, non_blocking=True)
        transfers.count_d2h(back)
        # with the tokens comes the word that a kernel sets when one of its bounded waits ran out
        gave_up = self._host_out[k][-1:]
        gave_up.copy_(kernels.error_word(self.device), non_blocking=True)
        transfers.count_d2h(gave_up)
        self._done[k].record(torch.cuda.current_stream(self.device))
        return PendingTokens(self, out, back, gave_up, self._done[k], list(states))
