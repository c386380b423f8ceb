"""One step's tokens as the kernels want them.

A step is either a *prefill* (every sequence brings its first tokens, lengths
may differ, rows are concatenated sequence after sequence) or a *decode* step
(every sequence brings one more token).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import transfers


@dataclass
class StepEntry:
    """The next tokens of one sequence and the places among them whose logits are wanted."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)


@dataclass
class StepBatch:
    is_prefill: bool
    n_tokens: int
    n_seqs: int
    max_len: int                        # longest sequence of the step (tokens brought)
    seq_lens: list                      # host: tokens brought per sequence
    tokens: torch.Tensor                # int32 [T]
    positions: torch.Tensor             # int32 [T] position of each token in its sequence
    seq_of_token: torch.Tensor          # int32 [T] index into slots
    slots: torch.Tensor                 # int32 [B] cache slot per sequence; -1 = padding
    len_after: torch.Tensor             # int32 [B] sequence length once the step is done
    seq_starts: torch.Tensor            # int32 [B + 1] first row of each sequence
    want_rows: Optional[torch.Tensor]   # int32 [R] rows whose logits are wanted
    n_want: int = 0
    max_len_after: int = 0              # host: longest sequence after the step
    step_kv: dict = field(default_factory=dict)   # cache id -> (k, v) of this step, for runs that share a cache
    # what parts make once per forward pass and share between layers (a table of rotary cosines and sines,
    # the tokens' rows in a group's cache pages); emptied when a pass begins
    aux: dict = field(default_factory=dict)


def build_batch(entries, lens_before, device, pad_to: int = 0) -> StepBatch:
    """Lay out ``entries`` (validated by the caller) on the device with one copy.
    ``pad_to`` > B adds padding sequences (slot -1, token 0) to a decode step."""
    is_prefill = all(n == 0 for n in lens_before)
    seq_lens = [len(e.tokens) for e in entries]
    B = len(entries)
    tokens, positions, seq_of, starts, want_rows = [], [], [], [0], []
    for b, (e, before) in enumerate(zip(entries, lens_before)):
        base = len(tokens)
        tokens.extend(e.tokens)
        positions.extend(range(before, before + len(e.tokens)))
        seq_of.extend([b] * len(e.tokens))
        starts.append(len(tokens))
        want_rows.extend(base + w for w in e.want)
    slots = [e.slot for e in entries]
    len_after = [before + n for before, n in zip(lens_before, seq_lens)]
    if pad_to > B:
        if is_prefill:
            raise ValueError("only decode steps are padded")
        for _ in range(pad_to - B):
            tokens.append(0)
            positions.append(0)
            seq_of.append(len(slots))
            slots.append(-1)
            len_after.append(0)
            starts.append(len(tokens))
    T, Bp, R = len(tokens), len(slots), len(want_rows)
    flat = tokens + positions + seq_of + slots + len_after + starts + want_rows
    host = torch.tensor(flat, dtype=torch.int32)
    if device.type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)
    transfers.count_h2d(host)
    o = 0

    def cut(n):
        nonlocal o
        t = dev[o:o + n]
        o += n
        return t

    return StepBatch(
        is_prefill=is_prefill, n_tokens=T, n_seqs=Bp, max_len=max(seq_lens), seq_lens=seq_lens,
        tokens=cut(T), positions=cut(T), seq_of_token=cut(T), slots=cut(Bp), len_after=cut(Bp),
        seq_starts=cut(Bp + 1), want_rows=cut(R) if R else None, n_want=R,
        max_len_after=max(len_after))
