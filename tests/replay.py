"""Ways of cutting the same requests into steps, all through the engine's own
step function (teacher-forced: the tokens are given, nothing is sampled)."""
from __future__ import annotations

import random

import torch

from airframe_b200.engine import StepEntry


def random_ids(vocab, n, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def run_whole(rt, ids):
    """The whole request in one step; logits at every position [T, V]."""
    s = rt.engine.take_slot()
    try:
        return rt.step([StepEntry(s, ids, list(range(len(ids))))]).cpu()
    finally:
        rt.engine.free_slot(s)


def run_tail(rt, ids, tail=32):
    """All but the last ``tail`` tokens in one step, then one token a step."""
    tail = min(tail, len(ids) - 1)
    head = len(ids) - tail
    s = rt.engine.take_slot()
    try:
        out = [rt.step([StepEntry(s, ids[:head], list(range(head)))])]
        for t in ids[head:]:
            out.append(rt.step([StepEntry(s, [t], [0])]))
        return torch.cat(out).cpu()
    finally:
        rt.engine.free_slot(s)


def run_batches(rt, requests, batch_size, prompt_lens):
    """Batches one after another.  A batch's requests start together with the
    first ``prompt_lens[i]`` tokens of each, then go on by one token a step;
    a request leaves (and gives its slot back) when its tokens run out.
    Returns request index -> logits at every position, and the slots used."""
    out = {}
    slots_used = []
    for b0 in range(0, len(requests), batch_size):
        idx = list(range(b0, min(b0 + batch_size, len(requests))))
        slots = {i: rt.engine.take_slot() for i in idx}
        slots_used.append([slots[i] for i in idx])
        fed = {i: min(prompt_lens[i], len(requests[i])) for i in idx}
        logits = rt.step([StepEntry(slots[i], requests[i][:fed[i]], list(range(fed[i]))) for i in idx])
        pieces = {i: [] for i in idx}
        o = 0
        for i in idx:
            pieces[i].append(logits[o:o + fed[i]].cpu())
            o += fed[i]
        live = list(idx)
        while True:
            for i in [i for i in live if fed[i] >= len(requests[i])]:
                rt.engine.free_slot(slots[i])
                live.remove(i)
            if not live:
                break
            logits = rt.step([StepEntry(slots[i], [requests[i][fed[i]]], [0]) for i in live])
            for r, i in enumerate(live):
                pieces[i].append(logits[r:r + 1].cpu())
                fed[i] += 1
        for i in idx:
            out[i] = torch.cat(pieces[i])
    return out, slots_used
