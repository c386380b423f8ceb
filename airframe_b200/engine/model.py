"""A model built from a :class:`~airframe_b200.config.ModelSpec`: embedding,
layers (each a block of parts), the schedule in which they run, final norm and
head.  Knows no architecture.

Reference: the layer loop of
``src/backend/bindless/pipeline/inference.rs:1061-1337`` and the final norm and
head at ``:873-916,1383-1480``; there the logits are made for the last token
only, here at every wanted row.
"""
from __future__ import annotations

import torch

from ..config.base import ModelSpec
from ..parts import BuildContext, build_part


def _build_layers(spec: ModelSpec, ctx: BuildContext):
    blocks = []
    for layer in spec.layers:
        mixer = build_part("mixer", layer.mixer, ctx)
        ffn = build_part("feed_forward", layer.feed_forward, ctx)
        norms = {role: build_part("norm", ns, ctx) for role, ns in layer.norms.items()}
        blocks.append(build_part("block", layer.block, ctx, mixer=mixer, feed_forward=ffn, norms=norms))
    return blocks


class Model:
    def __init__(self, spec: ModelSpec, compute_dtype=torch.bfloat16, device="cuda:0"):
        spec.validate()
        self.spec = spec
        self.ctx = BuildContext(compute_dtype=compute_dtype, device=torch.device(device))
        self.embedding = build_part("embedding", spec.embedding, self.ctx)
        self.blocks = _build_layers(spec, self.ctx)
        self.final_norm = build_part("norm", spec.final_norm, self.ctx)
        self.head = build_part("head", spec.head, self.ctx)
        self.loaded = False

    # ------------------------------------------------------------------ weights

    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def weight_decls(self) -> list:
        seen, out = set(), []
        for p in self.parts():
            for d in p.weight_decls():
                if d.name in seen:
                    # a tensor used twice (tied head): it must be required if any user requires it
                    for o in out:
                        if o.name == d.name and not d.optional:
                            o.optional = False
                    continue
                seen.add(d.name)
                out.append(d)
        return out

    def load(self, weights: dict) -> None:
        for p in self.parts():
            p.load(weights)
        self.loaded = True

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model can be captured into a CUDA graph."""
        return all(p.graph_safe for p in self.parts())

    # ------------------------------------------------------------------ cache

    def cache_needs(self) -> list:
        """Per schedule entry: (KVNeed | None, StateNeed | None, cache_from | None)."""
        out = []
        for e in self.spec.schedule:
            m = self.blocks[e.layer].mixer
            out.append((m.kv_need(), m.state_need(), e.cache_from))
        return out

    # ------------------------------------------------------------------ what a step costs

    def decode_bytes(self, lens) -> int:
        """Bytes a decode step of sequences that hold ``lens`` tokens has to read:
        every weight it uses once and the cache of the live sequences (the parts
        answer for themselves; a run that reads another run's cache reads it again)."""
        total = self.embedding.decode_bytes(lens) + self.final_norm.decode_bytes(lens) + self.head.decode_bytes(lens)
        return total + sum(self.blocks[e.layer].decode_bytes(lens) for e in self.spec.schedule)

    def prefill_flops(self, lens, n_logits: int) -> int:
        """Floating-point operations of a prefill of prompts of ``lens`` tokens with ``n_logits`` rows of logits."""
        total = sum(self.blocks[e.layer].prefill_flops(lens) for e in self.spec.schedule)
        flops = getattr(self.head, "logits_flops", None)
        return total + (flops(n_logits) if flops is not None else 0)

    def score_flops(self, lens) -> int:
        """The part of :meth:`prefill_flops` that the mixers spend on scores (those that say so)."""
        total = 0
        for e in self.spec.schedule:
            f = getattr(self.blocks[e.layer].mixer, "score_flops", None)
            total += f(lens) if f is not None else 0
        return total

    # ------------------------------------------------------------------ forward

    def hidden(self, batch, cache, probe=None) -> torch.Tensor:
        """The float32 residual stream [T, H] after all scheduled runs.
        ``probe`` (a :class:`~airframe_b200.engine.probe.LayerProbe`) is shown
        the stream after the embedding and after every run."""
        batch.aux.clear()       # (a captured step's tables are made inside the capture, not left from the run before)
        x = self.embedding.forward(batch.tokens)
        if probe is not None:
            probe.after(-1, -1, x, batch)
        sched = self.spec.schedule
        normed = None
        for i, e in enumerate(sched):
            blk = self.blocks[e.layer]
            nxt = self.blocks[sched[i + 1].layer].first_norm() if i + 1 < len(sched) else None
            normed = blk.forward(x, batch, cache.views[i], normed=normed, next_pre=nxt)
            if probe is not None:
                probe.after(i, e.layer, x, batch)
        return x

    def logits(self, x, want_rows) -> torch.Tensor:
        """float32 logits [R, V] at the wanted rows of the residual stream."""
        y = self.final_norm.forward(x, self.ctx.compute_dtype, rows=want_rows)
        return self.head.forward(y)

    def greedy_tokens(self, x, want_rows) -> torch.Tensor:
        """int32 [R]: the arg-max token at the wanted rows (a head that can, finds
        it without writing the logits)."""
        y = self.final_norm.forward(x, self.ctx.compute_dtype, rows=want_rows)
        best = getattr(self.head, "forward_argmax", None)
        if best is not None:
            return best(y)
        from .. import kernels
        logits = self.head.forward(y)
        tokens = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        kernels.sample(logits, tokens, 0.0, 1.0, 1.0)
        return tokens

    def forward(self, batch, cache, probe=None, greedy: bool = False):
        """Logits at the wanted rows, or with ``greedy`` their arg-max tokens."""
        x = self.hidden(batch, cache, probe)
        if batch.want_rows is None:
            return None
        return self.greedy_tokens(x, batch.want_rows) if greedy else self.logits(x, batch.want_rows)


def declared_weights(spec: ModelSpec) -> list:
    """The tensors a model of ``spec`` reads (no device is touched)."""
    return Model(spec, torch.bfloat16, "cpu").weight_decls()
