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

import os

from ..config.base import ModelSpec
from ..parts import BuildContext, NotFusable, build_part


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
        # opt-in (it is slower than the chain of kernels at the sizes measured so far): decode steps of
        # few tokens run as one kernel when every layer can say its step in phases
        self.fuse_decode = os.environ.get("AIRFRAME_B200_FUSE_DECODE", "0") == "1"
        self._programs: dict = {}
        self.not_fused_because = None

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

    # ------------------------------------------------------------------ forward

    def layer_program(self, batch, cache):
        """The one-kernel form of this decode step's layers, or None (then
        ``not_fused_because`` says why).  Programs are kept per step shape."""
        if (not self.fuse_decode or batch.is_prefill or self.ctx.compute_dtype != torch.bfloat16
                or self.ctx.device.type != "cuda"):
            return None
        from .. import kernels
        from .layer_program import LayerProgram
        if batch.n_tokens > kernels.decode_layers_limits()["tokens"]:
            return None
        # the number of splits of the keys depends on the longest sequence: steps of one shape share a program
        sched = self.spec.schedule
        needs = {cache.views[i].kv.need for i in range(len(sched)) if cache.views[i].kv is not None}
        shape = tuple(sorted(kernels.attn_decode_splits(batch.n_tokens, n.num_kv_heads, batch.max_len_after,
                                                        n.window or 0) for n in needs))
        # (a token of the cache's own stands for it: an id could be used again once a cache is gone, and a
        # program points into its cache's memory)
        key = (batch.n_tokens, cache.__dict__.setdefault("_program_key", object()), shape)
        if key not in self._programs:
            prog = None
            try:
                b = LayerProgram(batch.n_tokens, self.spec.hidden_size, self.ctx.device, batch.max_len_after)
                first = self.blocks[sched[0].layer].first_norm()
                if first is None:
                    raise NotFusable("the first layer does not start with a norm")
                b.norm(0, None, first)
                for i, e in enumerate(sched):
                    nxt = self.blocks[sched[i + 1].layer].first_norm() if i + 1 < len(sched) else None
                    self.blocks[e.layer].emit_decode(b, cache.views[i], nxt)
                prog = b.finish()
            except NotFusable as why:
                self.not_fused_because = str(why)
            self._programs[key] = prog
        return self._programs[key]

    def hidden(self, batch, cache) -> torch.Tensor:
        """The float32 residual stream [T, H] after all scheduled runs."""
        x = self.embedding.forward(batch.tokens)
        prog = self.layer_program(batch, cache)
        if prog is not None:
            prog.run(x, batch)
            return x
        sched = self.spec.schedule
        normed = None
        for i, e in enumerate(sched):
            blk = self.blocks[e.layer]
            nxt = self.blocks[sched[i + 1].layer].first_norm() if i + 1 < len(sched) else None
            normed = blk.forward(x, batch, cache.views[i], normed=normed, next_pre=nxt)
        return x

    def logits(self, x, want_rows) -> torch.Tensor:
        """float32 logits [R, V] at the wanted rows of the residual stream."""
        y = self.final_norm.forward(x, self.ctx.compute_dtype, rows=want_rows)
        return self.head.forward(y)

    def forward(self, batch, cache):
        x = self.hidden(batch, cache)
        if batch.want_rows is None:
            return None
        return self.logits(x, batch.want_rows)


def declared_weights(spec: ModelSpec) -> list:
    """The tensors a model of ``spec`` reads (no device is touched)."""
    return Model(spec, torch.bfloat16, "cpu").weight_decls()
