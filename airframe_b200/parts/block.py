"""Arrangements of a layer's parts around the float32 residual stream.

``sandwich``: x += post(mixer(pre(x))); x += post(ff(pre(x))) - norms before
and after both halves (reference order
``src/backend/bindless/pipeline/inference.rs:1096-1251``, net effect
x + norm(a) of ``sh_layer_v1.wgsl:834-849,869-884``).
``prenorm``: x += mixer(pre(x)); x += ff(pre(x)).
"""
from __future__ import annotations

from .. import kernels
from .base import Block, register_part
from .linear import PartialSums


def _dense(a):
    return a.parts if isinstance(a, PartialSums) else a


@register_part("block", "sandwich")
class SandwichBlock(Block):
    roles = ("pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward")

    def forward(self, x, batch, view, normed=None, next_pre=None):
        """Updates x in place.  ``normed`` may carry pre_mixer(x) made by the
        previous layer's last kernel; ``next_pre`` is the next layer's first
        norm, whose output is then returned (made by this layer's last kernel)."""
        n = self.norms
        dt = self.ctx.compute_dtype
        h = normed if normed is not None else n["pre_mixer"].forward(x, dt)
        a = self.mixer.forward(h, batch, view)
        h = n["post_mixer"].add_normed(x, a, then=n["pre_feed_forward"], out_dtype=dt)
        f = self.feed_forward.forward(h, batch)
        return n["post_feed_forward"].add_normed(x, f, then=next_pre, out_dtype=dt)

    def first_norm(self):
        return self.norms["pre_mixer"]


@register_part("block", "prenorm")
class PreNormBlock(Block):
    roles = ("pre_mixer", "pre_feed_forward")

    def forward(self, x, batch, view, normed=None, next_pre=None):
        n = self.norms
        dt = self.ctx.compute_dtype
        h = normed if normed is not None else n["pre_mixer"].forward(x, dt)
        kernels.add_(x, _dense(self.mixer.forward(h, batch, view)))
        kernels.add_(x, _dense(self.feed_forward.forward(n["pre_feed_forward"].forward(x, dt), batch)))
        return next_pre.forward(x, dt) if next_pre is not None else None

    def first_norm(self):
        return self.norms["pre_mixer"]
