"""Gated feed-forward: f = W_down (act(W_gate x) * (W_up x)).

Reference: ``src/backend/bindless/sh_layer_v1.wgsl:1024-1070`` (gate and up),
``:1079`` (tanh-GELU), ``:1082`` (SiLU), ``:1104-1140`` (down).  The reference
picks the activation by a proxy (softcap > 0); here it is a parameter.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import WeightDecl
from .base import FeedForward, register_part
from .linear import gated_linear, linear_split


@register_part("feed_forward", "gated_mlp")
class GatedMlp(FeedForward):
    """Parameters: ``hidden_size``, ``intermediate_size``, ``activation``
    (``gelu_tanh`` or ``silu``), ``gate_weight``/``up_weight``/``down_weight``."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.inter = int(self.param("intermediate_size"))
        self.activation = self.param("activation")
        if self.activation not in kernels.ACTIVATIONS:
            raise ConfigError(f"gated_mlp: unknown activation '{self.activation}' "
                              f"(known: {sorted(kernels.ACTIVATIONS)})")
        self.names = [self.param(k) for k in ("gate_weight", "up_weight", "down_weight")]
        self.w_gu = None
        self.interleaved = False
        self.w_down = None

    def weight_decls(self):
        g, u, d = self.names
        return [WeightDecl(g, (self.inter, self.hidden)), WeightDecl(u, (self.inter, self.hidden)),
                WeightDecl(d, (self.hidden, self.inter))]

    def load(self, weights):
        g, u, d = self.names
        dt = self.ctx.compute_dtype
        wg, wu = weights[g].to(dt), weights[u].to(dt)
        # bfloat16 with a K the tensor-core product takes: gate and up rows interleaved per
        # tile, activation in the product's epilogue; else [gate; up] and a kernel of its own
        self.interleaved = dt == torch.bfloat16 and self.hidden % 8 == 0
        self.w_gu = (kernels.interleave_gate_up(wg, wu) if self.interleaved
                     else torch.cat([wg, wu], dim=0).contiguous())
        self.w_down = weights[d].to(dt).contiguous()

    def decode_bytes(self, lens) -> int:
        return 3 * self.hidden * self.inter * (4 if self.ctx.compute_dtype == torch.float32 else 2)

    def prefill_flops(self, lens) -> int:
        return 2 * sum(lens) * 3 * self.hidden * self.inter

    def forward(self, x, batch):
        h = gated_linear(x, self.w_gu, self.inter, self.activation, self.interleaved)
        return linear_split(h, self.w_down)
