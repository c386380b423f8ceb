"""RMS norm with a weight offset: y = x * rsqrt(mean(x^2) + eps) * (offset + w).

Reference: ``src/backend/bindless/sh_layer_v1.wgsl:426-451``,
``src/backend/bindless/sh_rmsnorm.wgsl:69-93``; post norms fused with the
residual sum as x + norm(a) instead of the reference's add-then-correct
(``sh_layer_v1.wgsl:811-813,834-849``).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import Norm, register_part
from .linear import PartialSums


@register_part("norm", "rms_norm")
class RmsNorm(Norm):
    """Parameters: ``weight`` (tensor name), ``size``, ``eps``, ``weight_offset``."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.name = self.param("weight")
        self.size = int(self.param("size"))
        self.eps = float(self.param("eps"))
        self.offset = float(self.param("weight_offset"))
        self.w = None

    def weight_decls(self):
        return [WeightDecl(self.name, (self.size,), "norm")]

    def load(self, weights):
        # statistics and the (offset + w) factor are 32-bit in both precisions
        self.w = weights[self.name].to(torch.float32).contiguous()

    def decode_bytes(self, lens) -> int:
        return 4 * self.size

    def forward(self, x, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty(n, self.size, dtype=out_dtype, device=x.device)
        kernels.rmsnorm(y, x, self.w, self.eps, self.offset, rows)
        return y

    def add_normed(self, x, a, then=None, out_dtype=None):
        n_parts = 1
        if isinstance(a, PartialSums):
            n_parts, a = a.parts.shape[0], a.parts
        if then is not None and not (isinstance(then, RmsNorm) and then.offset == self.offset):
            kernels.add_rmsnorm(x, a, self.w, self.eps, self.offset, n_parts=n_parts)
            return then.forward(x, out_dtype)
        y = None
        if then is not None:
            y = torch.empty(x.shape[0], self.size, dtype=out_dtype, device=x.device)
        kernels.add_rmsnorm(x, a, self.w, self.eps, self.offset, y=y,
                            w_next=then.w if then is not None else None,
                            eps_next=then.eps if then is not None else 0.0, n_parts=n_parts)
        return y
