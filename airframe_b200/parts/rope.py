"""Rotary position encoding, applied to q and k before the cache write so
that cached keys are final (a ring of rows then works with plain dot products).

angle = position * theta^(-2p / rotary_dim), computed in 32 bits from a table
of inverse frequencies made in 64 bits.  Reference: ``theta_p`` of
``src/backend/bindless/preflight.rs:87-90``; rotation
``src/ops/reference/rope.rs:156-196`` (absolute) and
``src/backend/bindless/sh_layer_v1.wgsl:706-725`` (relative, at score time).
The reference pairs adjacent elements (GGUF row order); ``pairing`` selects
``half`` (element i with i + rotary_dim/2, Hugging Face row order) or ``adjacent``.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import ConfigError
from .base import PositionEncoding, register_part


@register_part("position", "rope")
class Rope(PositionEncoding):
    """Parameters: ``theta``, ``rotary_dim``, ``pairing``."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.theta = float(self.param("theta"))
        self.rotary_dim = int(self.param("rotary_dim"))
        self.pairing = self.param("pairing")
        if self.rotary_dim % 2 or self.rotary_dim < 0:
            raise ConfigError(f"rope: rotary_dim {self.rotary_dim} must be even")
        if self.pairing not in kernels.PAIRINGS:
            raise ConfigError(f"rope: unknown pairing '{self.pairing}'")
        p = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        inv = torch.tensor(self.theta, dtype=torch.float64) ** (-2.0 * p / max(self.rotary_dim, 1))
        self._inv_freq_host = inv.to(torch.float32)
        self.inv_freq = None

    def load(self, weights):
        self.inv_freq = self._inv_freq_host.to(self.ctx.device)

    def rotates_half_pairs(self, hd):
        return self.pairing == "half" and self.rotary_dim == hd

    def rotary_table(self, batch, hd):
        key = ("rope_table", self.theta, self.rotary_dim)
        if key not in batch.aux:
            batch.aux[key] = kernels.rope_table(batch.positions, self.inv_freq)
        return batch.aux[key]

    def encode(self, qkv, batch, nq, nkv, hd, parts=None):
        if self.rotary_dim > hd:
            raise ConfigError(f"rope: rotary_dim {self.rotary_dim} exceeds head_dim {hd}")
        kernels.rope_cache_write(qkv, batch.positions, self.inv_freq, nq, nkv, hd, self.rotary_dim,
                                 self.pairing, parts=parts)

    def encode_and_store(self, qkv, batch, nq, nkv, hd, kv, parts=None) -> bool:
        """The rotation and the mixer's cache store as one kernel (the rotated
        k rows are what the cache keeps)."""
        if self.rotary_dim > hd:
            raise ConfigError(f"rope: rotary_dim {self.rotary_dim} exceeds head_dim {hd}")
        # many rows (a prompt): the cosines and sines come from the step's table, made once for all layers
        table = None
        if (qkv.shape[0] >= kernels.ROPE_TABLE_ROWS and parts is None and qkv.dtype == torch.bfloat16
                and self.rotates_half_pairs(hd)):
            table = self.rotary_table(batch, hd)
        kernels.rope_cache_write(qkv, batch.positions, self.inv_freq, nq, nkv, hd, self.rotary_dim,
                                 self.pairing, seq_of_token=batch.seq_of_token, slots=batch.slots,
                                 len_after=batch.len_after, kcache=kv.k, vcache=kv.v,
                                 page_table=kv.page_table, ring_rows=kv.ring_rows, parts=parts, table=table)
        return True


@register_part("position", "none")
class NoPosition(PositionEncoding):
    """No encoding (the base class's behaviour under a name)."""
    graph_safe = True
