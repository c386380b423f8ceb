"""The parts a layer is put together from, and their registry.

Five categories: ``norm``, ``position``, ``mixer``, ``feed_forward`` and
``block`` (the arrangement of the other four in a layer), plus ``embedding``
and ``head`` at the model's ends.  A part is built from the parameters of its
:class:`~airframe_b200.config.PartSpec` alone: it takes every size and
constant from there and does not know which model it is in.  New kinds are
added with :func:`register_part`; nothing else has to change.

Reference: the parameterised operations of ``src/ops`` behind
``OpDispatcher`` (``src/ops/dispatch.rs:11-199``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.base import ConfigError, PartSpec

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_REGISTRY: dict = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str):
    """Class decorator: make ``kind`` buildable in ``category``."""
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category '{category}' (known: {CATEGORIES})")

    def deco(cls):
        _REGISTRY[category][kind] = cls
        cls.category = category
        cls.kind = kind
        return cls

    return deco


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY[category].pop(kind, None)


def known_parts(category: str) -> list:
    return sorted(_REGISTRY[category])


@dataclass
class BuildContext:
    """What every part is told besides its own parameters."""
    compute_dtype: torch.dtype      # bfloat16 or float32: activations, matrices, cache
    device: torch.device


def build_part(category: str, spec: PartSpec, ctx: BuildContext, **children):
    kinds = _REGISTRY[category]
    if spec.kind not in kinds:
        raise ConfigError(f"no {category} part of kind '{spec.kind}' (known: {sorted(kinds)})")
    return kinds[spec.kind](dict(spec.params), ctx, **children)


# --------------------------------------------------------------------------
# what the cache is asked for
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class KVNeed:
    """Keys and values per token.  ``window`` None: all of them are kept;
    otherwise the last ``window`` rows (a ring)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size: one tensor of ``shape`` per sequence,
    zero when the sequence starts."""
    shape: tuple
    dtype: str = "float32"


# --------------------------------------------------------------------------
# interfaces
# --------------------------------------------------------------------------

class Part:
    """Base of all parts.

    ``weight_decls`` lists the tensors the part reads from the model folder,
    ``load`` receives name -> tensor (already on the device, bfloat16, or
    float32 for tensors stored so or on the 32-bit path) and keeps what it
    needs in the layout its kernels want.
    """
    category = ""
    kind = ""
    # True when ``forward`` only launches kernels on the current stream (no
    # host reads of device data, no synchronisation), so that a decode step can
    # be captured into a CUDA graph.  A model is captured only if all its parts say so.
    graph_safe = False

    def __init__(self, params: dict, ctx: BuildContext):
        self.params = params
        self.ctx = ctx

    def weight_decls(self) -> list:
        return []

    def load(self, weights: dict) -> None:
        pass

    # ---- what a step costs, for measurement (rooflines): every part answers for itself

    def decode_bytes(self, lens) -> int:
        """Bytes that one decode step of sequences holding ``lens`` tokens has to
        read for this part: its weights once, and what it keeps per sequence."""
        return 0

    def prefill_flops(self, lens) -> int:
        """Floating-point operations of this part in a prefill of prompts of ``lens`` tokens."""
        return 0

    def param(self, key: str):
        if key not in self.params:
            raise ConfigError(f"{self.category} part '{self.kind}' needs parameter '{key}'")
        return self.params[key]


class Norm(Part):
    """x is the float32 residual stream [rows, H]."""

    def forward(self, x, out_dtype, rows=None):
        """norm(x) (of the listed rows when ``rows`` is given) in ``out_dtype``."""
        raise NotImplementedError

    def add_normed(self, x, a, then=None, out_dtype=None):
        """x += norm(a) in place (32-bit sum).  With ``then`` (another norm),
        also returns then.forward(x) in ``out_dtype``."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How a mixer's queries and keys learn their positions.  An encoding may
    rewrite the q and k rows (:meth:`encode`, e.g. a rotation), bias the
    scores (:meth:`score_slopes`), or both; storing keys and values in the
    cache is the mixer's business, not the encoding's."""

    def encode(self, qkv, batch, nq: int, nkv: int, hd: int, parts=None) -> None:
        """Encode positions into the q and k heads of the packed rows ``qkv``
        ([T, (nq + 2 nkv) hd], in place).  ``parts`` (float32 [S, T, width]),
        when given, are split-K partial sums of the rows: their sum is written
        to ``qkv`` first.  The default encodes nothing."""
        if parts is not None:
            from .. import kernels
            kernels.sum_parts(qkv, parts, batch, nq, nkv, hd)

    def score_slopes(self, nq: int):
        """None, or float32 [nq] on the device: slope[h] * (key position -
        query position) is added to head h's scores after scale and softcap."""
        return None

    def rotates_half_pairs(self, hd: int) -> bool:
        """True when :meth:`encode` is nothing but the rotation of the pairs
        (i, i + hd / 2) of every q and k head by an angle per token and pair,
        and :meth:`rotary_table` gives its cosines and sines: a mixer may then
        rotate in the epilogue of its projection instead of calling :meth:`encode`."""
        return False

    def rotary_table(self, batch, hd: int):
        """float32 [T, hd / 2, 2] of (cos, sin) for every token of the step and
        pair of the head (see :meth:`rotates_half_pairs`).  Made once per pass
        (kept in ``batch.aux``) for all layers that rotate alike."""
        raise NotImplementedError

    def encode_and_store(self, qkv, batch, nq: int, nkv: int, hd: int, kv, parts=None) -> bool:
        """Optional fast path: :meth:`encode` and the mixer's cache store in one
        kernel.  Returns False when the encoding has none (the mixer then calls
        :meth:`encode` and stores by itself)."""
        return False


class Mixer(Part):
    """Mixes information between the positions of a sequence."""

    def kv_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x, batch, view):
        """x [T, H] in the compute dtype (normalised) -> [T, H] in the compute
        dtype, or a :class:`~airframe_b200.parts.linear.PartialSums` of it.  ``batch`` is the :class:`~airframe_b200.engine.batch.StepBatch`,
        ``view`` the layer's :class:`~airframe_b200.cache.LayerCacheView`.

        A captured decode step is padded to a fixed number of rows: padding
        rows carry ``batch.slots[seq] == -1`` (token 0, position 0, length 0).
        A mixer must not read or write cache pages or per-sequence state for
        them (they have none) and may leave anything in their output rows;
        a ``graph_safe`` mixer meets them, others never do."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, batch):
        """x [T, H] compute dtype -> [T, H] compute dtype."""
        raise NotImplementedError


class Block(Part):
    """The arrangement of norms, mixer and feed-forward around the residual stream."""

    roles: tuple = ()

    def __init__(self, params, ctx, mixer: Mixer, feed_forward: FeedForward, norms: dict):
        super().__init__(params, ctx)
        missing = [r for r in self.roles if r not in norms]
        if missing:
            raise ConfigError(f"block '{self.kind}' needs norms for {missing}")
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def children(self):
        return [self.mixer, self.feed_forward, *self.norms.values()]

    @property
    def graph_safe(self):
        return all(c.graph_safe for c in self.children())

    def weight_decls(self):
        return [d for c in self.children() for d in c.weight_decls()]

    def load(self, weights):
        for c in self.children():
            c.load(weights)

    def first_norm(self):
        """The norm this block applies to x first, or None.  The layer before
        may compute it in its last kernel and pass the result as ``normed``."""
        return None

    def decode_bytes(self, lens) -> int:
        return sum(c.decode_bytes(lens) for c in self.children())

    def prefill_flops(self, lens) -> int:
        return sum(c.prefill_flops(lens) for c in self.children())

    def forward(self, x, batch, view, normed=None, next_pre=None):
        """Run the layer on the float32 residual stream x [T, H] in place.
        Returns next_pre.forward(x) in the compute dtype when ``next_pre`` (the
        next layer's first norm) is given, else None."""
        raise NotImplementedError
