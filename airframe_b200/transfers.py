"""Counters of the bytes that cross between host and device on the product
path (token ids and bookkeeping in, sampled tokens out).  Every place that
copies calls :func:`count_h2d` or :func:`count_d2h` with the tensor it sends."""
from __future__ import annotations

_h2d = 0
_d2h = 0


def count_h2d(t) -> None:
    global _h2d
    _h2d += t.numel() * t.element_size()


def count_d2h(t) -> None:
    global _d2h
    _d2h += t.numel() * t.element_size()


def snapshot() -> tuple:
    """(bytes host -> device, bytes device -> host) since the process began."""
    return _h2d, _d2h
