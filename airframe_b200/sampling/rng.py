"""The reference's deterministic generator: xorshift64* with state seed + 1,
u = (x * 0x2545F4914F6CDD1D >> 40) / 2^24 (``src/runtime/gpu.rs:50-62``)."""
from __future__ import annotations

_MASK = (1 << 64) - 1


class XorShift64Star:
    def __init__(self, seed: int):
        self.state = (seed + 1) & _MASK

    def next_f32(self) -> float:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & _MASK
        s ^= s >> 27
        self.state = s
        return float(((s * 0x2545F4914F6CDD1D) & _MASK) >> 40) / 16777216.0
