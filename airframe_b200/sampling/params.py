"""Sampling options, with the reference's names, defaults and meanings
(``SamplingParams``, ``src/runtime/gpu.rs:25-47``)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    """``temperature`` < 1e-7 means greedy.  ``repetition_penalty`` acts on the
    last 64 tokens of the sequence (``logit > 0 ? / p : * p``).
    ``stop_token_ids`` takes the place of the reference's ``extra_stop_tokens``
    (strings that encode to one token): the library starts at token ids.
    ``ignore_eos`` keeps generating through the model's own end tokens."""
    max_tokens: int = 64
    temperature: float = 0.8
    top_p: float = 0.95
    repetition_penalty: float = 1.1
    seed: int = 42
    stop_token_ids: list = field(default_factory=list)
    ignore_eos: bool = False

    def check(self) -> None:
        if self.max_tokens < 0:
            raise ValueError(f"max_tokens must be >= 0, got {self.max_tokens}")
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.repetition_penalty <= 0:
            raise ValueError(f"repetition_penalty must be > 0, got {self.repetition_penalty}")

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-7


RECENT_WINDOW = 64   # tokens the repetition penalty looks back on (crates/airframe_observe/src/isf.rs:395-396)
