"""Sampling options, the deterministic generator and the device sampler."""
from .params import RECENT_WINDOW, SamplingParams
from .rng import XorShift64Star

__all__ = ["RECENT_WINDOW", "SamplingParams", "XorShift64Star"]
