"""Sampling options, the deterministic generator and the device sampler."""
from .params import RECENT_WINDOW, SamplingParams
from .rng import XorShift64Star
from .sampler import Sampler, SequenceSamplingState

__all__ = ["RECENT_WINDOW", "SamplingParams", "XorShift64Star", "Sampler", "SequenceSamplingState"]
