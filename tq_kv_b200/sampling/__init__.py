"""Sampling: parameters, per-request random draws, the device sampler."""
from .params import GenerationParams
from .rng import uniform
from .sampler import Sampler

__all__ = ["GenerationParams", "Sampler", "uniform"]
