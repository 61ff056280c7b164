"""Uniform draws for sampling.  A draw depends on (seed, request index, index
of the sampled token) only, so a request's output does not depend on what else
is in its batch or on the slot it got.  (The reference seeds one generator per
call, src/engine.rs:362.)"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _mix(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, request: int, index: int) -> float:
    """A float in [0, 1) with 24 random bits (exact in float32)."""
    z = _mix(seed & _MASK)
    z = _mix(z ^ ((request * 0xD6E8FEB86659FD93) & _MASK))
    z = _mix(z ^ ((index * 0xA0761D6478BD642F) & _MASK))
    return (z >> 40) / float(1 << 24)
