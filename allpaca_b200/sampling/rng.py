"""Uniform numbers for sampling that depend only on (seed, request's step).

The reference seeds one generator per request from ``params.seed``, else the engine's
seed, else ``0xA110ACA`` (crates/allpaca-core/src/sampling.rs:5-8) and draws one number per
sampled token (:55-58).  Here the number for the n-th sampled token of a request is a
hash of ``(seed, n)``, so it does not depend on what else is in a batch or on whether the
request was preempted and recomputed.
"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, index: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32)."""
    h = _splitmix64(_splitmix64(seed & _MASK) ^ ((index * 0xD1B54A32D192ED03) & _MASK))
    return (h >> 40) / float(1 << 24)
