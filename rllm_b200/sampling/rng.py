"""Counter-based uniform numbers: u = f(seed, token index). The draw for a request's n-th
generated token depends on nothing else, so it is the same however the request was batched,
chunked or preempted. (The reference seeds a per-sequence SmallRng,
src/engine/mod.rs:284-287, whose state advances with every draw.)"""
from __future__ import annotations

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, index: int) -> float:
    """A float in [0, 1) with 24 random bits, from (seed, index)."""
    z = _splitmix64(_splitmix64(seed & _MASK) ^ ((index * 0xD1342543DE82EF95) & _MASK))
    return (z >> 40) / float(1 << 24)
