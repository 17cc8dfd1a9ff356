"""Host side of per-request sampling: the request's parameters and its per-token random seeds.

Mirrors the names of the reference's nanoserve/sampling.py (SamplingParams :26-43, mix_seed :46-51) so callers can pass
the same objects to `LLMEngine.add_request(..., sampling=...)`. Greedy parameters (temperature 0 or top_k 1) run on
this engine's argmax kernel; anything else is refused by the engine (`NotImplementedError`): the device-side
temperature / top-k / top-p / Gumbel-max kernel is not built. What IS fixed here, bit for bit, is the integer part of
the contract a future kernel has to honour: draw n of a request uses the seed mix_seed(request seed, n), so a request's
text does not depend on its batch neighbours or on a preemption + recompute.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

_U64 = (1 << 64) - 1
# splitmix64 (Steele, Lea, Flood 2014): increment, then two xor-shift-multiply rounds and a final xor-shift
_GOLDEN_GAMMA = 0x9E3779B97F4A7C15
_ROUNDS = ((30, 0xBF58476D1CE4E5B9), (27, 0x94D049BB133111EB))


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 = greedy; top_p 1 = off; top_k 0 = off; seed None = the engine draws one per request."""
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int | None = None

    def __post_init__(self):
        if math.isnan(self.temperature) or self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if math.isnan(self.top_p) or self.top_p <= 0 or self.top_p > 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0 or self.top_k == 1


def mix_seed(seed: int, step: int) -> int:
    """63-bit generator seed of a request's draw number `step`: one splitmix64 output whose state is
    seed * gamma + step + 1 (mod 2^64), with the top bit cleared (generator seeds are signed 64-bit)."""
    z = (seed * _GOLDEN_GAMMA + step + 1) & _U64
    for shift, mult in _ROUNDS:
        z = ((z ^ (z >> shift)) * mult) & _U64
    return (z ^ (z >> 31)) & (_U64 >> 1)
