"""Host side of per-request sampling: the request's parameters and its per-token random seeds.

Mirrors the names of the reference's nanoserve/sampling.py (SamplingParams :26-43, mix_seed :46-51) so callers can pass
the same objects to `LLMEngine.add_request(..., sampling=...)`. Greedy parameters (temperature 0 or top_k 1) use the
argmax the step's graph computes anyway; any other request's row is redrawn by the sampling kernel inside the same
graph (csrc/sampling.cu: temperature, top-k, top-p, Gumbel-max). The integer part of the contract is bit-exact with the
reference: draw n of a request uses the seed mix_seed(request seed, n), so a request's text does not depend on its batch
neighbours or on a preemption + recompute. The random stream behind a seed is the kernel's own (counter-based), not the
host generator's, so single draws differ from the reference's while the kept set and the distribution are the same.
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


def sample(logits, params: list, seeds: list[int], steps: list[int], return_survivors: bool = False):
    """logits [B, V] on the device -> one token per row, with the reference's signature (nanoserve/sampling.py:54).
    Row i uses params[i] (None = greedy) and draws from mix_seed(seeds[i], steps[i]). Greedy rows are the argmax kernel's
    tokens (lowest index on ties); the others are redrawn by the sampling kernel. return_survivors=True also returns,
    per row, (smallest surviving value of logits / temperature, number of survivors) for the sampled rows (None for
    greedy rows)."""
    import numpy as np
    import torch
    from nanoserve_b200 import _lib
    _lib.require_cuda(logits)
    assert logits.dim() == 2 and logits.stride(1) == 1
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int64, device=logits.device)
    code = _lib.dtype_code(logits.dtype)
    _lib.call("ns_argmax_rows", logits.data_ptr(), logits.stride(0), B, V, out.data_ptr(), None, None, code, _lib.stream_ptr())
    rows = [i for i, p in enumerate(params) if p is not None and not p.greedy]
    thr = kept = None
    if rows:
        host = np.zeros(8 * B, dtype=np.int32)
        as_f32 = host.view(np.float32)
        for i in rows:
            seed = mix_seed(seeds[i], steps[i])
            as_f32[8 * i], as_f32[8 * i + 1] = params[i].temperature, params[i].top_p
            host[8 * i + 2], host[8 * i + 3] = params[i].top_k, 1
            host[8 * i + 4:8 * i + 6] = np.array([seed & 0xFFFFFFFF, seed >> 32], dtype=np.uint32).view(np.int32)
        dev = torch.from_numpy(host).to(logits.device)
        if return_survivors:
            thr = torch.zeros(B, dtype=torch.float32, device=logits.device)
            kept = torch.zeros(B, dtype=torch.int32, device=logits.device)
        _lib.call("ns_sample_rows", logits.data_ptr(), logits.stride(0), B, V, dev.data_ptr(), out.data_ptr(), None, None,
                  _lib.ptr(thr), _lib.ptr(kept), code, _lib.stream_ptr())
    tokens = out.tolist()
    if not return_survivors:
        return tokens
    info = [None] * B
    if rows:
        t, k = thr.tolist(), kept.tolist()
        for i in rows:
            info[i] = (t[i], k[i])
    return tokens, info
