"""Sampling options and the per-request random stream.

Names and meanings follow the reference's ``SamplingParams``
(src/engine/sampler.ts:3-16): ``temperature`` 0 is greedy; ``top_k`` 0 and
``top_p`` 1.0 switch those filters off; ``repetition_penalty`` 1.0 is off;
``seed`` makes the draws reproducible.  Defaults are the command line's
(src/index.ts:130-215: temperature 0, top-k 0, top-p 1.0), not the class's.

The reference seeds one xorshift generator per sampler object (:37-51), so what a
request draws depends on what was sampled before it.  Here the n-th draw of a
request is a pure function of (seed, n): a request draws the same numbers
whatever else is in the batch and also after it was preempted and recomputed.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, n: int) -> float:
    """The n-th uniform number in [0, 1) of the stream ``seed`` (24 bits, exact in float32)."""
    z = _splitmix64(_splitmix64(seed & _MASK) ^ ((n * 0xD1342543DE82EF95) & _MASK))
    return (z >> 40) / float(1 << 24)


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    max_tokens: int = 100
    stop_token_ids: Tuple[int, ...] = ()     # besides the model's eos ids
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.seed is None:
            self.seed = int.from_bytes(os.urandom(8), "little")
        self.stop_token_ids = tuple(int(t) for t in self.stop_token_ids)

    @property
    def greedy(self) -> bool:
        return self.temperature == 0
