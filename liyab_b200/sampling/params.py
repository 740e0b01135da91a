"""Sampling options and the engine's random draws.

Names, meanings and defaults are the reference's `SamplingParams`
(include/liyab/types.h:215-222; C mirror include/liyab/liyab_c_api.h:128-135):
temperature <= 0 is greedy, top_k <= 0 and top_p >= 1 switch those cuts off, seed
0 picks a random seed.  `ignore_eos` is an addition for benchmarks, where a fixed
number of tokens must be generated.

The reference draws from std::mt19937_64 (src/core/sampling.cpp:9-10, 66-69); a
sampler on the GPU cannot share that stream, so draws here are counter-based:
uniform(seed, stream, counter) is SplitMix64 of a key built from the three, top
53 bits scaled by 2^-53.  A request's n-th draw is therefore the same number
whatever the batch it is drawn in, and after a preemption too.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

from ..status import invalid_argument

_MASK = 0xFFFFFFFFFFFFFFFF


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8      # <= 0 selects greedy decoding
    top_k: int = 40               # <= 0 disables
    top_p: float = 0.95           # >= 1 disables
    seed: int = 0                 # 0 picks a random seed
    max_tokens: int = 256
    ignore_eos: bool = False

    def validate(self) -> None:
        if self.max_tokens <= 0:
            raise invalid_argument(f"max_tokens must be positive (got {self.max_tokens})")
        if not (self.temperature == self.temperature) or not (self.top_p == self.top_p):
            raise invalid_argument("temperature and top_p must be numbers")
        if self.top_p <= 0 and self.temperature > 0:
            raise invalid_argument(f"top_p must be positive (got {self.top_p})")
        if self.seed < 0:
            raise invalid_argument(f"seed must not be negative (got {self.seed})")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    def resolved_seed(self) -> int:
        """The seed itself, or a random one when it is 0."""
        if self.seed != 0:
            return self.seed
        return int.from_bytes(os.urandom(8), "little") | 1


def uniform_draw(seed: int, stream: int, counter: int) -> float:
    """The `counter`-th draw in [0, 1) of stream `stream` under `seed`."""
    x = (seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + counter * 0x8CB92BA72F3D8DD7) & _MASK
    z = (x + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 11) * (1.0 / 9007199254740992.0)
