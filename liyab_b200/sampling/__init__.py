"""Sampling options and the engine's random draws.

Names, meanings and defaults are the reference's `SamplingParams`
(include/liyab/types.h:215-222; C mirror include/liyab/liyab_c_api.h:128-135):
temperature <= 0 is greedy, top_k <= 0 and top_p >= 1 switch those cuts off, seed
0 picks a random seed.  `ignore_eos` is an addition for benchmarks, where a fixed
number of tokens must be generated.  Draws are counter-based (see the library's
sampling.h): `uniform_draw(seed, stream, counter)`.
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import _capi


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8      # <= 0 selects greedy decoding
    top_k: int = 40               # <= 0 disables
    top_p: float = 0.95           # >= 1 disables
    seed: int = 0                 # 0 picks a random seed
    max_tokens: int = 256
    ignore_eos: bool = False

    def to_c(self) -> "_capi.SamplingParamsC":
        return _capi.SamplingParamsC(float(self.temperature), int(self.top_k), float(self.top_p), int(self.seed),
                                     int(self.max_tokens), 1 if self.ignore_eos else 0)


def uniform_draw(seed: int, stream: int, counter: int) -> float:
    """The `counter`-th draw in [0, 1) of stream `stream` under `seed`."""
    return float(_capi.lib().lb_uniform_draw(seed, stream, counter))


__all__ = ["SamplingParams", "uniform_draw"]
