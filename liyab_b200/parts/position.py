"""Position encodings that act where the tokens are embedded.

`learned_absolute` adds a row of a learned table for each token's position
(reference: add_positions, src/core/transformer.cpp:2791-2808); the gather of the
embedding row and this sum are one kernel.  `none` embeds only.  An encoding
that acts inside the mixer instead (a rotation of queries and keys, a bias on
scores) registers here with an `embed` that embeds only, and offers the mixer
what it needs through the step context's positions.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .. import ops
from ..config.spec import PositionSpec
from .base import Runtime, StepContext
from .registry import POSITIONS


@POSITIONS.register("learned_absolute")
class LearnedAbsolutePosition:
    def __init__(self, spec: PositionSpec, params: Dict[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.table = params["weight"]

    @classmethod
    def parameters(cls, spec: PositionSpec) -> Dict[str, Tuple[tuple, str]]:
        return {"weight": ((spec.max_positions, spec.size), "table")}

    @property
    def max_positions(self) -> int:
        return self.spec.max_positions

    def embed(self, ctx: StepContext, table: torch.Tensor, scale: float, x: torch.Tensor) -> torch.Tensor:
        return ops.embed_positions(ctx.tokens, ctx.positions, table, self.table, x, scale)


@POSITIONS.register("none")
class NoPosition:
    def __init__(self, spec, params, runtime: Runtime):
        self.spec = spec

    @classmethod
    def parameters(cls, spec) -> Dict[str, Tuple[tuple, str]]:
        return {}

    @property
    def max_positions(self) -> int:
        return getattr(self.spec, "max_positions", 0) or (1 << 30)

    def embed(self, ctx: StepContext, table: torch.Tensor, scale: float, x: torch.Tensor) -> torch.Tensor:
        return ops.embed_positions(ctx.tokens, ctx.positions, table, None, x, scale)
