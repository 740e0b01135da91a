"""LayerNorm with 32-bit statistics (reference: src/core/transformer.cpp:77-106)."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import ops
from ..config.spec import NormSpec
from .base import Runtime, StepContext
from .registry import NORMS


@NORMS.register("layernorm")
class LayerNorm:
    def __init__(self, spec: NormSpec, params: Dict[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.weight = params["weight"]
        self.bias = params.get("bias")

    @classmethod
    def parameters(cls, spec: NormSpec) -> Dict[str, Tuple[tuple, str]]:
        p = {"weight": ((spec.size,), "vector")}
        if spec.bias:
            p["bias"] = ((spec.size,), "vector")
        return p

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor, n_rows: int,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.layernorm(x, self.weight, self.bias, self.spec.eps, out, n_rows, rows)
