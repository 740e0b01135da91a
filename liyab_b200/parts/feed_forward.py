"""The dense, ungated feed-forward: down(act(up(x))).

Reference: dense_ffn, ungated branch (src/core/transformer.cpp:4903-4913) with the
activations of :125-142.  Bias and activation ride in the first product's
epilogue, bias and the residual sum in the second's.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.spec import DenseFeedForwardSpec
from ..status import unsupported
from .base import Runtime, StepContext
from .linear import Linear
from .registry import FEED_FORWARDS

_ACTIVATIONS = ("gelu_tanh", "gelu_erf", "none")


@FEED_FORWARDS.register("dense")
class DenseFeedForward:
    def __init__(self, spec: DenseFeedForwardSpec, params: Dict[str, torch.Tensor], runtime: Runtime):
        if spec.activation not in _ACTIVATIONS:
            raise unsupported(f"feed-forward activation {spec.activation!r} is not supported; "
                              f"supported: {', '.join(_ACTIVATIONS)}")
        self.spec = spec
        self.runtime = runtime
        self.up = Linear(params["up.weight"], params.get("up.bias"), "feed_forward.up")
        self.down = Linear(params["down.weight"], params.get("down.bias"), "feed_forward.down")

    @classmethod
    def parameters(cls, spec: DenseFeedForwardSpec) -> Dict[str, Tuple[tuple, str]]:
        p = {}
        for k, v in Linear.parameters(spec.inner, spec.hidden, spec.bias).items():
            p["up." + k] = v
        for k, v in Linear.parameters(spec.hidden, spec.inner, spec.bias).items():
            p["down." + k] = v
        return p

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor) -> None:
        T = ctx.n_tokens
        inner = ctx.workspace.get("ff.inner", T, self.spec.inner, self.runtime.dtype)
        self.up.forward(h, inner, T, activation=self.spec.activation, workspace=ctx.workspace)
        self.down.forward(inner, x, T, residual=x, workspace=ctx.workspace)
