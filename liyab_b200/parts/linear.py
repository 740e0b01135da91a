"""A matrix with an optional bias: y = act(x W^T + b) (+ residual).

The matrix is kept [out, in] in the compute type and the bias in float32.  The
product runs on the tensor-core kernel when the operands are bfloat16 and the
sizes suit it, else on the 32-bit units; both fuse bias, activation and the
residual sum into their epilogue, in the reference's order (bias, activation,
residual: src/core/transformer.cpp:111-118, 4903-4912, 5526-5532).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import ops
from ..status import invalid_model


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], name: str = "linear"):
        if weight.dim() != 2:
            raise invalid_model(f"{name}: weight must be a matrix, got shape {tuple(weight.shape)}")
        if bias is not None and tuple(bias.shape) != (weight.shape[0],):
            raise invalid_model(f"{name}: bias has shape {tuple(bias.shape)}, expected [{weight.shape[0]}]")
        self.weight = weight
        self.bias = bias
        self.name = name
        self.out_features, self.in_features = weight.shape

    @staticmethod
    def parameters(out_features: int, in_features: int, bias: bool) -> Dict[str, Tuple[tuple, str]]:
        p = {"weight": ((out_features, in_features), "matrix")}
        if bias:
            p["bias"] = ((out_features,), "vector")
        return p

    def forward(self, a: torch.Tensor, out: torch.Tensor, m: int, activation: str = "none",
                residual: Optional[torch.Tensor] = None, workspace=None) -> torch.Tensor:
        """out[:m] = act(a[:m] @ W^T + b) + residual[:m]; `workspace` lends scratch for products of few tokens."""
        return ops.linear(a, self.weight, self.bias, out, m, activation, residual, workspace)
