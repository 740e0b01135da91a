"""How a layer's parts are arranged around the residual stream.

`pre_norm`: x += mixer(norm(x)); x += feed_forward(norm(x)), the reference's
run_block for this architecture (src/core/transformer.cpp:5574-5577, 5633-5637,
5647, 5663-5666, 5684-5685, 5692).  The residual stream stays float32 in every
mode; the normalised input of a part is in the compute type.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..config.spec import LayerSpec
from .base import CacheUnit, Runtime, StepContext
from .registry import ARRANGEMENTS


@dataclass
class LayerParts:
    mixer_norm: Any
    mixer: Any
    ff_norm: Any
    feed_forward: Any


@ARRANGEMENTS.register("pre_norm")
class PreNormBlock:
    def __init__(self, spec: LayerSpec, parts: LayerParts, runtime: Runtime):
        self.spec = spec
        self.parts = parts
        self.runtime = runtime

    def forward(self, ctx: StepContext, x: torch.Tensor, unit: CacheUnit) -> None:
        p, T = self.parts, ctx.n_tokens
        h = ctx.workspace.get("block.normed", T, x.shape[1], self.runtime.dtype)
        p.mixer_norm.forward(ctx, x, h, T)
        p.mixer.forward(ctx, h, x, unit)
        p.ff_norm.forward(ctx, x, h, T)
        p.feed_forward.forward(ctx, h, x)
