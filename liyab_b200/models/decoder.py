"""A decoder put together from a `ModelSpec`: embedding, position encoding, the
layers in their run order, final norm and the head.

Nothing here is particular to an architecture: the spec says which parts every
layer has, the registries say which class implements each kind, and the
parameters arrive as {path: tensor} with paths made of the part's place
("layers.3.mixer.qkv.weight").  The forward pass follows the reference's
(embed -> add_positions -> every block -> final norm and head on the wanted rows
only: src/core/transformer.cpp:6589-6769).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import ops
from ..cache.pages import KvNeed, StateNeed
from ..config.spec import LayerSpec, ModelSpec
from ..parts.base import CacheUnit, Runtime, StepContext
from ..parts.block import LayerParts
from ..parts.registry import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from ..status import invalid_model


def _sub(params: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    n = len(prefix)
    return {k[n:]: v for k, v in params.items() if k.startswith(prefix)}


def parameter_shapes(spec: ModelSpec) -> Dict[str, Tuple[tuple, str]]:
    """Every parameter the model needs: {path: (shape, kind)}, from the parts' own declarations."""
    out: Dict[str, Tuple[tuple, str]] = {
        "embedding.weight": ((spec.embedding.vocab_size, spec.embedding.size), "table")}
    for name, s in POSITIONS.get(spec.position.kind).parameters(spec.position).items():
        out["position." + name] = s
    for i, layer in enumerate(spec.layers):
        for role, registry, part in (("mixer_norm", NORMS, layer.mixer_norm), ("mixer", MIXERS, layer.mixer),
                                     ("ff_norm", NORMS, layer.ff_norm),
                                     ("feed_forward", FEED_FORWARDS, layer.feed_forward)):
            for name, s in registry.get(part.kind).parameters(part).items():
                out[f"layers.{i}.{role}.{name}"] = s
    for name, s in NORMS.get(spec.final_norm.kind).parameters(spec.final_norm).items():
        out["final_norm." + name] = s
    if not spec.head.tied:
        out["head.weight"] = ((spec.head.vocab_size, spec.head.size), "matrix")
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, params: Mapping[str, torch.Tensor], runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        want = parameter_shapes(spec)
        missing = [f"missing parameter '{k}'" for k in want if k not in params]
        wrong = [f"parameter '{k}' has shape {list(params[k].shape)}, expected {list(s)}"
                 for k, (s, _) in want.items() if k in params and tuple(params[k].shape) != tuple(s)]
        if missing or wrong:
            raise invalid_model("; ".join(missing + wrong))
        self._params = {k: params[k] for k in want}
        self.embedding = params["embedding.weight"]
        self.position = POSITIONS.get(spec.position.kind)(spec.position, _sub(params, "position."), runtime)
        self.layers = [self._build_layer(layer, _sub(params, f"layers.{i}.")) for i, layer in enumerate(spec.layers)]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, _sub(params, "final_norm."), runtime)
        self.head_weight = self.embedding if spec.head.tied else params["head.weight"]
        self.head_bias = params.get("head.bias") if spec.head.bias else None
        n = len(spec.run_order)
        for i, entry in enumerate(spec.run_order):
            if not (0 <= entry.layer < len(self.layers)) or not (0 <= entry.cache < n):
                raise invalid_model(f"run order entry {i} names layer {entry.layer} / cache {entry.cache} out of range")
            if entry.cache != i and spec.run_order[entry.cache].cache != entry.cache:
                raise invalid_model(f"run order entry {i} reads the cache of entry {entry.cache}, which keeps none")
            if entry.cache > i:
                raise invalid_model(f"run order entry {i} reads the cache of a later entry {entry.cache}")

    def _build_layer(self, layer: LayerSpec, params: Dict[str, torch.Tensor]):
        rt = self.runtime
        parts = LayerParts(
            mixer_norm=NORMS.get(layer.mixer_norm.kind)(layer.mixer_norm, _sub(params, "mixer_norm."), rt),
            mixer=MIXERS.get(layer.mixer.kind)(layer.mixer, _sub(params, "mixer."), rt),
            ff_norm=NORMS.get(layer.ff_norm.kind)(layer.ff_norm, _sub(params, "ff_norm."), rt),
            feed_forward=FEED_FORWARDS.get(layer.feed_forward.kind)(layer.feed_forward, _sub(params, "feed_forward."), rt))
        return ARRANGEMENTS.get(layer.arrangement)(layer, parts, rt)

    # -- what the cache manager has to provide ---------------------------------

    def kv_needs(self) -> Dict[int, KvNeed]:
        """Cache units (run-order entries that write keys and values) and their needs."""
        out = {}
        for i, entry in enumerate(self.spec.run_order):
            if entry.cache == i:
                need = self.layers[entry.layer].parts.mixer.kv_need()
                if need is not None:
                    out[i] = need
        for i, entry in enumerate(self.spec.run_order):
            if entry.cache != i:
                mine = self.layers[entry.layer].parts.mixer.kv_need()
                if mine is not None and out.get(entry.cache) != mine:
                    raise invalid_model(f"run order entry {i} reads the cache of entry {entry.cache}, whose keys and "
                                        f"values have another shape or window")
        return out

    def state_needs(self) -> Dict[int, StateNeed]:
        out = {}
        for i, entry in enumerate(self.spec.run_order):
            need = self.layers[entry.layer].parts.mixer.state_need()
            if need is not None:
                out[i] = need
        return out

    @property
    def max_positions(self) -> int:
        return min(self.spec.max_positions, self.position.max_positions)

    def weight_bytes(self) -> int:
        """Bytes of all parameters, a tied table counted once."""
        seen, total = set(), 0
        for t in self._params.values():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    # -- the forward pass of one step -------------------------------------------

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Runs the step's tokens; returns logits [R, vocab] float32 at ctx.logit_rows (None if R = 0)."""
        T, width = ctx.n_tokens, self.spec.hidden
        x = ctx.workspace.get("residual", T, width, torch.float32)
        self.position.embed(ctx, self.embedding, self.spec.embedding.scale, x)
        for i, entry in enumerate(self.spec.run_order):
            self.layers[entry.layer].forward(ctx, x, CacheUnit(read=entry.cache, write=entry.cache == i))
        R = ctx.n_logit_rows
        if R == 0:
            return None
        y = ctx.workspace.get("head.normed", R, width, self.runtime.dtype)
        self.final_norm.forward(ctx, x, y, R, rows=ctx.logit_rows)
        logits = ctx.workspace.get("logits", R, self.spec.vocab_size, torch.float32)
        ops.linear(y, self.head_weight, self.head_bias, logits, R, workspace=ctx.workspace)
        return logits[:R]
