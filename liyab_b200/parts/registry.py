"""Registries from a part's `kind` to the class that implements it.

One registry per role: norms, position encodings, mixers, feed-forwards and
block arrangements.  The model builder looks every part of every layer up here
by the `kind` in its spec, so a new kind is added by registering a class, with
no change to the model, the step function or the cache manager.

Interfaces (what a registered class must offer):

  every part     __init__(spec, params, runtime): `params` maps the part's own
                 parameter names to tensors; `runtime` gives dtype and device.
                 classmethod parameters(spec) -> {name: (shape, kind)} with kind
                 "matrix", "table" or "vector".
  norm           forward(ctx, x, out, n_rows, rows=None): out[r] = norm(x[rows[r]]).
  position       embed(ctx, table, scale, x): x[t] = table[token t] * scale (+ its encoding).
  mixer          kv_need() -> KvNeed | None, state_need() -> StateNeed | None,
                 forward(ctx, h, x, unit): adds the mixer's output for the step's
                 tokens to the residual stream x; `unit` says which cache unit to
                 read and whether to write it.
  feed-forward   forward(ctx, h, x): adds its output to the residual stream x.
  arrangement    __init__(spec, parts, runtime); forward(ctx, x, unit): runs
                 norms, mixer and feed-forward around the residual stream.
"""
from __future__ import annotations

from typing import Callable, Dict, Generic, TypeVar

from ..status import unsupported

T = TypeVar("T")


class PartRegistry(Generic[T]):
    def __init__(self, role: str):
        self.role = role
        self._kinds: Dict[str, T] = {}

    def register(self, kind: str) -> Callable[[T], T]:
        def deco(cls: T) -> T:
            self._kinds[kind] = cls
            return cls
        return deco

    def get(self, kind: str) -> T:
        if kind not in self._kinds:
            raise unsupported(f"no {self.role} of kind {kind!r} is registered; registered: "
                              f"{', '.join(sorted(self._kinds)) or 'none'}")
        return self._kinds[kind]

    def kinds(self):
        return sorted(self._kinds)


NORMS: PartRegistry = PartRegistry("norm")
POSITIONS: PartRegistry = PartRegistry("position encoding")
MIXERS: PartRegistry = PartRegistry("mixer")
FEED_FORWARDS: PartRegistry = PartRegistry("feed-forward")
ARRANGEMENTS: PartRegistry = PartRegistry("block arrangement")
