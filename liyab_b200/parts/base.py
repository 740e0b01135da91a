"""What every part sees of a step: the batch's layout on the device, the cache
views of its unit, and scratch buffers.

A step is a flat batch of T tokens from S requests.  Request i contributes
q_len[i] consecutive tokens starting at row q_start[i]; its first token sits at
position n_past[i] of its sequence.  The reference resolves the same facts per
segment (`Segment{first, n, kv, n_past}` with `pos_of` and `row_of`:
src/core/transformer.h:890-916); here they are arrays on the device, built once
per step, that every kernel indexes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.pages import CacheManager, KvGroup


@dataclass(frozen=True)
class Runtime:
    """Element type of activations and matrices, and the device."""
    dtype: torch.dtype
    device: torch.device

    @property
    def is_reduced(self) -> bool:
        return self.dtype != torch.float32


@dataclass(frozen=True)
class CacheUnit:
    """Which cache unit a run of a layer reads, and whether it writes it."""
    read: int
    write: bool


class Workspace:
    """Named scratch buffers that persist across steps.

    A buffer is created at first use and grows when a step needs more rows, so a
    steady state allocates nothing; `reserve_rows` sizes everything up front,
    which keeps addresses fixed for captured CUDA graphs.
    """

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[tuple, torch.Tensor] = {}
        self.min_rows = 0
        self.generation = 0          # grows whenever a buffer is created or moved (captured graphs check it)

    def reserve_rows(self, rows: int) -> None:
        self.min_rows = max(self.min_rows, rows)

    def get(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, cols, dtype)        # layers of different sizes get buffers of their own
        buf = self._buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            cap = max(rows, self.min_rows, 1)
            buf = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf

    def flat(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """A one-dimensional scratch buffer of at least `numel` elements (not subject to the row floor).
        `zero`: filled with zeros when created (for counters that kernels leave at zero)."""
        key = (name, "flat", dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < numel:
            cap = 1 << max(10, (max(numel, 1) - 1).bit_length())
            buf = (torch.zeros if zero else torch.empty)(cap, dtype=dtype, device=self.device)
            self._buffers[key] = buf
            self.generation += 1
        return buf

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class GroupView:
    """One cache group as a step sees it."""
    group: KvGroup
    block_table: torch.Tensor        # int32 [S, width] on the device
    slot_mapping: torch.Tensor       # int32 [T] on the device


@dataclass
class StepContext:
    runtime: Runtime
    workspace: Workspace
    cache: CacheManager
    n_tokens: int
    n_seq: int
    # device, int32
    tokens: torch.Tensor             # [T]
    positions: torch.Tensor          # [T] absolute position of each token
    tok_seq: torch.Tensor            # [T] row of the token's request in this step
    q_start: torch.Tensor            # [S + 1] first row of each request
    n_past: torch.Tensor             # [S] tokens each request held before the step
    state_slots: torch.Tensor        # [S] the requests' state slots
    logit_rows: torch.Tensor         # [R] rows whose logits are wanted
    n_logit_rows: int
    groups: List[GroupView]
    # host copies of the same layout
    requests: Sequence[Hashable] = ()
    host_q_start: Sequence[int] = ()
    host_n_past: Sequence[int] = ()
    max_q_len: int = 0
    max_kv_len: int = 0
    decode_only: bool = False
    max_positions: int = 0           # the longest sequence the engine serves (fixes split counts and table widths)
    extras: Dict[str, object] = field(default_factory=dict)

    def kv(self, unit: int) -> Tuple[torch.Tensor, GroupView]:
        """The unit's pages [page, K|V, kv_head, slot, head_dim] and its group's view."""
        gi = self.cache.group_of_unit[unit]
        view = self.groups[gi]
        return view.group.unit_storage(unit), view

    def state(self, unit: int) -> torch.Tensor:
        """The unit's state storage [slot, ...]; index it with `state_slots`."""
        return self.cache.states.storage[unit]
