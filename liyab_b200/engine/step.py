"""The one step function: a batch of (request, its next tokens) in, logits at
the wanted places out.

A step may hold portions of prompts beside single decoded tokens, cut anywhere.
It runs only the tokens it is given, as one flat batch, against what earlier
steps left in the cache, and then makes every request longer by what it brought.
This is the reference's `forward_batch` (src/core/transformer.h:731-764,
src/core/transformer.cpp:6589-6769): items of 1..n tokens appended at each
sequence's own n_past, pages mapped for every item before any compute so that a
failure leaves every position as it was (:6652-6654), n_past advanced after all
blocks ran (:6726-6735), logits only for the rows asked for (:6739-6767).
Refusals follow :6596-6624: an empty batch or item, a token id outside the
vocabulary, a request named twice; plus an unknown request and a sequence that
would pass the model's positions (ContextFull, :2791-2808).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache.pages import CacheManager, OutOfPages
from ..models.decoder import DecoderModel
from ..parts.base import GroupView, StepContext, Workspace
from ..status import context_full, invalid_argument
from .fused_decode import FusedDecodeStack


@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepOutput:
    logits: Optional[torch.Tensor]                 # [R, vocab] float32 on the device; valid until the next step
    rows: List[Tuple[Hashable, int]] = field(default_factory=list)   # (request, index among its tokens) per row


class _DecodeGraph:
    """A captured decode step for a fixed number of requests: its layout buffer, graph and logits view."""

    def __init__(self, dev: torch.Tensor, generation: int):
        self.dev = dev
        self.generation = generation
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None


class Stepper:
    """Owns the step's device-side layout buffers, the workspace and the captured decode graphs.

    A step whose entries all bring one token and want its logits (a decode step)
    always has the same launches for a given number of requests; with
    `cuda_graphs` it is captured once per that number and replayed afterwards, its
    layout arrays (tokens, positions, block tables, slots) rewritten in place
    before each replay.  The kernels and the cache are the same either way.
    """

    def __init__(self, model: DecoderModel, cache: CacheManager, max_step_tokens: int = 0, cuda_graphs: bool = False,
                 max_positions: int = 0, fused_decode: bool = True):
        self.model = model
        self.cache = cache
        self.device = model.runtime.device
        self.max_positions = min(max_positions or model.max_positions, model.max_positions)
        self.workspace = Workspace(self.device)
        if max_step_tokens:
            self.workspace.reserve_rows(max_step_tokens)
        # Pinned int32 staging, two buffers used in turn: a buffer is rewritten only
        # after the copy that last read it has finished on the device.
        self._host: List[Optional[torch.Tensor]] = [None, None]
        self._copied: List[Optional[torch.cuda.Event]] = [None, None]
        self._dev: Optional[torch.Tensor] = None
        self._turn = 0
        self.cuda_graphs = cuda_graphs
        # Decode steps of a few tokens go to the one-kernel path where the model is made of standard parts.
        self.fused = FusedDecodeStack.try_build(model, cache) if fused_decode else None
        self.fused_steps = 0
        self._graphs: dict = {}
        self.graph_launches: dict = {}       # kernels in the captured step, by number of requests
        self.steps = 0
        self.graph_steps = 0
        self.tokens_run = 0

    # -- validation (no side effects) -------------------------------------------

    def validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise invalid_argument("a step needs at least one entry")
        seen = set()
        vocab = self.model.spec.vocab_size
        limit = self.max_positions
        for e in entries:
            if e.request in seen:
                raise invalid_argument(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if not self.cache.is_open(e.request):
                raise invalid_argument(f"request {e.request!r} is not open")
            n = len(e.tokens)
            if n == 0:
                raise invalid_argument(f"request {e.request!r} brings no tokens")
            toks = np.asarray(e.tokens)
            if toks.min() < 0 or toks.max() >= vocab:
                raise invalid_argument(f"request {e.request!r} has a token id outside [0, {vocab})")
            if self.cache.length(e.request) + n > limit:
                raise context_full(f"request {e.request!r} would reach {self.cache.length(e.request) + n} tokens; "
                                   f"the model has {limit} positions")
            for w in e.want:
                if not (0 <= w < n):
                    raise invalid_argument(f"request {e.request!r} wants logits at {w}, outside its {n} tokens")

    # -- the step -----------------------------------------------------------------

    def step(self, entries: Sequence[StepEntry]) -> StepOutput:
        self.validate(entries)
        cache = self.cache
        wants = {e.request: len(e.tokens) for e in entries}
        if not cache.can_reserve(wants):
            raise OutOfPages(f"the step's {sum(wants.values())} tokens of {len(wants)} request(s) do not fit the free "
                             f"pages {cache.free_pages()}")
        for e in entries:
            cache.reserve(e.request, len(e.tokens))
        decode = all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        if decode and self.fused is not None and self.fused.accepts(len(entries)):
            ctx, rows = self._layout(entries)
            logits = self.fused.run(ctx)
            self.fused_steps += 1
        elif decode and self.cuda_graphs:
            logits, rows = self._graph_step(entries)
        else:
            ctx, rows = self._layout(entries)
            logits = self.model.forward(ctx)
        for e in entries:
            cache.commit(e.request, len(e.tokens))
        self.steps += 1
        self.tokens_run += sum(wants.values())
        return StepOutput(logits=logits, rows=rows)

    def _graph_step(self, entries: Sequence[StepEntry]):
        S = len(entries)
        g = self._graphs.get(S)
        if g is None or g.generation != self.workspace.generation:
            # First decode step of this size (or buffers moved since): run it eagerly on a
            # buffer of its own so every scratch buffer exists, then capture the same launches.
            widths = [(self.max_positions + grp.page_size - 1) // grp.page_size for grp in self.cache.groups]
            total = self._layout_size(S, S, S, widths)
            g = _DecodeGraph(torch.empty(total, dtype=torch.int32, device=self.device), -1)
            ctx, rows = self._layout(entries, static=g)
            self.model.forward(ctx)
            torch.cuda.current_stream().synchronize()
            g.generation = self.workspace.generation
            graph = torch.cuda.CUDAGraph()
            before = ops.LAUNCHES
            with torch.cuda.graph(graph):
                g.logits = self.model.forward(ctx)
            self.graph_launches[S] = ops.LAUNCHES - before
            if g.generation != self.workspace.generation:
                raise RuntimeError("a scratch buffer was created while a decode step was being captured")
            g.graph = graph
            self._graphs[S] = g
        else:
            _, rows = self._layout(entries, static=g)
        g.graph.replay()
        self.graph_steps += 1
        return g.logits, rows

    @staticmethod
    def _layout_size(S: int, T: int, R: int, widths: Sequence[int]) -> int:
        sizes = [T, T, T, S + 1, S, S, R] + [S * w for w in widths] + [T for _ in widths]
        return sum((n + 3) // 4 * 4 for n in sizes)

    def _layout(self, entries: Sequence[StepEntry], static: Optional[_DecodeGraph] = None
                ) -> Tuple[StepContext, List[Tuple[Hashable, int]]]:
        cache = self.cache
        S = len(entries)
        q_len = np.array([len(e.tokens) for e in entries], dtype=np.int64)
        n_past = np.array([cache.length(e.request) for e in entries], dtype=np.int64)
        q_start = np.zeros(S + 1, dtype=np.int64)
        np.cumsum(q_len, out=q_start[1:])
        T = int(q_start[-1])
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        tok_seq = np.repeat(np.arange(S, dtype=np.int32), q_len)
        positions = (np.arange(T, dtype=np.int64) - np.repeat(q_start[:-1], q_len) + np.repeat(n_past, q_len)).astype(np.int32)
        requests = [e.request for e in entries]
        rows: List[Tuple[Hashable, int]] = []
        logit_rows: List[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                rows.append((e.request, int(w)))
                logit_rows.append(int(q_start[i]) + int(w))
        state_slots = np.array([cache.state_slot(r) for r in requests], dtype=np.int32)
        G = len(cache.groups)
        fixed = None
        if static is not None:      # widths that never change, so the captured launches stay valid
            fixed = [(self.max_positions + grp.page_size - 1) // grp.page_size for grp in cache.groups]
        tables = [cache.block_table(g, requests, width=fixed[g] if fixed else None) for g in range(G)]
        slots = [np.concatenate([cache.slot_mapping(g, e.request, int(n_past[i]), int(q_len[i]))
                                 for i, e in enumerate(entries)]) for g in range(G)]
        # One staging buffer, one copy to the device; views are carved out of it.
        pieces = [tokens, positions, tok_seq, q_start.astype(np.int32), n_past.astype(np.int32), state_slots,
                  np.asarray(logit_rows, dtype=np.int32)] + [t.reshape(-1) for t in tables] + slots
        offsets, total = [], 0
        for p in pieces:
            offsets.append(total)
            total += (p.size + 3) // 4 * 4           # keep every view 16-byte aligned
        turn = self._turn = 1 - self._turn
        if static is not None:
            dev = static.dev
            assert dev.numel() == total
        else:
            if self._dev is None or self._dev.numel() < total:
                self._dev = torch.empty(max(total, 4096), dtype=torch.int32, device=self.device)
            dev = self._dev
        if self._host[turn] is None or self._host[turn].numel() < total:
            self._host[turn] = torch.empty(max(total, 4096), dtype=torch.int32).pin_memory()
            self._copied[turn] = torch.cuda.Event()
        else:
            self._copied[turn].synchronize()
        host = self._host[turn].numpy()
        for p, o in zip(pieces, offsets):
            host[o:o + p.size] = p
        dev[:total].copy_(self._host[turn][:total], non_blocking=True)
        self._copied[turn].record()

        def view(i: int) -> torch.Tensor:
            return dev[offsets[i]:offsets[i] + pieces[i].size]

        groups = [GroupView(group=cache.groups[g], block_table=view(7 + g).view(S, tables[g].shape[1]),
                            slot_mapping=view(7 + G + g)) for g in range(G)]
        ctx = StepContext(
            runtime=self.model.runtime, workspace=self.workspace, cache=cache, n_tokens=T, n_seq=S,
            tokens=view(0), positions=view(1), tok_seq=view(2), q_start=view(3), n_past=view(4), state_slots=view(5),
            logit_rows=view(6), n_logit_rows=len(logit_rows), groups=groups, requests=requests,
            host_q_start=q_start.tolist(), host_n_past=n_past.tolist(), max_q_len=int(q_len.max()),
            max_kv_len=int((n_past + q_len).max()), decode_only=bool((q_len == 1).all()))
        return ctx, rows
