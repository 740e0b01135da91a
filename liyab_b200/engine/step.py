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
class DeviceTokens:
    """Tokens of a step that are still on the device: entry i's (single) token is source[index[i]] where
    index[i] >= 0; other entries bring their tokens from the host as usual."""
    source: torch.Tensor          # int32 on the device, e.g. the ids the previous step sampled
    index: Sequence[int]


@dataclass
class StepOutput:
    logits: Optional[torch.Tensor]                 # [R, vocab] float32 on the device; valid until the next step
    rows: List[Tuple[Hashable, int]] = field(default_factory=list)   # (request, index among its tokens) per row


class _DecodeGraph:
    """A captured step of one shape: its layout buffer, graph and logits view."""

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
        self._seen: dict = {}                # how often a shape without a graph has come up
        self.graph_launches: dict = {}       # kernels in the captured step, by number of requests
        self._device_tokens: Optional[DeviceTokens] = None
        self.steps = 0
        self.graph_steps = 0
        self.tokens_run = 0

    # -- validation (no side effects) -------------------------------------------

    def validate(self, entries: Sequence[StepEntry]):
        """Checks a step before anything is touched; returns (rows, q_len, tokens) as arrays."""
        if not entries:
            raise invalid_argument("a step needs at least one entry")
        cache = self.cache
        S = len(entries)
        try:
            rows = cache.rows([e.request for e in entries])
        except KeyError as e:
            raise invalid_argument(f"request {e.args[0]!r} is not open") from None
        if len(np.unique(rows)) != S:
            seen = set()
            for e in entries:
                if e.request in seen:
                    raise invalid_argument(f"request {e.request!r} appears twice in one step")
                seen.add(e.request)
        q_len = np.fromiter((len(e.tokens) for e in entries), dtype=np.int64, count=S)
        if (q_len == 0).any():
            raise invalid_argument(f"request {entries[int(np.argmin(q_len))].request!r} brings no tokens")
        if S > 1 and int(q_len.max()) == 1:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int64, count=S)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if tokens.min() < 0 or tokens.max() >= self.model.spec.vocab_size:
            bad = next(e for e in entries if min(e.tokens) < 0 or max(e.tokens) >= self.model.spec.vocab_size)
            raise invalid_argument(f"request {bad.request!r} has a token id outside [0, {self.model.spec.vocab_size})")
        over = cache.length_arr[rows] + q_len > self.max_positions
        if over.any():
            i = int(np.argmax(over))
            raise context_full(f"request {entries[i].request!r} would reach {int(cache.length_arr[rows[i]] + q_len[i])} "
                               f"tokens; the model has {self.max_positions} positions")
        for e, n in zip(entries, q_len):
            for w in e.want:
                if not (0 <= w < n):
                    raise invalid_argument(f"request {e.request!r} wants logits at {w}, outside its {int(n)} tokens")
        return rows, q_len, tokens.astype(np.int32)

    # -- the step -----------------------------------------------------------------

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[DeviceTokens] = None) -> StepOutput:
        rows, q_len, tokens = self.validate(entries)
        self._device_tokens = device_tokens
        cache = self.cache
        cache.reserve_rows(rows, q_len)          # all or nothing: raises OutOfPages and takes no page
        decode = int(q_len.max()) == 1 and all(len(e.want) == 1 for e in entries)
        if decode and self.fused is not None and self.fused.accepts(len(entries)):
            ctx, out_rows = self._layout(entries, rows, q_len, tokens)
            logits = self.fused.run(ctx)
            self.fused_steps += 1
        elif self.cuda_graphs and (decode or self._worth_capturing(entries, q_len)):
            logits, out_rows = self._graph_step(entries, rows, q_len, tokens)
        else:
            ctx, out_rows = self._layout(entries, rows, q_len, tokens)
            logits = self.model.forward(ctx)
        cache.commit_rows(rows, q_len)
        self.steps += 1
        self.tokens_run += int(q_len.sum())
        return StepOutput(logits=logits, rows=out_rows)

    def _shape_key(self, entries: Sequence[StepEntry], q_len: np.ndarray):
        S, T = len(entries), int(q_len.sum())
        return S, T, sum(len(e.want) for e in entries), ((int(q_len.max()) + 63) // 64 * 64 if T != S else 1)

    def _worth_capturing(self, entries: Sequence[StepEntry], q_len: np.ndarray) -> bool:
        """A step with prompt portions is captured when its shape comes up for the third time (capturing costs
        several eager steps) and the scratch buffers are sized so that they will not move."""
        if int(q_len.sum()) > self.workspace.min_rows:
            return False
        key = self._shape_key(entries, q_len)
        if key in self._graphs:
            return True
        self._seen[key] = self._seen.get(key, 0) + 1
        if len(self._seen) > 4096:
            self._seen.clear()
        return self._seen[key] >= 3

    def _graph_step(self, entries: Sequence[StepEntry], rows, q_len, tokens):
        """Runs the step through a captured graph.  A graph fits every step with the same number of requests,
        tokens and wanted rows whose longest portion falls into the same bucket of 64 tokens; everything else
        about the step (tokens, positions, where portions start, block tables, slots) is data the graph reads."""
        key = self._shape_key(entries, q_len)
        S, T, R, bucket = key
        g = self._graphs.get(key)
        if g is None or g.generation != self.workspace.generation:
            # First step of this shape (or buffers moved since): run it eagerly on a buffer of its own so
            # every scratch buffer exists, then capture the same launches.
            widths = [(self.max_positions + grp.page_size - 1) // grp.page_size for grp in self.cache.groups]
            total = self._layout_size(S, T, R, widths)
            g = _DecodeGraph(torch.empty(total, dtype=torch.int32, device=self.device), -1)
            ctx, out_rows = self._layout(entries, rows, q_len, tokens, static=g, max_q_len=bucket)
            self.model.forward(ctx)
            torch.cuda.current_stream().synchronize()
            g.generation = self.workspace.generation
            graph = torch.cuda.CUDAGraph()
            before = ops.LAUNCHES
            with torch.cuda.graph(graph):
                g.logits = self.model.forward(ctx)
            self.graph_launches[key] = ops.LAUNCHES - before
            if S == T:
                self.graph_launches[S] = self.graph_launches[key]
            if g.generation != self.workspace.generation:
                raise RuntimeError("a scratch buffer was created while a step was being captured")
            g.graph = graph
            if len(self._graphs) >= 48:                   # keep the most recent shapes
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = g
        else:
            _, out_rows = self._layout(entries, rows, q_len, tokens, static=g, max_q_len=bucket)
        g.graph.replay()
        self.graph_steps += 1
        return g.logits, out_rows

    @staticmethod
    def _layout_size(S: int, T: int, R: int, widths: Sequence[int]) -> int:
        sizes = [T, T, T, S + 1, S, S, R] + [S * w for w in widths] + [T for _ in widths] + [T]
        return sum((n + 3) // 4 * 4 for n in sizes)

    def _layout(self, entries: Sequence[StepEntry], rows: np.ndarray, q_len: np.ndarray, tokens: np.ndarray,
                static: Optional[_DecodeGraph] = None, max_q_len: int = 0
                ) -> Tuple[StepContext, List[Tuple[Hashable, int]]]:
        cache = self.cache
        S = len(entries)
        n_past = cache.length_arr[rows]
        q_start = np.zeros(S + 1, dtype=np.int64)
        np.cumsum(q_len, out=q_start[1:])
        T = int(q_start[-1])
        requests = [e.request for e in entries]
        if T == S:                                  # one token each
            tok_seq = np.arange(S, dtype=np.int32)
            positions = n_past
            token_rows = rows
        else:
            tok_seq = np.repeat(np.arange(S, dtype=np.int32), q_len)
            positions = np.arange(T, dtype=np.int64) - np.repeat(q_start[:-1], q_len) + np.repeat(n_past, q_len)
            token_rows = np.repeat(rows, q_len)
        out_rows: List[Tuple[Hashable, int]] = []
        logit_rows: List[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                out_rows.append((e.request, int(w)))
                logit_rows.append(int(q_start[i]) + int(w))
        G = len(cache.groups)
        fixed = None
        if static is not None:      # widths that never change, so the captured launches stay valid
            fixed = [(self.max_positions + grp.page_size - 1) // grp.page_size for grp in cache.groups]
        tables = [cache.table_rows(g, rows, width=fixed[g] if fixed else None) for g in range(G)]
        slots = [cache.slots_of(g, token_rows, positions) for g in range(G)]
        pieces = [tokens, positions.astype(np.int32), tok_seq, q_start.astype(np.int32), n_past.astype(np.int32),
                  rows.astype(np.int32), np.asarray(logit_rows, dtype=np.int32)] + [t.reshape(-1) for t in tables] + slots
        rows_out = out_rows
        dt = self._device_tokens
        if dt is not None:          # where each token comes from on the device (-1: from the host array)
            index = np.asarray(dt.index, dtype=np.int32)
            if len(index) != S or (q_len[index >= 0] != 1).any():
                raise invalid_argument("a token can stay on the device only as the single token of its request")
            token_map = np.full(T, -1, dtype=np.int32)
            token_map[q_start[:-1]] = index
            pieces.append(token_map)
        elif static is not None:
            pieces.append(np.full(T, -1, dtype=np.int32))      # a captured step keeps room for the map
        # One staging buffer, one copy to the device; views are carved out of it.
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

        if dt is not None:
            ops.gather_tokens(view(0), dt.source, view(len(pieces) - 1), T)
        groups = [GroupView(group=cache.groups[g], block_table=view(7 + g).view(S, tables[g].shape[1]),
                            slot_mapping=view(7 + G + g)) for g in range(G)]
        ctx = StepContext(
            runtime=self.model.runtime, workspace=self.workspace, cache=cache, n_tokens=T, n_seq=S,
            tokens=view(0), positions=view(1), tok_seq=view(2), q_start=view(3), n_past=view(4), state_slots=view(5),
            logit_rows=view(6), n_logit_rows=len(logit_rows), groups=groups, requests=requests,
            host_q_start=q_start.tolist(), host_n_past=n_past.tolist(), max_q_len=max_q_len or int(q_len.max()),
            max_kv_len=int((n_past + q_len).max()), decode_only=T == S, max_positions=self.max_positions)
        return ctx, rows_out
