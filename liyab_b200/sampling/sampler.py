"""Batched next-token choice on the device.

One kernel launch picks a token for every row of logits, each row with its own
temperature, top-k, top-p and uniform draw (csrc/sampling.cu restates the
reference's sampler, src/core/sampling.cpp:16-79).  The per-row options travel
in one pinned staging buffer per step.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams


class DeviceSampler:
    def __init__(self, device: torch.device, max_rows: int = 256):
        self.device = device
        self._cap = 0
        self._last_key, self._last_params, self._last_greedy = None, None, False
        self._grow(max_rows)

    def _grow(self, rows: int) -> None:
        if rows <= self._cap:
            return
        self._cap = rows
        self._last_key = None
        # [temperature f32 | top_p f32 | top_k i32 | pad | uniform f64] per row, as 5 x 4-byte words... kept
        # as separate arrays inside one allocation so that one copy moves them all.
        # Two pinned staging buffers used in turn: one is rewritten only after the copy that last read it has
        # run on the device (the host may be a step ahead of the GPU).
        self._hosts = [torch.empty(rows * 6, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._copied = [torch.cuda.Event(), torch.cuda.Event()]
        self._turn = 0
        self._dev = torch.empty(rows * 6, dtype=torch.int32, device=self.device)
        self.out_ids = torch.empty(rows, dtype=torch.int32, device=self.device)
        self._host_ids = torch.empty(rows, dtype=torch.int32).pin_memory()
        self._tickets = [(torch.empty(rows, dtype=torch.int32).pin_memory(), torch.cuda.Event()) for _ in range(2)]
        self._next_ticket = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], uniforms: Sequence[float],
               out_probs: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Token ids (int32, on the device) for rows 0 .. len(params)-1 of `logits`."""
        n = len(params)
        self._grow(n)
        cap = self._cap
        key = tuple(map(id, params))
        same = key == self._last_key
        greedy = same and self._last_greedy
        if not greedy:
            turn = self._turn = 1 - self._turn
            self._copied[turn].synchronize()
            host = self._hosts[turn]
            h = host.numpy()
            h[0:n].view(np.float32)[:] = [p.temperature for p in params]
            h[cap:cap + n].view(np.float32)[:] = [p.top_p for p in params]
            h[2 * cap:2 * cap + n] = [min(p.top_k, 2 ** 31 - 1) for p in params]
            if not same:
                self._last_key, self._last_params = key, list(params)      # the list keeps the ids from being reused
                self._last_greedy = all(p.temperature <= 0 for p in params)
            h[4 * cap:4 * cap + 2 * n].view(np.float64)[:] = uniforms
            self._dev.copy_(host, non_blocking=True)
            self._copied[turn].record()
        d = self._dev
        ops.sample(logits, n, d[0:cap].view(torch.float32), d[2 * cap:3 * cap], d[cap:2 * cap].view(torch.float32),
                   d[4 * cap:6 * cap].view(torch.float64), self.out_ids, out_probs)
        return self.out_ids[:n]

    def to_host(self, n: int) -> list:
        """The last `n` sampled ids as a Python list (waits for the device)."""
        self._host_ids[:n].copy_(self.out_ids[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host_ids[:n].tolist()

    def fetch_async(self, n: int) -> int:
        """Starts copying the last `n` sampled ids to the host; returns a ticket for `wait`.  Two tickets are
        live at most: the one before last must have been waited for."""
        ticket = self._next_ticket
        self._next_ticket = 1 - ticket
        host, event = self._tickets[ticket]
        host[:n].copy_(self.out_ids[:n], non_blocking=True)
        event.record()
        return ticket

    def wait(self, ticket: int, n: int) -> list:
        host, event = self._tickets[ticket]
        event.synchronize()
        return host[:n].tolist()
