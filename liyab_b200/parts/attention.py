"""Causal self-attention over the paged cache, with one fused projection of
queries, keys and values.

Sizes and constants are the spec's: heads, key/value heads, head size, the
factor on the scores and the window.  The step's keys and values are written to
the unit's pages first; attention then reads every key, old and new, from the
pages, so a token's result does not depend on how its sequence was cut into
steps.  Reference: attention_mixer (src/core/transformer.cpp:3035-3142): fused
projection and split [q | k | v] (:2657-2673), biases (:3089-3101), store_kv
(:2875-2890), attention (:2130-2453), output projection (:3139-3140).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .. import ops
from ..cache.pages import KvNeed, StateNeed
from ..config.spec import AttentionSpec
from ..status import invalid_model
from .base import CacheUnit, Runtime, StepContext
from .linear import Linear
from .registry import MIXERS


@MIXERS.register("attention")
class CausalSelfAttention:
    def __init__(self, spec: AttentionSpec, params: Dict[str, torch.Tensor], runtime: Runtime):
        if spec.n_head % spec.n_kv_head != 0:
            raise invalid_model(f"attention: n_head {spec.n_head} is not a multiple of n_kv_head {spec.n_kv_head}")
        self.spec = spec
        self.runtime = runtime
        self.q_dim = spec.n_head * spec.head_dim
        self.kv_dim = spec.n_kv_head * spec.head_dim
        self.qkv = Linear(params["qkv.weight"], params.get("qkv.bias"), "attention.qkv")
        self.out = Linear(params["out.weight"], params.get("out.bias"), "attention.out")

    @classmethod
    def parameters(cls, spec: AttentionSpec) -> Dict[str, Tuple[tuple, str]]:
        q, kv = spec.n_head * spec.head_dim, spec.n_kv_head * spec.head_dim
        p = {}
        for k, v in Linear.parameters(q + 2 * kv, spec.hidden, spec.bias).items():
            p["qkv." + k] = v
        for k, v in Linear.parameters(spec.hidden, q, spec.bias).items():
            p["out." + k] = v
        return p

    def kv_need(self) -> Optional[KvNeed]:
        return KvNeed(n_kv_head=self.spec.n_kv_head, head_dim=self.spec.head_dim, window=self.spec.window)

    def state_need(self) -> Optional[StateNeed]:
        return None

    def _attend(self, ctx: StepContext, q, cache, view, att, page_size: int) -> None:
        """Chooses the attention kernel.  bfloat16: a split-key decode kernel for steps of single tokens (on the
        tensor cores where that one takes the shape, else scalar), the tensor-core prefill kernel for steps with
        prompt portions, where they take the shape.  Else the generic
        kernel; all of the 32-bit engine runs on it, so that there a position's result has the same bits
        however the work was cut."""
        s, T = self.spec, ctx.n_tokens
        scalar, tensor = (ops.decode_attention_kernels(s.n_head, s.n_kv_head, s.head_dim, page_size)
                          if ctx.decode_only and self.runtime.dtype == torch.bfloat16 else (False, False))
        if scalar or tensor:
            splits = ops.decode_splits(T, s.n_kv_head, ctx.max_positions, tensor_cores=tensor)
            partial = counters = None
            if splits > 1:
                partial = ctx.workspace.flat("attn.decode.partial", T * s.n_head * splits * (s.head_dim + 2), torch.float32)
                counters = ctx.workspace.flat("attn.decode.counters", T * s.n_kv_head, torch.int32, zero=True)
            ops.decode_attention(q, cache, ctx.positions, view.block_table, att, partial, counters, T, s.n_head,
                                 s.n_kv_head, s.head_dim, page_size, s.scale, s.window, splits, tensor_cores=tensor)
            return
        if (self.runtime.dtype == torch.bfloat16
                and ops.prefill_attention_supports(s.n_head, s.n_kv_head, s.head_dim, page_size)):
            ops.prefill_attention(q, cache, ctx.q_start, ctx.n_past, view.block_table, att, ctx.n_seq, ctx.max_q_len,
                                  s.n_head, s.n_kv_head, s.head_dim, page_size, s.scale, s.window)
            return
        ops.paged_attention_generic(q, cache, ctx.tok_seq, ctx.positions, view.block_table, att, T, s.n_head,
                                    s.n_kv_head, s.head_dim, page_size, s.scale, s.window)

    def forward(self, ctx: StepContext, h: torch.Tensor, x: torch.Tensor, unit: CacheUnit) -> None:
        s, T, dt = self.spec, ctx.n_tokens, self.runtime.dtype
        ws = ctx.workspace
        qkv = ws.get("attn.qkv", T, self.q_dim + 2 * self.kv_dim, dt)
        cache, view = ctx.kv(unit.read)
        page_size = view.group.page_size
        w = self.qkv.weight
        if (unit.write and dt == torch.bfloat16 and 16 < T <= 64 and w.shape[1] <= 1024 and ops.gemm_rows_supports(h, w, T)):
            # A step of a few dozen tokens: the projection's epilogue also puts the new keys and values into their pages.
            ops.gemm_rows(h, w, self.qkv.bias, qkv, T,
                          kv=(cache, view.slot_mapping, self.q_dim, s.n_kv_head, s.head_dim, page_size))
        elif (unit.write and dt == torch.bfloat16 and T > 64 and ops.gemm_persistent_tile(h, w, qkv, T) > 0
              and ops.gemm_persistent_kv_supports(w, qkv, self.q_dim, s.n_kv_head, s.head_dim, page_size)):
            # Many tokens: the same from the tensor-core product's epilogue (only the queries go to `qkv`).
            ops.gemm_persistent(h, w, self.qkv.bias, qkv, T,
                                kv=(cache, view.slot_mapping, self.q_dim, s.n_kv_head, s.head_dim, page_size))
        else:
            self.qkv.forward(h, qkv, T, workspace=ws)
            if unit.write:
                k = qkv[:, self.q_dim:self.q_dim + self.kv_dim]
                v = qkv[:, self.q_dim + self.kv_dim:]
                ops.kv_append(k, v, view.slot_mapping, cache, T, s.n_kv_head, s.head_dim, page_size)
        q = qkv[:, :self.q_dim]
        att = ws.get("attn.out", T, self.q_dim, dt)
        self._attend(ctx, q, cache, view, att, page_size)
        self.out.forward(att, x, T, residual=x, workspace=ws)
