"""The fused decode step: a stack of pre-norm blocks run by one persistent kernel.

A decode step of a few requests is bound by launch count and memory round
trips, not by bytes or flops.  Where a model is made of nothing but the standard
parts (LayerNorm, attention with a fused projection, dense feed-forward,
pre-norm arrangement, learned or no positions) in bfloat16, its decode steps of
up to 16 tokens are handed to `csrc/decode_stack.cu`, which runs the whole step
as one cooperative kernel.  Anything else (another mixer, another arrangement,
float32, more tokens, prompt portions) takes the part-by-part path; the results
agree to bfloat16 rounding, which the tests check.

This module only describes the model to the kernel: it packs one record per
run-order entry from the parts' own parameters and owns the step's buffers.
"""
from __future__ import annotations

import ctypes
import struct
from typing import Optional

import torch

from .. import ops
from ..parts.attention import CausalSelfAttention
from ..parts.base import StepContext
from ..parts.block import PreNormBlock
from ..parts.feed_forward import DenseFeedForward
from ..parts.norm import LayerNorm
from ..parts.position import LearnedAbsolutePosition, NoPosition

MAX_TOKENS = 16
_LAYER_FORMAT = "<13Q3f6i4x"
_c = ctypes
_p, _i, _f = _c.c_void_p, _c.c_int, _c.c_float

ops.declare("lb_decode_stack", [_p, _i, _i, _i, _i, _p, _p, _f, _p, _p, _f, _p, _p, _p, _p, _p, _i, _p, _i, _p, _p, _p, _p,
                                _p, _p, _p, _p, _i, _i, _i, _i, _p, _p])
ops.declare("lb_decode_stack_status", [_p])
ops.declare("lb_decode_stack_layer_bytes", [])


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


class FusedDecodeStack:
    """Built once per model and cache; `run(ctx)` computes the logits of a decode step."""

    @staticmethod
    def try_build(model, cache) -> Optional["FusedDecodeStack"]:
        rt, spec = model.runtime, model.spec
        if rt.dtype != torch.bfloat16 or len(cache.groups) != 1 or cache.states.needs:
            return None
        if type(model.position) not in (LearnedAbsolutePosition, NoPosition) or type(model.final_norm) is not LayerNorm:
            return None
        ps = cache.page_size
        if ps & (ps - 1) or ps < 16 or spec.hidden % 8:        # the attention phase takes its 16-key tiles from one page
            return None
        head_dim = None
        for i, entry in enumerate(spec.run_order):
            if entry.cache != i:
                return None
            block = model.layers[entry.layer]
            parts = block.parts
            if (type(block) is not PreNormBlock or type(parts.mixer_norm) is not LayerNorm or type(parts.ff_norm) is not LayerNorm
                    or type(parts.mixer) is not CausalSelfAttention or type(parts.feed_forward) is not DenseFeedForward):
                return None
            a, f = parts.mixer.spec, parts.feed_forward.spec
            if a.head_dim not in (64, 128) or (head_dim or a.head_dim) != a.head_dim or f.inner % 8:
                return None
            if a.n_head // a.n_kv_head > 16:       # the query heads of a key/value head are the 16 rows of a tile
                return None
            if f.activation not in ops.ACTIVATIONS:
                return None
            head_dim = a.head_dim
        if head_dim is None:
            return None
        if struct.calcsize(_LAYER_FORMAT) != ops.lib().lb_decode_stack_layer_bytes():
            return None
        stack = FusedDecodeStack(model, cache, head_dim)
        max_k = stack.max_k
        smem = (max(MAX_TOKENS * ((max_k + 63) // 64 * 64 + 32) * 2 + 8 * 8 * 128 * 4, 200 * 1024) + 64 + 16 + 16 + 256
                + stack.n_layers * struct.calcsize(_LAYER_FORMAT))
        return stack if smem <= 227 * 1024 else None

    def __init__(self, model, cache, head_dim: int):
        self.model, self.cache, self.head_dim = model, cache, head_dim
        spec, dev = model.spec, model.runtime.device
        records = []
        self.max_k, self.max_qd, self.max_inner, self.max_heads, self.max_kv_heads = spec.hidden, 0, 0, 0, 0
        for i, entry in enumerate(spec.run_order):
            parts = model.layers[entry.layer].parts
            a, f = parts.mixer.spec, parts.feed_forward.spec
            mixer, ff = parts.mixer, parts.feed_forward
            qd = a.n_head * a.head_dim
            self.max_qd, self.max_inner = max(self.max_qd, qd), max(self.max_inner, f.inner)
            self.max_heads = max(self.max_heads, a.n_head)
            self.max_kv_heads = max(self.max_kv_heads, a.n_kv_head)
            self.max_k = max(self.max_k, qd, f.inner)
            unit = cache.groups[0].unit_storage(i)
            records.append(struct.pack(
                _LAYER_FORMAT, _ptr(parts.mixer_norm.weight), _ptr(parts.mixer_norm.bias), _ptr(parts.ff_norm.weight),
                _ptr(parts.ff_norm.bias), _ptr(mixer.qkv.weight), _ptr(mixer.qkv.bias), _ptr(mixer.out.weight),
                _ptr(mixer.out.bias), _ptr(ff.up.weight), _ptr(ff.up.bias), _ptr(ff.down.weight), _ptr(ff.down.bias),
                unit.data_ptr(), parts.mixer_norm.spec.eps, parts.ff_norm.spec.eps, a.scale, a.n_head, a.n_kv_head,
                a.head_dim, f.inner, ops.ACTIVATIONS[f.activation], a.window))
        blob = b"".join(records)
        self.layers = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(dev)
        self.n_layers = len(records)
        T, V, d = MAX_TOKENS, spec.vocab_size, spec.hidden
        self.x = torch.empty((T, d), dtype=torch.float32, device=dev)
        self.q = torch.empty((T, self.max_qd), dtype=torch.bfloat16, device=dev)
        self.att = torch.empty((T, self.max_qd), dtype=torch.bfloat16, device=dev)
        self.inner = torch.empty((T, self.max_inner), dtype=torch.bfloat16, device=dev)
        self.logits = torch.empty((T, V), dtype=torch.float32, device=dev)
        self.partial = torch.empty(T * self.max_heads * 64 * (head_dim + 2), dtype=torch.float32, device=dev)
        self.counters = torch.zeros(T * self.max_heads, dtype=torch.int32, device=dev)
        self.barrier = torch.zeros(2, dtype=torch.int32, device=dev)      # two counters, used by alternate launches
        self.pos_table = getattr(model.position, "table", None)
        self.launches = 0
        self.n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        self.timing: Optional[torch.Tensor] = None     # int64 [2 + 5 * layers + 1] when phase stamps are wanted

    def accepts(self, n_tokens: int) -> bool:
        return 1 <= n_tokens <= MAX_TOKENS

    def splits(self, n_tokens: int) -> int:
        """(key ranges per (token, key/value head), warps per work item): a function of the batch's shape only.
        A range merged across blocks costs a round of atomics and reloads, so from 64 pairs on a pair is one item,
        served by a whole block (eight warps) while there are blocks enough for that, else by half a block; fewer
        pairs are split until every half block has an item."""
        pairs = n_tokens * self.max_kv_heads
        if pairs >= 64:
            return 1, (8 if pairs <= self.n_sm else 4)
        return max(1, min(8, (2 * self.n_sm) // pairs)), 4        # more ranges only lengthen the last group's merge

    def run(self, ctx: StepContext) -> torch.Tensor:
        m, spec = self.model, self.model.spec
        B = ctx.n_tokens
        view = ctx.groups[0]
        ops.check(ops.lib().lb_decode_stack(
            self.layers.data_ptr(), self.n_layers, B, spec.hidden, spec.vocab_size, m.embedding.data_ptr(),
            _ptr(self.pos_table), float(spec.embedding.scale), _ptr(m.final_norm.weight), _ptr(m.final_norm.bias),
            float(m.final_norm.spec.eps), m.head_weight.data_ptr(), _ptr(m.head_bias), ctx.tokens.data_ptr(),
            ctx.positions.data_ptr(), view.block_table.data_ptr(), view.block_table.stride(0), view.slot_mapping.data_ptr(),
            self.cache.page_size, self.x.data_ptr(), self.q.data_ptr(), self.att.data_ptr(), self.inner.data_ptr(),
            self.partial.data_ptr(), self.counters.data_ptr(), self.logits.data_ptr(), self.barrier.data_ptr() + 4 * (self.launches & 1), self.max_k,
            self.head_dim, *self.splits(B), _ptr(self.timing), ops.stream_ptr()), "decode_stack")
        self.launches += 1
        return self.logits[:B]

    @staticmethod
    def status() -> int:
        """0 unless a grid barrier gave up since the last call (then the phase's code).  Synchronises the device."""
        status = ctypes.c_int(0)
        ops.check(ops.lib().lb_decode_stack_status(ctypes.byref(status)), "decode_stack_status")
        return status.value
