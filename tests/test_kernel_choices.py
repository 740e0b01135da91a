"""Which kernel takes which shape: the library's host-side predicates and split choices, without a GPU.

These decide whether a size that the configuration allows reaches a specialised kernel, the generic one, or a
clear refusal, so they are pinned here for the sizes the kernels' comments promise."""
from __future__ import annotations

import pytest

from liyab_b200 import ops


def test_decode_attention_shapes():
    # (scalar kernel, tensor-core kernel)
    assert ops.decode_attention_kernels(12, 12, 64, 16) == (True, True)
    assert ops.decode_attention_kernels(32, 8, 128, 16) == (True, True)
    assert ops.decode_attention_kernels(48, 3, 64, 32)[1]                  # sixteen query heads per key/value head
    assert not ops.decode_attention_kernels(34, 2, 64, 32)[1]              # seventeen: too many rows for one tile
    assert ops.decode_attention_kernels(3, 3, 32, 16) == (True, False)      # head size 32: scalar only
    assert not ops.decode_attention_kernels(12, 12, 64, 8)[1]              # a tile of 16 keys must lie in one page
    assert ops.decode_attention_kernels(5, 5, 48, 16) == (False, False)    # head size 48: the generic kernel's
    assert ops.decode_attention_kernels(12, 5, 64, 16) == (False, False)   # heads that do not divide


def test_prefill_attention_shapes():
    assert ops.prefill_attention_supports(12, 12, 64, 16) and ops.prefill_attention_tc_supports(12, 12, 64, 16)
    assert ops.prefill_attention_supports(8, 2, 128, 16) and not ops.prefill_attention_tc_supports(8, 2, 128, 16)
    assert ops.prefill_attention_supports(3, 3, 32, 16)
    assert not ops.prefill_attention_tc_supports(12, 12, 64, 8)
    assert not ops.prefill_attention_supports(4, 4, 24, 16)                # head sizes in steps of 16 up to 128 only


@pytest.mark.parametrize("n_seq,n_kv,ctx,tensor", [(1, 12, 1024, True), (8, 12, 1024, True), (64, 12, 1024, True),
                                                   (1, 12, 1024, False), (64, 12, 1024, False), (3, 1, 96, False),
                                                   (5, 2, 0, True)])
def test_decode_splits_depend_on_the_shape_only(n_seq, n_kv, ctx, tensor):
    s = ops.decode_splits(n_seq, n_kv, ctx, tensor_cores=tensor)
    assert 1 <= s <= 32 and s == ops.decode_splits(n_seq, n_kv, ctx, tensor_cores=tensor)
    if ctx:
        assert s <= max(1, ctx // (96 if tensor else 128))                # no key range shorter than that
    if n_seq * n_kv >= 444:
        assert ops.decode_splits(n_seq, n_kv, ctx, tensor_cores=True) == 1


def test_gemm_split_of_k():
    assert ops.gemm_splits(65, 768, 768) == 1 and ops.gemm_splits(0, 768, 768) == 1
    assert ops.gemm_splits(8, 768, 3072) == 16                             # 6 tiles of features: K in 16 parts
    assert ops.gemm_splits(8, 50257, 768) == 1                             # a vocabulary fills the GPU by itself
    assert ops.gemm_splits(8, 768, 64) == 1                                # one k-block cannot be split


def test_cache_destination_of_the_projection():
    """The many-token projection sends keys and values to the cache only in whole 64-feature strips of one head."""
    f = ops.lib().lb_gemm_persistent_kv_supports
    bf16, f32, none, gelu = ops.BF16, ops.F32, ops.ACTIVATIONS["none"], ops.ACTIVATIONS["gelu_tanh"]
    assert f(bf16, 2304, none, 0, 768, 12, 64, 16)
    assert f(bf16, 4096 + 2 * 1024, none, 0, 4096, 8, 128, 32)
    assert not f(f32, 2304, none, 0, 768, 12, 64, 16)                       # a float32 product
    assert not f(bf16, 2304, gelu, 0, 768, 12, 64, 16) and not f(bf16, 2304, none, 1, 768, 12, 64, 16)
    assert not f(bf16, 288, none, 0, 96, 1, 96, 16)                         # head size 96
    assert not f(bf16, 2304, none, 0, 768, 12, 64, 24)                      # a page that is no power of two
    assert not f(bf16, 2300, none, 0, 768, 12, 64, 16)                      # not [q | k | v]
