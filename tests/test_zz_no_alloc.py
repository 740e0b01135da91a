"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called through its exported C
symbol the way a user without an allocator would call it, against the ordinary entry point.

The file's name sorts it last, so a run that stops at the first failure has run every other test first.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 1 << 20


def _symbol():
    from liyab_b200.csrc.build import ensure_built
    lib = ctypes.CDLL(ensure_built())
    fn = lib.lb_decode_attention_noalloc
    c = ctypes
    fn.argtypes = [c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_int64, c.c_int,
                   c.c_int, c.c_int, c.c_int, c.c_int, c.c_float, c.c_int, c.c_int, c.c_void_p]
    fn.restype = c.c_int
    lib.lb_last_error.restype = c.c_char_p
    return lib, fn


def _case(dev, seed, n_seq, n_head, n_kv_head, head_dim, page_size, max_len):
    rng = np.random.default_rng(seed)
    lens = rng.integers(1, max_len + 1, size=n_seq)
    lens[0] = max_len
    pages_per = -(-max_len // page_size)
    n_pages = n_seq * pages_per
    cache = (torch.randn(n_pages, 2, n_kv_head, page_size, head_dim, device=dev)).to(torch.bfloat16)
    table = torch.from_numpy(rng.permutation(n_pages).astype(np.int32).reshape(n_seq, pages_per)).to(dev)
    q = torch.randn(n_seq, n_head * head_dim, device=dev).to(torch.bfloat16)
    positions = torch.from_numpy((lens - 1).astype(np.int32)).to(dev)
    return q, cache, positions, table


def _plain_attention(q, cache, positions, table, n_head, n_kv_head, head_dim, page_size, scale, window):
    """Decode attention in float64 from the pages: every request's one query over the keys it may see."""
    q, cache = q.double().cpu(), cache.double().cpu()
    positions, table = positions.cpu().numpy(), table.cpu().numpy()
    group = n_head // n_kv_head
    out = torch.zeros(q.shape[0], n_head, head_dim, dtype=torch.float64)
    for i, pos in enumerate(positions):
        lo = max(0, pos - window + 1) if window > 0 else 0
        pages = table[i, : pos // page_size + 1]
        k = torch.cat([cache[p, 0] for p in pages], dim=1)[:, lo:pos + 1]      # [kv_head, keys, head_dim]
        v = torch.cat([cache[p, 1] for p in pages], dim=1)[:, lo:pos + 1]
        for h in range(n_head):
            s = (k[h // group] @ q[i, h * head_dim:(h + 1) * head_dim]) * scale
            out[i, h] = torch.softmax(s, dim=0) @ v[h // group]
    return out.reshape(q.shape[0], -1)


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,splits,window", [(12, 12, 64, 7, 0), (8, 2, 128, 4, 0), (4, 4, 32, 1, 0),
                                                                     (12, 12, 64, 5, 100), (8, 2, 128, 1, 33)])
def test_no_alloc_entry_point_matches_the_ordinary_one(n_head, n_kv_head, head_dim, splits, window):
    from liyab_b200 import ops
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    lib, fn = _symbol()
    page_size, n_seq = 16, 9
    scale = 1.0 / math.sqrt(head_dim)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):           # two calls in a row share the built-in scratch, with different inputs
        q, cache, positions, table = _case(dev, 100 + call, n_seq, n_head, n_kv_head, head_dim, page_size, 700)
        want = torch.empty_like(q)
        partial = torch.empty(n_seq * n_head * splits * (head_dim + 2), device=dev)
        counters = torch.zeros(n_seq * n_kv_head, dtype=torch.int32, device=dev)
        ops.decode_attention(q, cache, positions, table, want, partial, counters, n_seq, n_head, n_kv_head, head_dim,
                             page_size, scale, window, splits, tensor_cores=False)    # the kernel the entry point is a variant of
        got = torch.full_like(q, float("nan"))
        rc = fn(q.data_ptr(), q.stride(0), cache.data_ptr(), positions.data_ptr(), table.data_ptr(), table.stride(0),
                got.data_ptr(), got.stride(0), n_seq, n_head, n_kv_head, head_dim, page_size, scale, window, splits, stream)
        assert rc == 0, lib.lb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert (got.float() - want.float()).abs().max().item() <= 1.5e-2, f"call {call}"
        # and against the attention formula itself, in float64 (not only against the sibling kernel)
        ref = _plain_attention(q, cache, positions, table, n_head, n_kv_head, head_dim, page_size, scale, window)
        assert (got.double().cpu() - ref).abs().max().item() <= 1.5e-2, f"call {call}"


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold():
    dev = torch.device("cuda:0")
    lib, fn = _symbol()
    n_head = n_kv_head = 16
    head_dim, page_size, splits = 128, 16, 32
    n_seq = SCRATCH_FLOATS // (n_head * splits * (head_dim + 2)) + 1
    q, cache, positions, table = _case(dev, 1, n_seq, n_head, n_kv_head, head_dim, page_size, 16)
    out = torch.empty_like(q)
    rc = fn(q.data_ptr(), q.stride(0), cache.data_ptr(), positions.data_ptr(), table.data_ptr(), table.stride(0),
            out.data_ptr(), out.stride(0), n_seq, n_head, n_kv_head, head_dim, page_size, 0.1, 0, splits,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    msg = lib.lb_last_error().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
    rc = fn(q.data_ptr(), q.stride(0), cache.data_ptr(), positions.data_ptr(), table.data_ptr(), table.stride(0),
            out.data_ptr(), out.stride(0), 2, 6, 4, head_dim, page_size, 0.1, 0, 2, torch.cuda.current_stream().cuda_stream)
    assert rc == 4      # a shape the kernel does not take is refused, not run
    # without a split of the keys no scratch is used, so the same large call is taken
    rc = fn(q.data_ptr(), q.stride(0), cache.data_ptr(), positions.data_ptr(), table.data_ptr(), table.stride(0),
            out.data_ptr(), out.stride(0), n_seq, n_head, n_kv_head, head_dim, page_size, 0.1, 0, 1,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.lb_last_error().decode()
    torch.cuda.synchronize()
    ref = _plain_attention(q[:8], cache, positions[:8], table[:8], n_head, n_kv_head, head_dim, page_size, 0.1, 0)
    assert (out[:8].double().cpu() - ref).abs().max().item() <= 1.5e-2
