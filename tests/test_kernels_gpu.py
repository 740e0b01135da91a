"""Each kernel alone against a plain float32/float64 PyTorch restatement, at
sizes other than the engine's."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_gpt2 as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def _rand(shape, seed, dev, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [48, 200, 1600])
def test_embed_positions(dev, dtype, width):
    from liyab_b200 import ops
    V, P, T = 301, 77, 19
    table, pos_table = _rand((V, width), 1, dev, dtype), _rand((P, width), 2, dev, dtype)
    tokens = torch.randint(0, V, (T,), dtype=torch.int32, device=dev)
    positions = torch.randint(0, P, (T,), dtype=torch.int32, device=dev)
    out = torch.empty((T, width), dtype=torch.float32, device=dev)
    ops.embed_positions(tokens, positions, table, pos_table, out, scale=1.0)
    ref = table.float()[tokens.long()] + pos_table.float()[positions.long()]
    assert torch.equal(out, ref)
    ops.embed_positions(tokens, positions, table, None, out, scale=0.5)
    assert torch.equal(out, table.float()[tokens.long()] * 0.5)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,eps", [(48, 1e-5), (250, 1e-6), (1600, 1e-3), (4100, 1e-5)])
def test_layernorm(dev, out_dtype, width, eps):
    from liyab_b200 import ops
    R = 37
    x = _rand((R, width), 3, dev) * 3.0 + 5.0          # a mean far from zero shows a one-pass variance
    w, b = _rand((width,), 4, dev) + 1.0, _rand((width,), 5, dev)
    out = torch.empty((R, width), dtype=out_dtype, device=dev)
    ops.layernorm(x, w, b, eps, out, R)
    ref = torch.from_numpy(plain.layernorm(x.double().cpu().numpy(), w.double().cpu().numpy(), b.double().cpu().numpy(), eps))
    tol = 2e-5 if out_dtype == torch.float32 else 2e-2
    assert (out.double().cpu() - ref).abs().max().item() < tol * ref.abs().max().item()
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device=dev)
    out2 = torch.empty((4, width), dtype=out_dtype, device=dev)
    ops.layernorm(x, w, b, eps, out2, 4, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 50, 24), (7, 333, 100), (64, 96, 96), (130, 257, 72), (300, 1000, 513)])
@pytest.mark.parametrize("act", ["none", "gelu_tanh", "gelu_erf"])
def test_gemm_ffma(dev, dtypes, M, N, K, act):
    from liyab_b200 import ops
    tin, tout = dtypes
    a, w = _rand((M, K), 6, dev, tin), _rand((N, K), 7, dev, tin, 0.2)
    bias, res = _rand((N,), 8, dev), _rand((M, N), 9, dev)
    ref = a.double() @ w.double().t() + bias.double()
    ref = {"none": lambda v: v, "gelu_tanh": lambda v: torch.from_numpy(plain.gelu_tanh(v.cpu().numpy())).to(dev),
           "gelu_erf": lambda v: torch.from_numpy(plain.gelu_erf(v.cpu().numpy())).to(dev)}[act](ref)
    out = torch.empty((M, N), dtype=tout, device=dev)
    ops.gemm_ffma(a, w, bias, out, M, act)
    tol = 1e-5 if tout == torch.float32 else 1e-2
    assert (out.double() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    if tout == torch.float32:
        out2 = res.clone()
        ops.gemm_ffma(a, w, bias, out2, M, act, residual=out2)
        assert (out2.double() - (ref + res.double())).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
        # A row's bits do not depend on how many rows share the launch.
        one = torch.empty((1, N), dtype=tout, device=dev)
        ops.gemm_ffma(a[M - 1:M], w, bias, one, 1, act)
        assert torch.equal(one[0], out[M - 1])


def _paged_case(dev, dtype, n_head, n_kv_head, head_dim, page_size, lens, q_lens, seed, boost=None):
    """Random q/k/v for requests with `lens` tokens, of which the last `q_lens` are this step's.
    Returns kernel inputs and the float64 reference output."""
    rng = np.random.default_rng(seed)
    S = len(lens)
    n_pages = sum(-(-l // page_size) for l in lens) + 3
    perm = rng.permutation(n_pages)
    # What no request has written holds NaN: a kernel that lets such a place reach its output, even with weight 0, shows.
    cache = torch.full((n_pages, 2, n_kv_head, page_size, head_dim), float("nan"), dtype=dtype)
    width = max(-(-l // page_size) for l in lens)
    table = np.full((S, width), -1, dtype=np.int32)
    qs, refs, tok_seq, positions = [], [], [], []
    at = 0
    for s, (L, Q) in enumerate(zip(lens, q_lens)):
        k = torch.from_numpy(rng.standard_normal((L, n_kv_head, head_dim))).to(dtype)
        v = torch.from_numpy(rng.standard_normal((L, n_kv_head, head_dim))).to(dtype)
        q = torch.from_numpy(rng.standard_normal((Q, n_head, head_dim))).to(dtype)
        if boost is not None:          # one far key that the query must find among many
            key_pos, factor = boost
            if key_pos < L:
                k[key_pos] = q[-1, ::n_head // n_kv_head] * factor
        for p in range(-(-L // page_size)):
            table[s, p] = perm[at]
            lo, hi = p * page_size, min(L, (p + 1) * page_size)
            cache[perm[at], 0, :, :hi - lo] = k[lo:hi].permute(1, 0, 2)
            cache[perm[at], 1, :, :hi - lo] = v[lo:hi].permute(1, 0, 2)
            at += 1
        qs.append(q)
        tok_seq += [s] * Q
        positions += list(range(L - Q, L))
        refs.append((q.double(), k.double(), v.double(), L - Q))
    q_all = torch.cat(qs).reshape(-1, n_head * head_dim)
    return (q_all.to(dev), cache.to(dev), torch.tensor(tok_seq, dtype=torch.int32, device=dev),
            torch.tensor(positions, dtype=torch.int32, device=dev), torch.from_numpy(table).to(dev), refs)


def _attention_reference(refs, n_head, n_kv_head, scale, window):
    outs = []
    group = n_head // n_kv_head
    for q, k, v, first in refs:
        Q, L = q.shape[0], k.shape[0]
        o = torch.zeros(Q, n_head, q.shape[2], dtype=torch.float64)
        for h in range(n_head):
            s = (q[:, h] @ k[:, h // group].t()) * scale
            pos = torch.arange(first, first + Q)[:, None]
            j = torch.arange(L)[None, :]
            mask = j <= pos
            if window > 0:
                mask &= j > pos - window
            s = s.masked_fill(~mask, float("-inf"))
            o[:, h] = torch.softmax(s, dim=-1) @ v[:, h // group]
        outs.append(o.reshape(Q, -1))
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window", [
    (4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (6, 2, 48, 32, 0), (5, 1, 64, 64, 0), (2, 2, 128, 16, 0),
    (7, 7, 80, 16, 0), (4, 2, 256, 16, 0), (4, 4, 32, 16, 40), (2, 1, 64, 32, 7)])
def test_paged_attention_generic(dev, dtype, n_head, n_kv_head, head_dim, page_size, window):
    from liyab_b200 import ops
    lens, q_lens = [1, 37, 130, 64, 300], [1, 37, 2, 1, 45]
    scale = 0.37 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, dtype, n_head, n_kv_head, head_dim, page_size, lens,
                                                            q_lens, seed=head_dim + n_head)
    out = torch.empty_like(q)
    ops.paged_attention_generic(q, cache, tok_seq, positions, table, out, q.shape[0], n_head, n_kv_head, head_dim,
                                page_size, scale, window)
    ref = _attention_reference(refs, n_head, n_kv_head, scale, window)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    assert (out.double().cpu() - ref).abs().max().item() < tol


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window", [(4, 2, 64, 16, 0), (3, 3, 48, 32, 70), (2, 1, 128, 16, 0)])
def test_float32_attention_of_few_and_of_many_pairs_agree_bit_for_bit(dev, n_head, n_kv_head, head_dim, page_size, window):
    """Launches of few (token, head) pairs take a kernel arranged around memory latency, larger ones the plain one;
    both make the same sums in the same order, so a token's output does not depend on how many others ran beside it."""
    from liyab_b200 import ops
    lens, q_lens = [330, 210, 97], [330, 210, 97]
    scale = 1.0 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, torch.float32, n_head, n_kv_head, head_dim, page_size, lens,
                                                            q_lens, seed=3 * head_dim)
    n = q.shape[0]
    assert n * n_head > 1024
    whole = torch.empty_like(q)
    ops.paged_attention_generic(q, cache, tok_seq, positions, table, whole, n, n_head, n_kv_head, head_dim, page_size, scale, window)
    ref = _attention_reference(refs, n_head, n_kv_head, scale, window)
    assert (whole.double().cpu() - ref).abs().max().item() < 2e-5
    for lo, hi in ((0, 1), (300, 340), (529, 540), (n - 64, n)):
        assert (hi - lo) * n_head <= 1024
        part = torch.empty((hi - lo, q.shape[1]), dtype=torch.float32, device=dev)
        ops.paged_attention_generic(q[lo:hi].contiguous(), cache, tok_seq[lo:hi].contiguous(), positions[lo:hi].contiguous(), table,
                                    part, hi - lo, n_head, n_kv_head, head_dim, page_size, scale, window)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key(dev, dtype):
    """One key far back, scaled so that its score stands out among hundreds: a kernel that drops a page,
    a tile or the first key shows it."""
    from liyab_b200 import ops
    n_head, n_kv_head, head_dim, page_size = 4, 2, 64, 16
    for key_pos in (0, 15, 16, 271, 511):
        q, cache, tok_seq, positions, table, refs = _paged_case(
            dev, dtype, n_head, n_kv_head, head_dim, page_size, [512], [1], seed=key_pos, boost=(key_pos, 4.0))
        out = torch.empty_like(q)
        ops.paged_attention_generic(q, cache, tok_seq, positions, table, out, 1, n_head, n_kv_head, head_dim,
                                    page_size, 1.0 / math.sqrt(head_dim), 0)
        ref = _attention_reference(refs, n_head, n_kv_head, 1.0 / math.sqrt(head_dim), 0)
        tol = 2e-5 if dtype == torch.float32 else 1.5e-2
        assert (out.double().cpu() - ref).abs().max().item() < tol, f"far key at {key_pos}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kv_append(dev, dtype):
    from liyab_b200 import ops
    n_kv_head, head_dim, page_size, n_pages, T = 3, 48, 16, 9, 40
    qkv = _rand((T, 5 * n_kv_head * head_dim), 11, dev, dtype)
    k = qkv[:, n_kv_head * head_dim: 2 * n_kv_head * head_dim]
    v = qkv[:, 3 * n_kv_head * head_dim: 4 * n_kv_head * head_dim]
    slots = torch.randperm(n_pages * page_size)[:T].to(torch.int32)
    slots[5] = -1
    cache = torch.zeros((n_pages, 2, n_kv_head, page_size, head_dim), dtype=dtype, device=dev)
    ops.kv_append(k, v, slots.to(dev), cache, T, n_kv_head, head_dim, page_size)
    ref = torch.zeros_like(cache)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        ref[s // page_size, 0, :, s % page_size] = k[t].reshape(n_kv_head, head_dim)
        ref[s // page_size, 1, :, s % page_size] = v[t].reshape(n_kv_head, head_dim)
    assert torch.equal(cache, ref)


@pytest.mark.parametrize("vocab", [50, 1000, 50257])
def test_sampling_matches_plain(dev, vocab):
    from liyab_b200 import ops
    rng = np.random.default_rng(vocab)
    cases = [(0.0, 0, 1.0), (0.8, 40, 0.95), (0.8, 0, 1.0), (1.3, 5, 1.0), (0.7, 0, 0.5), (1.0, 1000000, 0.9),
             (0.5, 3, 0.2), (2.0, 17, 0.999), (1.0, 1024, 0.97), (0.9, 1025, 0.9), (1.1, 300, 1.0), (0.9, 256, 0.9),
             (0.9, 257, 1.0), (1.0, 255, 0.5), (0.6, 1, 1.0), (1.0, 2, 0.99)]
    R = len(cases)
    logits = rng.standard_normal((R, vocab)).astype(np.float32) * 2.0
    logits[1, 7] = logits[1].max() + 0.5
    logits[3, :] = np.round(logits[3, :])          # many exact ties, also at the top-k edge
    u = rng.random(R)
    out_ids = torch.empty(R, dtype=torch.int32, device=dev)
    probs = torch.empty((R, vocab), dtype=torch.float32, device=dev)
    ops.sample(torch.from_numpy(logits).to(dev), R, torch.tensor([c[0] for c in cases], dtype=torch.float32, device=dev),
               torch.tensor([c[1] for c in cases], dtype=torch.int32, device=dev),
               torch.tensor([c[2] for c in cases], dtype=torch.float32, device=dev),
               torch.from_numpy(u).to(dev), out_ids, probs)
    got_ids, got_probs = out_ids.cpu().numpy(), probs.cpu().numpy()
    for r, (t, k, p) in enumerate(cases):
        ref = plain.sampler_probabilities(logits[r], t, k, p)
        assert (ref > 0).sum() == (got_probs[r] > 0).sum(), f"case {r}: kept sets differ in size"
        assert np.array_equal(ref > 0, got_probs[r] > 0), f"case {r}: kept sets differ"
        assert np.abs(ref - got_probs[r]).max() < 2e-6, f"case {r}"
        if t <= 0:
            assert got_ids[r] == int(np.argmax(logits[r]))
        else:
            assert got_ids[r] == plain.sampler_draw(got_probs[r], float(u[r])), f"case {r}"


@pytest.mark.parametrize("vocab", [300, 50257])
def test_sampling_top_p_alone_on_peaked_rows(dev, vocab):
    """Top-p without top-k on rows peaked enough that the few largest logits hold the asked share (the short way)
    and on one that is not (the general way), with ties at the cut: kept sets, probabilities and draws as the plain
    sampler's."""
    from liyab_b200 import ops
    rng = np.random.default_rng(vocab + 1)
    cases = [(1.0, 0, 0.9), (0.7, 0, 0.3), (1.0, 0, 0.999), (1.5, 0, 0.95), (1.0, 0, 0.6)]
    R = len(cases)
    logits = rng.standard_normal((R, vocab)).astype(np.float32) * 8.0
    logits[3] *= 0.05                                   # flat: the nucleus holds thousands of ids
    logits[4, :] = np.round(logits[4, :] / 4.0) * 4.0   # many exact ties, also at the cut
    u = rng.random(R)
    out_ids = torch.empty(R, dtype=torch.int32, device=dev)
    probs = torch.empty((R, vocab), dtype=torch.float32, device=dev)
    ops.sample(torch.from_numpy(logits).to(dev), R, torch.tensor([c[0] for c in cases], dtype=torch.float32, device=dev),
               torch.tensor([c[1] for c in cases], dtype=torch.int32, device=dev),
               torch.tensor([c[2] for c in cases], dtype=torch.float32, device=dev),
               torch.from_numpy(u).to(dev), out_ids, probs)
    got_ids, got_probs = out_ids.cpu().numpy(), probs.cpu().numpy()
    for r, (t, k, p) in enumerate(cases):
        ref = plain.sampler_probabilities(logits[r], t, k, p)
        assert np.array_equal(ref > 0, got_probs[r] > 0), f"case {r}: kept sets differ ({(ref > 0).sum()} vs {(got_probs[r] > 0).sum()})"
        assert np.abs(ref - got_probs[r]).max() < 2e-6, f"case {r}"
        assert got_ids[r] == plain.sampler_draw(got_probs[r], float(u[r])), f"case {r}"


def test_greedy_takes_the_first_maximum(dev):
    from liyab_b200 import ops
    logits = torch.zeros((2, 3000), dtype=torch.float32, device=dev)
    logits[0, [2999, 1234, 77]] = 5.0
    logits[1, :] = -1.0
    out = torch.empty(2, dtype=torch.int32, device=dev)
    z = torch.zeros(2, device=dev)
    ops.sample(logits, 2, z, torch.zeros(2, dtype=torch.int32, device=dev), z + 1, z.double(), out)
    assert out.tolist() == [77, 0]


def test_sampling_of_rows_that_hold_no_numbers_stays_inside_the_vocabulary(dev):
    """Logits that are no numbers (a model that overflowed) count as the lowest; whatever the row holds, the id
    that comes out indexes the embedding table of the next step, so it lies inside the vocabulary."""
    from liyab_b200 import ops
    vocab = 3001
    nan = float("nan")
    logits = torch.full((6, vocab), nan, dtype=torch.float32, device=dev)
    logits[1, 100] = -3.0
    logits[2, :] = 1.0
    logits[2, ::7] = nan
    logits[2, 2222] = 4.0
    logits[4, 5] = 2.0
    logits[4, 9] = 2.5
    logits[5, :] = float("-inf")
    temp = torch.tensor([0, 0, 0, 0.8, 0.8, 0.8], dtype=torch.float32, device=dev)
    top_k = torch.tensor([0, 0, 0, 0, 40, 0], dtype=torch.int32, device=dev)
    top_p = torch.tensor([1, 1, 1, 0.9, 1.0, 0.5], dtype=torch.float32, device=dev)
    u = torch.tensor([0.1, 0.2, 0.3, 0.4, 0.99, 0.6], dtype=torch.float64, device=dev)
    out = torch.full((6,), -7, dtype=torch.int32, device=dev)
    ops.sample(logits, 6, temp, top_k, top_p, u, out)
    ids = out.tolist()
    assert ids[:3] == [0, 100, 2222]
    assert all(0 <= i < vocab for i in ids), ids
    assert ids[4] in (5, 9)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K,tile", [
    (1, 128, 64, 0), (8, 768, 768, 0), (5, 1000, 96, 0), (16, 130, 72, 0), (33, 50257, 256, 0), (64, 2304, 768, 0),
    (100, 320, 3072, 0), (300, 777, 200, 0), (1025, 384, 136, 0), (2048, 768, 768, 256), (70, 96, 320, 16),
    (257, 257, 64, 32), (64, 64, 1024, 64)])
def test_gemm_tcgen05(dev, out_dtype, M, N, K, tile):
    """The tensor-core product against float64, over every token tile, ragged edges in M, N and K,
    a K that wraps the stage ring several times, and all epilogues."""
    from liyab_b200 import ops
    a, w = _rand((M, K), 16, dev, torch.bfloat16), _rand((N, K), 17, dev, torch.bfloat16, 0.2)
    bias, res = _rand((N,), 18, dev), _rand((M, N), 19, dev)
    base = a.double() @ w.double().t()
    scale = max(1.0, base.abs().max().item())
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
    ops.gemm_tcgen05(a, w, None, out, M, token_tile=tile)
    assert ops.device_status() == 0
    assert (out.double() - base).abs().max().item() <= tol * scale
    for act, fn in (("gelu_tanh", plain.gelu_tanh), ("gelu_erf", plain.gelu_erf)):
        ops.gemm_tcgen05(a, w, bias, out, M, act, token_tile=tile)
        ref = torch.from_numpy(fn((base + bias.double()).cpu().numpy())).to(dev)
        assert (out.double() - ref).abs().max().item() <= tol * scale, act
    if out_dtype == torch.float32:
        out2 = res.clone()
        ops.gemm_tcgen05(a, w, bias, out2, M, "none", residual=out2, token_tile=tile)
        assert (out2.double() - (base + bias.double() + res.double())).abs().max().item() <= tol * scale
    # a view with a row stride (the attention output inside a wider buffer) and fewer rows than the buffer holds
    wide = torch.zeros((M + 3, K + 8), dtype=torch.bfloat16, device=dev)
    wide[:M, :K] = a
    out3 = torch.full((M + 3, N), 7.0, dtype=out_dtype, device=dev)
    ops.gemm_tcgen05(wide[:, :K], w, None, out3, M, token_tile=tile)
    assert (out3[:M].double() - base).abs().max().item() <= tol * scale and (out3[M:] == 7.0).all()
    assert ops.device_status() == 0


@pytest.mark.parametrize("out_dtype,M,N,K,tile", [
    (torch.float32, 65, 96, 64, 0), (torch.float32, 130, 200, 136, 0), (torch.float32, 300, 768, 3072, 0),
    (torch.float32, 2048, 768, 768, 96), (torch.float32, 5000, 1000, 72, 128), (torch.float32, 257, 36, 520, 32),
    (torch.float32, 1024, 352, 264, 160), (torch.bfloat16, 100, 72, 64, 0), (torch.bfloat16, 2048, 2304, 768, 0),
    (torch.bfloat16, 777, 3072, 768, 192), (torch.bfloat16, 6000, 520, 200, 64), (torch.bfloat16, 4100, 1280, 328, 256)])
def test_gemm_persistent(dev, out_dtype, M, N, K, tile):
    """The persistent tensor-core product against float64: ragged edges in M, N and K, feature tiles of every
    kind, several tiles per block (both accumulators, the staging buffer used again), all epilogues, the
    residual in place, and a strided input."""
    from liyab_b200 import ops
    a, w = _rand((M, K), 36, dev, torch.bfloat16), _rand((N, K), 37, dev, torch.bfloat16, 0.2)
    bias, res = _rand((N,), 38, dev), _rand((M, N), 39, dev)
    assert ops.gemm_persistent_tile(a, w, torch.empty((M, N), dtype=out_dtype, device=dev), M) > 0
    base = a.double() @ w.double().t()
    scale = max(1.0, base.abs().max().item())
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
    ops.gemm_persistent(a, w, None, out, M, feature_tile=tile)
    assert ops.device_status() == 0
    assert (out.double() - base).abs().max().item() <= tol * scale
    for act, fn in (("gelu_tanh", plain.gelu_tanh), ("gelu_erf", plain.gelu_erf)):
        ops.gemm_persistent(a, w, bias, out, M, act, feature_tile=tile)
        ref = torch.from_numpy(fn((base + bias.double()).cpu().numpy())).to(dev)
        assert (out.double() - ref).abs().max().item() <= tol * scale, act
    if out_dtype == torch.float32:
        out2 = res.clone()
        ops.gemm_persistent(a, w, bias, out2, M, "none", residual=out2, feature_tile=tile)
        assert (out2.double() - (base + bias.double() + res.double())).abs().max().item() <= tol * scale
        same = torch.empty_like(out2)
        ops.gemm_tcgen05(a, w, bias, same, M, "none", residual=res)
        assert (out2 - same).abs().max().item() <= 1e-5 * scale          # the one-tile kernel agrees
    # a view with a row stride and fewer rows than the buffer holds: rows past M stay as they were
    wide = torch.zeros((M + 3, K + 8), dtype=torch.bfloat16, device=dev)
    wide[:M, :K] = a
    out3 = torch.full((M + 3, N), 7.0, dtype=out_dtype, device=dev)
    ops.gemm_persistent(wide[:, :K], w, None, out3, M, feature_tile=tile)
    assert (out3[:M].double() - base).abs().max().item() <= tol * scale and (out3[M:] == 7.0).all()
    assert ops.device_status() == 0


@pytest.mark.parametrize("out_dtype,M,N,K", [
    (torch.float32, 17, 768, 768), (torch.float32, 64, 768, 3072), (torch.float32, 33, 1000, 200), (torch.float32, 48, 36, 4096),
    (torch.float32, 50, 130, 1032), (torch.bfloat16, 64, 2304, 768), (torch.bfloat16, 40, 3072, 768), (torch.bfloat16, 25, 4800, 1600),
    (torch.bfloat16, 64, 72, 328), (torch.bfloat16, 18, 5000, 2048), (torch.bfloat16, 1, 2304, 768), (torch.float32, 8, 768, 768),
    (torch.bfloat16, 16, 3072, 1024), (torch.float32, 5, 130, 72), (torch.float32, 8, 768, 3072), (torch.bfloat16, 3, 1024, 4096),
    (torch.float32, 16, 1600, 1600), (torch.bfloat16, 8, 4800, 1600), (torch.float32, 4, 2500, 4096), (torch.bfloat16, 16, 9000, 768),
    (torch.float32, 2, 3840, 1280)])
def test_gemm_rows(dev, out_dtype, M, N, K):
    """The one-launch product for 1 to 64 tokens against float64: every number of token tiles and of groups per
    pass, several passes per block, ragged edges in M, N and K, all epilogues, the residual in place, a strided
    input; and a row's bits do not depend on how many rows share the launch."""
    from liyab_b200 import ops
    a, w = _rand((M, K), 46, dev, torch.bfloat16), _rand((N, K), 47, dev, torch.bfloat16, 0.2)
    bias, res = _rand((N,), 48, dev), _rand((M, N), 49, dev)
    assert ops.gemm_rows_supports(a, w, M)
    base = a.double() @ w.double().t()
    scale = max(1.0, base.abs().max().item())
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
    ops.gemm_rows(a, w, None, out, M)
    assert (out.double() - base).abs().max().item() <= tol * scale
    for act, fn in (("gelu_tanh", plain.gelu_tanh), ("gelu_erf", plain.gelu_erf)):
        ops.gemm_rows(a, w, bias, out, M, act)
        ref = torch.from_numpy(fn((base + bias.double()).cpu().numpy())).to(dev)
        assert (out.double() - ref).abs().max().item() <= tol * scale, act
    if out_dtype == torch.float32:
        out2 = res.clone()
        ops.gemm_rows(a, w, bias, out2, M, "none", residual=out2)
        assert (out2.double() - (base + bias.double() + res.double())).abs().max().item() <= tol * scale
        n_few = 17 if M > 17 else max(1, M - 3)
        fewer = torch.empty((n_few, N), dtype=out_dtype, device=dev)
        ops.gemm_rows(a[:n_few], w, bias, fewer, n_few, "none", residual=res[:n_few])
        assert torch.equal(fewer, out2[:n_few])
    wide = torch.zeros((M + 3, K + 8), dtype=torch.bfloat16, device=dev)
    wide[:M, :K] = a
    out3 = torch.full((M + 3, N), 7.0, dtype=out_dtype, device=dev)
    ops.gemm_rows(wide[:, :K], w, None, out3, M)
    assert (out3[:M].double() - base).abs().max().item() <= tol * scale and (out3[M:] == 7.0).all()


def test_gemm_rows_writes_keys_and_values_into_their_pages(dev):
    """A fused query/key/value projection whose epilogue also fills the cache, against the product followed by
    lb_kv_append: the same bits in the cache, tokens with a negative slot left out, other pages untouched."""
    from liyab_b200 import ops
    M, n_head, n_kv_head, head_dim, page_size, n_pages, K = 37, 6, 2, 64, 16, 9, 520
    q_dim, kv_dim = n_head * head_dim, n_kv_head * head_dim
    a, w = _rand((M, K), 56, dev, torch.bfloat16), _rand((q_dim + 2 * kv_dim, K), 57, dev, torch.bfloat16, 0.2)
    bias = _rand((q_dim + 2 * kv_dim,), 58, dev)
    rng = np.random.default_rng(5)
    slots = rng.permutation(n_pages * page_size)[:M].astype(np.int32)
    slots[[3, 20]] = -1
    slot_mapping = torch.from_numpy(slots).to(dev)
    want_cache = torch.full((n_pages, 2, n_kv_head, page_size, head_dim), 3.0, dtype=torch.bfloat16, device=dev)
    got_cache = want_cache.clone()
    want = torch.empty((M, q_dim + 2 * kv_dim), dtype=torch.bfloat16, device=dev)
    ops.gemm_rows(a, w, bias, want, M)
    ops.kv_append(want[:, q_dim:q_dim + kv_dim], want[:, q_dim + kv_dim:], slot_mapping, want_cache, M, n_kv_head, head_dim, page_size)
    got = torch.empty_like(want)
    ops.gemm_rows(a, w, bias, got, M, kv=(got_cache, slot_mapping, q_dim, n_kv_head, head_dim, page_size))
    assert torch.equal(got, want) and torch.equal(got_cache, want_cache)
    assert (got_cache != 3.0).any()


def test_gemm_rows_refuses_what_it_cannot_take(dev):
    from liyab_b200 import ops, LiyabError
    a, w = _rand((64, 4104), 1, dev, torch.bfloat16), _rand((16, 4104), 2, dev, torch.bfloat16)
    assert not ops.gemm_rows_supports(a, w, 64)                # a reduction length past 4096
    assert ops.gemm_rows_supports(a[:, :768], w[:, :768], 16) and ops.gemm_rows_supports(a[:, :768], w[:, :768], 1)
    assert not ops.gemm_rows_supports(a[:, :768], w[:, :768], 0) and not ops.gemm_rows_supports(a[:, :768], w[:, :768], 65)
    big = _rand((50304, 64), 3, dev, torch.bfloat16)
    assert not ops.gemm_rows_supports(a[:, :64].contiguous(), big, 64)          # a vocabulary: too many groups per block
    with pytest.raises(LiyabError):
        ops.gemm_rows(a, w, None, torch.empty((64, 16), dtype=torch.float32, device=dev), 64)


@pytest.mark.parametrize("M,n_head,n_kv_head,head_dim,page_size,tile", [
    (300, 6, 2, 64, 16, 0), (300, 6, 2, 64, 16, 64), (1000, 3, 3, 128, 32, 192), (130, 5, 1, 64, 64, 0)])
def test_gemm_persistent_writes_keys_and_values_into_their_pages(dev, M, n_head, n_kv_head, head_dim, page_size, tile):
    """The fused projection of many tokens with the cache filled from the epilogue, against the product followed by
    lb_kv_append: the same queries, the same bits in the cache, tokens with a negative slot left out, other slots
    untouched; the key and value columns of `out` are left alone."""
    from liyab_b200 import ops
    K = 264
    q_dim, kv_dim = n_head * head_dim, n_kv_head * head_dim
    N = q_dim + 2 * kv_dim
    n_pages = (M + page_size - 1) // page_size + 3
    a, w = _rand((M, K), 66, dev, torch.bfloat16), _rand((N, K), 67, dev, torch.bfloat16, 0.2)
    bias = _rand((N,), 68, dev)
    rng = np.random.default_rng(6)
    slots = rng.permutation(n_pages * page_size)[:M].astype(np.int32)
    slots[[3, 20, M - 1]] = -1
    slot_mapping = torch.from_numpy(slots).to(dev)
    want_cache = torch.full((n_pages, 2, n_kv_head, page_size, head_dim), 3.0, dtype=torch.bfloat16, device=dev)
    got_cache = want_cache.clone()
    want = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    ops.gemm_persistent(a, w, bias, want, M, feature_tile=tile)
    ops.kv_append(want[:, q_dim:q_dim + kv_dim], want[:, q_dim + kv_dim:], slot_mapping, want_cache, M, n_kv_head, head_dim, page_size)
    assert ops.gemm_persistent_kv_supports(w, want, q_dim, n_kv_head, head_dim, page_size)
    got = torch.full_like(want, 5.0)
    ops.gemm_persistent(a, w, bias, got, M, feature_tile=tile, kv=(got_cache, slot_mapping, q_dim, n_kv_head, head_dim, page_size))
    assert ops.device_status() == 0
    assert torch.equal(got[:, :q_dim], want[:, :q_dim]) and (got[:, q_dim:] == 5.0).all()
    assert torch.equal(got_cache, want_cache) and (got_cache != 3.0).any()


def test_gemm_persistent_refuses_what_it_cannot_take(dev):
    from liyab_b200 import ops, LiyabError
    a, w = _rand((100, 64), 1, dev, torch.bfloat16), _rand((50, 64), 2, dev, torch.bfloat16)
    odd = torch.empty((100, 50), dtype=torch.bfloat16, device=dev)           # rows of 100 bytes: off TMA's 16-byte rule
    assert ops.gemm_persistent_tile(a, w, odd, 100) == 0
    with pytest.raises(LiyabError):
        ops.gemm_persistent(a, w, None, odd, 100)
    # keys and values go to the cache only in strips of 64 features that lie inside one head
    w2, out2 = _rand((3 * 96, 64), 3, dev, torch.bfloat16), torch.empty((100, 3 * 96), dtype=torch.bfloat16, device=dev)
    assert not ops.gemm_persistent_kv_supports(w2, out2, 96, 1, 96, 16)
    cache = torch.zeros((8, 2, 1, 16, 96), dtype=torch.bfloat16, device=dev)
    with pytest.raises(LiyabError):
        ops.gemm_persistent(a, w2, None, out2, 100, kv=(cache, torch.zeros(100, dtype=torch.int32, device=dev), 96, 1, 96, 16))
    ops.linear(a, w, None, odd, 100)                                         # the dispatcher takes the one-tile kernel
    assert (odd.double() - a.double() @ w.double().t()).abs().max().item() < 0.1
    few = torch.empty((64, 50), dtype=torch.float32, device=dev)
    assert ops.gemm_persistent_tile(a[:64], w, few, 64) == 0                  # 64 tokens or fewer: weights on the lanes


def test_gemm_tcgen05_refuses_what_tma_cannot_fetch(dev):
    from liyab_b200 import ops, LiyabError
    a, w = _rand((4, 100), 1, dev, torch.bfloat16), _rand((8, 100), 2, dev, torch.bfloat16)
    out = torch.empty((4, 8), dtype=torch.bfloat16, device=dev)
    assert not ops.tcgen05_accepts(a, w)
    with pytest.raises(LiyabError):
        ops.gemm_tcgen05(a, w, None, out, 4)
    ops.linear(a, w, None, out, 4)          # the dispatcher falls back to the 32-bit units
    assert (out.double() - a.double() @ w.double().t()).abs().max().item() < 0.1


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window,splits", [
    (12, 12, 64, 16, 0, 1), (12, 12, 64, 16, 0, 5), (4, 4, 16, 16, 0, 3), (3, 3, 32, 32, 0, 32), (8, 2, 128, 16, 0, 4),
    (16, 2, 64, 64, 0, 7), (2, 1, 256, 16, 0, 2), (6, 3, 64, 16, 33, 4), (4, 4, 32, 16, 5, 16), (32, 2, 64, 16, 0, 3),
    (5, 5, 128, 32, 70, 2), (16, 1, 128, 16, 0, 1), (12, 12, 64, 16, 0, 12), (16, 1, 128, 16, 0, 8), (12, 12, 64, 16, 0, 8)])
def test_decode_attention(dev, n_head, n_kv_head, head_dim, page_size, window, splits):
    """One new token per request over its pages, keys split several ways (two to eight ranges merge inside a
    cluster, more through global memory), against float64; the same scratch is used by two launches in a row (the
    kernel must leave its counters at zero)."""
    from liyab_b200 import ops
    scalar, tensor = ops.decode_attention_kernels(n_head, n_kv_head, head_dim, page_size)
    assert scalar or tensor
    lens = [1, 2, 17, 64, 65, 300, 1024, 33]
    scale = 0.5 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, torch.bfloat16, n_head, n_kv_head, head_dim, page_size,
                                                            lens, [1] * len(lens), seed=7 * head_dim + splits)
    S = len(lens)
    partial = torch.full((S * n_head * splits * (head_dim + 2),), float("nan"), device=dev)
    counters = torch.zeros(S * n_kv_head, dtype=torch.int32, device=dev)
    ref = _attention_reference(refs, n_head, n_kv_head, scale, window)
    kinds = ([False] if scalar else []) + ([True] if tensor else [])
    for tensor_cores in kinds + kinds:          # each kernel twice over the same scratch
        out = torch.full_like(q, float("nan"))
        ops.decode_attention(q, cache, positions, table, out, partial, counters, S, n_head, n_kv_head, head_dim,
                             page_size, scale, window, splits, tensor_cores=tensor_cores)
        assert (out.double().cpu() - ref).abs().max().item() < 1.5e-2, f"tensor_cores={tensor_cores}"
        assert int(counters.abs().sum()) == 0
    generic = torch.empty_like(q)
    ops.paged_attention_generic(q, cache, tok_seq, positions, table, generic, S, n_head, n_kv_head, head_dim, page_size,
                                scale, window)
    assert (out.float() - generic.float()).abs().max().item() < 1.5e-2


def test_decode_attention_finds_a_far_key(dev):
    from liyab_b200 import ops
    n_head, n_kv_head, head_dim, page_size = 4, 2, 64, 16
    for key_pos, splits in ((0, 4), (15, 1), (16, 9), (271, 4), (1023, 32), (511, 3)):
        q, cache, _, positions, table, refs = _paged_case(dev, torch.bfloat16, n_head, n_kv_head, head_dim, page_size,
                                                          [1024], [1], seed=key_pos, boost=(key_pos, 4.0))
        partial = torch.zeros(n_head * splits * (head_dim + 2), device=dev)
        counters = torch.zeros(n_kv_head, dtype=torch.int32, device=dev)
        ref = _attention_reference(refs, n_head, n_kv_head, 1.0 / math.sqrt(head_dim), 0)
        for tensor_cores in (False, True):
            out = torch.empty_like(q)
            ops.decode_attention(q, cache, positions, table, out, partial, counters, 1, n_head, n_kv_head, head_dim,
                                 page_size, 1.0 / math.sqrt(head_dim), 0, splits, tensor_cores=tensor_cores)
            assert (out.double().cpu() - ref).abs().max().item() < 1.5e-2, f"far key at {key_pos}, tensor_cores={tensor_cores}"


@pytest.mark.parametrize("n_head,n_kv_head,head_dim,page_size,window", [
    (12, 12, 64, 16, 0), (4, 4, 16, 16, 0), (3, 3, 32, 16, 0), (6, 2, 48, 32, 0), (5, 1, 64, 64, 0), (2, 2, 128, 16, 0),
    (7, 7, 80, 16, 0), (4, 2, 96, 8, 0), (2, 1, 112, 16, 0), (4, 4, 32, 16, 40), (2, 1, 64, 32, 7), (3, 3, 64, 16, 100)])
def test_prefill_attention(dev, n_head, n_kv_head, head_dim, page_size, window):
    """Prompt portions of every kind in one launch: a whole prompt, a portion that continues a long
    context, single tokens, two-token portions, portions that end inside a page and a tile."""
    from liyab_b200 import ops
    assert ops.prefill_attention_supports(n_head, n_kv_head, head_dim, page_size)
    lens = [1, 37, 130, 64, 300, 2, 129, 1024]
    q_lens = [1, 37, 2, 1, 45, 2, 65, 200]
    scale = 0.6 / math.sqrt(head_dim)
    q, cache, tok_seq, positions, table, refs = _paged_case(dev, torch.bfloat16, n_head, n_kv_head, head_dim, page_size,
                                                            lens, q_lens, seed=head_dim + n_head + window)
    q_start = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=dev)
    n_past = torch.tensor([l - ql for l, ql in zip(lens, q_lens)], dtype=torch.int32, device=dev)
    ref = _attention_reference(refs, n_head, n_kv_head, scale, window)
    kinds = [False] + ([True] if ops.prefill_attention_tc_supports(n_head, n_kv_head, head_dim, page_size) else [])
    for tcgen05 in kinds:
        out = torch.full_like(q, float("nan"))
        ops.prefill_attention(q, cache, q_start, n_past, table, out, len(lens), max(q_lens), n_head, n_kv_head, head_dim,
                              page_size, scale, window, tcgen05=tcgen05)
        assert ops.device_status() == 0
        err = (out.double().cpu() - ref).abs().max().item()
        assert err < 1.5e-2, (tcgen05, err)


def test_prefill_attention_finds_a_far_key_and_the_diagonal(dev):
    """A key scaled so that its score stands out, placed at a page's edge, a tile's edge, position 0 and on the
    diagonal of the last query: dropping a tile, a page or the query's own key shows."""
    from liyab_b200 import ops
    n_head, n_kv_head, head_dim, page_size = 4, 2, 64, 16
    for key_pos in (0, 15, 16, 63, 64, 271, 511):
        q, cache, _, _, table, refs = _paged_case(dev, torch.bfloat16, n_head, n_kv_head, head_dim, page_size, [512], [100],
                                                  seed=key_pos, boost=(key_pos, 4.0))
        q_start = torch.tensor([0, 100], dtype=torch.int32, device=dev)
        n_past = torch.tensor([412], dtype=torch.int32, device=dev)
        ref = _attention_reference(refs, n_head, n_kv_head, 1.0 / math.sqrt(head_dim), 0)
        for tcgen05 in (False, True):
            out = torch.empty_like(q)
            ops.prefill_attention(q, cache, q_start, n_past, table, out, 1, 100, n_head, n_kv_head, head_dim, page_size,
                                  1.0 / math.sqrt(head_dim), 0, tcgen05=tcgen05)
            assert (out.double().cpu() - ref).abs().max().item() < 1.5e-2, f"far key at {key_pos}, tcgen05={tcgen05}"


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K,splits", [(64, 768, 3072, 16), (17, 768, 768, 12), (33, 2304, 768, 6), (5, 1000, 200, 4),
                                          (64, 130, 4096, 7), (20, 256, 64, 5)])
def test_gemm_tcgen05_split_k(dev, out_dtype, M, N, K, splits):
    """K split over blocks (few tokens): same result as unsplit to rounding, the same bits on a second call
    (the splits are summed in order), counters left at zero, residual in place."""
    from liyab_b200 import ops
    a, w = _rand((M, K), 26, dev, torch.bfloat16), _rand((N, K), 27, dev, torch.bfloat16, 0.2)
    bias, res = _rand((N,), 28, dev), _rand((M, N), 29, dev)
    partial = torch.full((splits * M * N,), float("nan"), device=dev)
    counters = torch.zeros(-(-N // 128), dtype=torch.int32, device=dev)
    ref = torch.from_numpy(plain.gelu_tanh((a.double() @ w.double().t() + bias.double()).cpu().numpy())).to(dev)
    scale = max(1.0, ref.abs().max().item())
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    outs = []
    for _ in range(2):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
        ops.gemm_tcgen05(a, w, bias, out, M, "gelu_tanh", partial=partial, counters=counters, n_splits=splits)
        assert (out.double() - ref).abs().max().item() <= tol * scale
        assert ops.device_status() == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    if out_dtype == torch.float32:
        x = res.clone()
        ops.gemm_tcgen05(a, w, bias, x, M, "none", residual=x, partial=partial, counters=counters, n_splits=splits)
        want = a.double() @ w.double().t() + bias.double() + res.double()
        assert (x.double() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("out_dtype,M,N,K", [
    (torch.bfloat16, 8, 2304, 768), (torch.bfloat16, 1, 130, 72), (torch.bfloat16, 16, 3072, 1024), (torch.float32, 5, 768, 768),
    (torch.float32, 13, 1000, 328), (torch.bfloat16, 9, 4096, 1024)])
def test_gemm_rows_with_layernorm_made_in_the_kernel(dev, out_dtype, M, N, K):
    """The product of a few tokens whose activations are the LayerNorm of float32 rows, normalised by every block
    itself: as the LayerNorm kernel followed by the plain product (to a rounding of bfloat16 here and there: the two sum a
    row's statistics in different trees), and right against float64."""
    from liyab_b200 import ops
    x = _rand((M + 2, K + 8), 70, dev) * 3.0 + 0.5
    gain, offs = _rand((K,), 71, dev) * 0.1 + 1.0, _rand((K,), 72, dev) * 0.1
    w, bias = _rand((N, K), 73, dev, torch.bfloat16, 0.2), _rand((N,), 74, dev)
    res = _rand((M, N), 75, dev)
    eps = 1e-5
    normed = torch.empty((M, K), dtype=torch.bfloat16, device=dev)
    ops.layernorm(x[:M, :K].contiguous(), gain, offs, eps, normed, M)
    for act in ("none", "gelu_tanh"):
        want = torch.empty((M, N), dtype=out_dtype, device=dev)
        ops.gemm_rows(normed, w, bias, want, M, act)
        got = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
        ops.gemm_rows_normed(x[:, :K], gain, offs, eps, w, bias, got, M, act)
        assert (got.double() - want.double()).abs().max().item() <= 1e-2 * max(1.0, want.double().abs().max().item()), act
    xd = x[:M, :K].double()
    ref_normed = (xd - xd.mean(1, keepdim=True)) / torch.sqrt(xd.var(1, unbiased=False, keepdim=True) + eps) * gain.double() + offs.double()
    base = ref_normed.float().to(torch.bfloat16).double() @ w.double().t()
    scale = max(1.0, base.abs().max().item())
    if out_dtype == torch.float32:
        out2 = res.clone()
        ops.gemm_rows_normed(x[:, :K], gain, None, eps, w, bias, out2, M, "none", residual=out2)
        ref2 = ((xd - xd.mean(1, keepdim=True)) / torch.sqrt(xd.var(1, unbiased=False, keepdim=True) + eps) * gain.double())
        base2 = ref2.float().to(torch.bfloat16).double() @ w.double().t()
        assert (out2.double() - (base2 + bias.double() + res.double())).abs().max().item() <= 2e-3 * scale
    got = torch.empty((M, N), dtype=out_dtype, device=dev)
    ops.gemm_rows_normed(x[:, :K], gain, offs, eps, w, bias, got, M)
    assert (got.double() - (base + bias.double())).abs().max().item() <= (2e-3 if out_dtype == torch.float32 else 1e-2) * scale
