"""A wait inside a kernel that nothing ends runs to its limit, reports it and lets the kernel return.

The failure is made on the host's order and faults nothing: one launch is told to leave a barrier one signal
short (the tensor-core product's accumulator-ready barrier; one block's arrival at the fused step's first grid
barrier).  The waiting threads poll to their limit of about two seconds, write the status word and go to the
kernel's end, where tensor memory is given back.  The tests check the word, that the device still computes right
results afterwards, and what the engine does with a step that reported one."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from tiny_models import CONFIGS, random_tokens, write_model

pytestmark = pytest.mark.gpu
REL_TOL = 2.5e-2


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return write_model(str(tmp_path_factory.mktemp("wait_models")), "D", "bfloat16")


@pytest.fixture(autouse=True)
def no_order_left_behind():
    """An order that no launch used (a test that failed early) does not reach the next test."""
    from liyab_b200.engine import device_status, withhold_next
    yield
    withhold_next(0, False)
    withhold_next(1, False)
    device_status()


def test_product_whose_accumulator_is_never_reported_gives_up_and_the_next_one_is_right():
    from liyab_b200 import ops
    from liyab_b200.engine import device_status, withhold_next
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    M, N, K = 8, 256, 320
    a = torch.randn((M, K), generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn((N, K), generator=g) * 0.2).to(torch.bfloat16).to(dev)
    want = a.double() @ w.double().t()
    out = torch.zeros((M, N), dtype=torch.float32, device=dev)
    assert device_status() == (0, 0)
    withhold_next(0)
    ops.gemm_tcgen05(a, w, None, out, M)
    torch.cuda.synchronize()
    word, barrier = device_status()
    assert word >> 8 == 3 and 0 <= (word & 0xFF) < 4, f"the epilogue's wait reports itself (site 3, its quarter): {word:#x}"
    assert barrier == 0
    # The order held for one launch; the device, its tensor memory included, serves the next one.
    for _ in range(3):
        out.fill_(float("nan"))
        ops.gemm_tcgen05(a, w, None, out, M)
        torch.cuda.synchronize()
        assert (out.double() - want).abs().max().item() <= 1e-5 * max(1.0, want.abs().max().item())
    assert device_status() == (0, 0)


def test_fused_step_whose_barrier_is_one_block_short_gives_up_and_later_steps_are_right(folder):
    from liyab_b200.engine import Replayer, StepEntry, device_status, withhold_next
    raw, seed = CONFIGS["D"]
    V = raw["vocab_size"]
    toks = random_tokens(900 + seed, 40, V)
    want = plain.forward_logits(plain.load_plain_model(folder), toks)
    scale = np.abs(want).max()
    engine = Replayer(folder, "bfloat16", max_tokens=256, fused_decode=True, cuda_graphs=False)
    engine.cache.open("a")
    engine.step([StepEntry("a", toks[:30], [29])])
    assert device_status() == (0, 0)
    before = engine.counters()["fused_steps"]
    withhold_next(1)
    engine.step([StepEntry("a", toks[30:31], [0])])
    assert engine.counters()["fused_steps"] == before + 1, "the step of one token is the one-kernel step"
    word, barrier = device_status()
    assert word == 0 and barrier == 1, f"the first grid barrier (code 1) reports itself: {barrier:#x}"
    # What that step left in the cache is not to be trusted: the request ends, and a new one is right on both paths.
    engine.cache.close("a")
    engine.cache.open("b")
    rows = engine.step([StepEntry("b", toks[:30], [29])]).logits
    assert np.abs(rows[0] - want[29]).max() <= REL_TOL * scale
    for i in range(30, 40):
        rows = engine.step([StepEntry("b", toks[i:i + 1], [0])]).logits
        assert np.abs(rows[0] - want[i]).max() <= REL_TOL * scale, i
    assert engine.counters()["fused_steps"] == before + 11
    assert device_status() == (0, 0)


def test_engine_ends_the_requests_of_a_step_whose_wait_ran_out_and_goes_on(tmp_path):
    from liyab_b200 import ErrorCode
    from liyab_b200.engine import Engine, EngineConfig, device_status, withhold_next
    from liyab_b200.sampling import SamplingParams
    from liyab_b200.weights import write_random_model
    # A vocabulary of 20,000: the head of a decode step is then a tcgen05 product (the one-launch mma.sync kernel takes
    # the layers' projections but not that many features), the family whose wait this test makes run out.
    raw, seed = dict(CONFIGS["D"][0], vocab_size=20000), CONFIGS["D"][1]
    folder = write_random_model(str(tmp_path / "m"), raw, seed=seed, dtype="bfloat16")
    prompt = random_tokens(77 + seed, 5, raw["vocab_size"])
    params = SamplingParams(temperature=0.0, max_tokens=8)
    engine = Engine(EngineConfig(model=folder, dtype="bfloat16", max_requests=2, max_batched_tokens=64, num_pages=32, fused_decode=True))
    good = engine.generate_tokens(prompt, params)
    assert good.error is None and len(good.tokens) == 8
    withhold_next(0)
    bad = engine.generate_tokens(prompt, params)
    assert bad.error is not None and bad.error.code == ErrorCode.INTERNAL and "bounded wait" in bad.error.message
    assert bad.finish_reason == "error"
    st = engine.stats()
    assert 1 <= st["device_faults"] <= 2 and st["pages_in_use"] == 0 and device_status() == (0, 0)
    again = engine.generate_tokens(prompt, params)
    assert again.error is None and again.tokens == good.tokens
    assert engine.stats()["fused_steps"] > st["fused_steps"], "a product's fault leaves the one-kernel step in use"
