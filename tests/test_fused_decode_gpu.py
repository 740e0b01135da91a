"""The one-kernel decode step against the plain implementation and against the part-by-part path."""
from __future__ import annotations

import numpy as np
import pytest

import plain_gpt2 as plain
import trace_tools as tt
from tiny_models import CONFIGS, random_tokens, write_model

pytestmark = pytest.mark.gpu
REL_TOL = 2.5e-2


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = str(tmp_path_factory.mktemp("fused_models"))
    return {n: write_model(base, n, "bfloat16") for n in ("D", "E")}


def requests_for(name):
    raw, seed = CONFIGS[name]
    P, V = raw["n_positions"], raw["vocab_size"]
    return {f"r{i}": random_tokens(50 * seed + i, n, V) for i, n in enumerate((P, 77, 40, 33, 150, 9))}


def decode_heavy(reqs, live=4):
    """Each request: a short prompt portion, then every further token alone, up to `live` requests side by side."""
    return tt.mixed(reqs, max_live=live, seed=11, prompt_frac=0.25)


@pytest.mark.parametrize("name", ["D", "E"])
def test_fused_decode_matches_plain_and_parts(name, folders):
    from liyab_b200.engine import Replayer, device_status
    reqs = requests_for(name)
    oracle = plain.load_plain_model(folders[name])
    want = {r: plain.forward_logits(oracle, toks) for r, toks in reqs.items()}
    steps = decode_heavy(reqs)
    results = {}
    for fused in (True, False):
        engine = Replayer(folders[name], "bfloat16", max_tokens=4 * 320, fused_decode=fused)
        assert engine.info["fused"] == fused
        results[fused] = tt.collect(engine, steps)
        if fused:
            assert engine.counters()["fused_steps"] > 50, "most steps of this trace are decode steps"
            assert device_status() == (0, 0)
    for (r, pos), row in results[True].items():
        scale = np.abs(want[r]).max()
        assert np.abs(row - want[r][pos]).max() <= REL_TOL * scale, (r, pos)
        assert np.abs(row - results[False][(r, pos)]).max() <= REL_TOL * scale, (r, pos)


def test_fused_decode_up_to_sixteen_requests_and_long_contexts(folders):
    """Sixteen requests decode side by side (the kernel's limit) at contexts from 1 to the model's last position."""
    from liyab_b200.engine import Replayer, StepEntry
    raw, _ = CONFIGS["D"]
    P, V = raw["n_positions"], raw["vocab_size"]
    stepper = Replayer(folders["D"], "bfloat16", max_tokens=17 * 320, max_requests=17, fused_decode=True)
    cache = stepper.cache
    oracle = plain.load_plain_model(folders["D"])
    lens = [1, 2, 15, 16, 17, 31, 64, 65, 100, 128, 129, 200, 255, 256, 290, P - 1]
    toks = {f"s{i}": random_tokens(900 + i, n + 1, V) for i, n in enumerate(lens)}
    for r, t in toks.items():
        cache.open(r)
        stepper.step([StepEntry(r, t[:-1], [])])
    out = stepper.step([StepEntry(r, [t[-1]], [0]) for r, t in toks.items()])
    assert stepper.counters()["fused_steps"] == 1
    got = out.logits
    for i, (r, t) in enumerate(toks.items()):
        ref = plain.forward_logits(oracle, t)
        assert np.abs(got[i] - ref[-1]).max() <= REL_TOL * np.abs(ref).max(), r
    # seventeen requests are one too many for the kernel: the step takes the other path and still agrees
    cache.open("extra")
    extra = random_tokens(5, 10, V)
    stepper.step([StepEntry("extra", extra[:-1], [])])
    for r in toks:
        cache.truncate(r, len(toks[r]) - 1)
    out = stepper.step([StepEntry(r, [t[-1]], [0]) for r, t in toks.items()] + [StepEntry("extra", [extra[-1]], [0])])
    assert stepper.counters()["fused_steps"] == 1
    got2 = out.logits
    assert np.abs(got2[:16] - got).max() <= REL_TOL * np.abs(got).max()


@pytest.mark.parametrize("name", ["D", "E"])
@pytest.mark.parametrize("graphs", [False, True])
def test_decode_steps_of_dozens_of_requests(name, graphs, folders):
    """Forty requests decode side by side for several steps (too many for the one-kernel step: the products of 17
    to 64 tokens, the projection that fills the cache from its epilogue and the tensor-core decode attention), with
    prompts added in groups while others are live; every logit against the plain implementation."""
    from liyab_b200.engine import Replayer, StepEntry
    raw, seed = CONFIGS[name]
    V = raw["vocab_size"]
    stepper = Replayer(folders[name], "bfloat16", max_tokens=42 * 128, max_requests=42, cuda_graphs=graphs)
    cache = stepper.cache
    oracle = plain.load_plain_model(folders[name])
    n_new = 4
    toks = {f"q{i}": random_tokens(700 + 40 * seed + i, 3 + (i * 7) % 90 + n_new, V) for i in range(40)}
    names = list(toks)
    got = {r: [] for r in names}
    for lo in range(0, 40, 13):                        # prompts in groups of 13, beside nothing else
        group = names[lo:lo + 13]
        for r in group:
            cache.open(r)
        out = stepper.step([StepEntry(r, toks[r][:-n_new], [len(toks[r]) - n_new - 1]) for r in group])
        for r, row in zip(group, out.logits):
            got[r].append(row)
    for k in range(n_new - 1):
        out = stepper.step([StepEntry(r, [toks[r][len(toks[r]) - n_new + k]], [0]) for r in names])
        for r, row in zip(names, out.logits):
            got[r].append(row)
    assert stepper.counters()["fused_steps"] == 0 and (stepper.counters()["graph_steps"] > 0) == graphs
    for r in names:
        ref = plain.forward_logits(oracle, toks[r][:-1])
        first = len(toks[r]) - n_new - 1
        for k, row in enumerate(got[r]):
            assert np.abs(row - ref[first + k]).max() <= REL_TOL * np.abs(ref).max(), (r, k)


def test_models_of_other_parts_do_not_take_the_fused_path(tmp_path):
    from liyab_b200.engine import Replayer
    on = dict(max_tokens=256, fused_decode=True)
    assert not Replayer(write_model(str(tmp_path), "B", "bfloat16"), "bfloat16", **on).info["fused"]    # head size 32 is not one the kernel takes
    assert not Replayer(write_model(str(tmp_path), "D", "float32"), "float32", **on).info["fused"]      # the 32-bit engine keeps its part-by-part kernels
    assert Replayer(write_model(str(tmp_path), "D", "bfloat16"), "bfloat16", **on).info["fused"]
    assert not Replayer(write_model(str(tmp_path), "D", "bfloat16"), "bfloat16", max_tokens=256).info["fused"]     # it is an option, off unless asked for
