"""The engine against the plain implementation where the tiny configurations do not reach: steps replayed from
captured CUDA graphs, the layer sizes the benchmark runs (GPT-2 small and XL widths, the 50,257-token vocabulary),
and bfloat16 steps of more than 64 tokens that hold prompt portions and decoded tokens together."""
from __future__ import annotations

import numpy as np
import pytest

import plain_gpt2 as plain
import trace_tools as tt
from tiny_models import CONFIGS, random_tokens, write_model

pytestmark = pytest.mark.gpu
REL_TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
BIG_REL_TOL = {"float32": 1e-4, "bfloat16": 2.5e-2}


def requests_for(name, lengths):
    raw, seed = CONFIGS[name]
    return {f"r{i}": random_tokens(300 * seed + i, n, raw["vocab_size"]) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16"), ("D", "bfloat16"), ("D", "float32")])
def test_replayed_graphs_give_the_same_logits(name, dtype, tmp_path):
    """Every cutting twice on one engine with graphs on: the second pass meets shapes that were captured during the
    first (decode steps at once, steps with portions at their third occurrence) and replays them."""
    from liyab_b200.engine import Replayer
    folder = write_model(str(tmp_path), name, dtype)
    P = CONFIGS[name][0]["n_positions"]
    reqs = requests_for(name, [P, 70, 33, 13, 7, 2, 1, 45])
    oracle = plain.load_plain_model(folder)
    want = {r: plain.forward_logits(oracle, toks) for r, toks in reqs.items()}
    engine = Replayer(folder, dtype, max_tokens=4 * 320, cuda_graphs=True, max_step_tokens=320, fused_decode=False)
    traces = [tt.tail_one_by_one(reqs, 32), tt.changing_portions(reqs), tt.mixed(reqs, max_live=4, seed=3), tt.whole(reqs)]
    first = None
    for trace in traces + traces:
        before = engine.counters()
        got = tt.collect(engine, trace)
        tt.check_rows(got, want, REL_TOL[dtype])
        if trace is traces[0]:
            if first is None:
                first = got
            elif dtype == "float32":         # a replayed step computes the same bits as the step it was captured from
                assert all(np.array_equal(first[k], got[k]) for k in first)
    c = engine.counters()
    assert c["graph_steps"] > 100 and c["graphs_captured"] > 5
    # the second pass replayed more than the first: by then every repeating shape had its graph
    assert c["graph_steps"] > c["eager_steps"]


def test_a_replay_with_shorter_portions_than_the_captured_step(tmp_path):
    """Steps of one shape (two requests, 19 tokens, all logits wanted) whose portions differ: (16, 3), (3, 16), (10, 9).
    The third is captured, the later ones replay it with other starts, lengths and a shorter longest portion."""
    from liyab_b200.engine import Replayer, StepEntry
    folder = write_model(str(tmp_path), "B", "float32")
    V = CONFIGS["B"][0]["vocab_size"]
    oracle = plain.load_plain_model(folder)
    engine = Replayer(folder, "float32", max_tokens=1024, cuda_graphs=True, max_step_tokens=64)
    toks = {r: random_tokens(77 + i, 120, V) for i, r in enumerate("ab")}
    want = {r: plain.forward_logits(oracle, t) for r, t in toks.items()}
    at = {"a": 0, "b": 0}
    for r in toks:
        engine.cache.open(r)
    for k, (na, nb) in enumerate([(16, 3), (3, 16), (10, 9), (9, 10), (16, 3), (1, 18), (18, 1), (7, 12)]):
        out = engine.step([StepEntry("a", toks["a"][at["a"]:at["a"] + na], list(range(na))),
                           StepEntry("b", toks["b"][at["b"]:at["b"] + nb], list(range(nb)))])
        rows = iter(out.logits)
        for r, n in (("a", na), ("b", nb)):
            for i in range(n):
                ref = want[r][at[r] + i]
                assert np.abs(next(rows) - ref).max() <= REL_TOL["float32"] * np.abs(want[r]).max(), (k, r, i)
            at[r] += n
    c = engine.counters()
    assert c["graphs_captured"] == 1 and c["graph_steps"] == 5 and c["eager_steps"] == 3


def test_bfloat16_steps_of_many_tokens_with_portions_and_decoded_tokens_together(tmp_path):
    """Head size 64, more than 64 tokens a step, portions beside single tokens: the projection that fills the cache
    from its epilogue and the tensor-core prefill attention with entries of one token."""
    from liyab_b200.engine import Replayer
    folder = write_model(str(tmp_path), "D", "bfloat16")
    reqs = requests_for("D", [130, 130, 290, 290])
    oracle = plain.load_plain_model(folder)
    want = {r: plain.forward_logits(oracle, toks) for r, toks in reqs.items()}
    # r0 and r1 bring 100 tokens each in one step and then go on one token a step; beside them r2 and r3 bring
    # their prompts in portions of 37 and 41 tokens: steps of 80 tokens, two of them single ones.
    at = {r: 0 for r in reqs}

    def take(r, n):
        n = min(n, len(reqs[r]) - at[r])
        entry = (r, reqs[r][at[r]:at[r] + n], list(range(n)))
        at[r] += n
        return entry

    steps = [([take("r0", 100), take("r1", 100)], [])]
    while any(at[r] < len(reqs[r]) for r in reqs):
        entries = [take(r, n) for r, n in (("r0", 1), ("r1", 1), ("r2", 37), ("r3", 41)) if at[r] < len(reqs[r])]
        steps.append((entries, [r for r, _, _ in entries if at[r] == len(reqs[r])]))
    both = [sum(len(t) for _, t, _ in e) for e, _ in steps if any(len(t) == 1 for _, t, _ in e) and any(len(t) > 1 for _, t, _ in e)]
    assert max(both) > 64 and sum(1 for n in both if n > 64) >= 5, "the trace must hold large steps of both kinds of entries"
    for graphs in (False, True):
        engine = Replayer(folder, "bfloat16", max_tokens=tt.peak_tokens(steps), cuda_graphs=graphs, max_step_tokens=256)
        got = tt.collect(engine, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        tt.check_rows(got, want, REL_TOL["bfloat16"], 1e-4, 0.99)


SMALL_WIDTH = dict(model_type="gpt2", n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024,
                   layer_norm_epsilon=1e-5, activation_function="gelu_new")
XL_WIDTH = dict(SMALL_WIDTH, n_embd=1600, n_head=25, n_inner=6400)


@pytest.mark.parametrize("label,raw,dtype", [
    ("small-2", dict(SMALL_WIDTH, n_layer=2), "float32"), ("small-2", dict(SMALL_WIDTH, n_layer=2), "bfloat16"),
    ("small-12", dict(SMALL_WIDTH, n_layer=12), "bfloat16"),
    ("xl-2", dict(XL_WIDTH, n_layer=2), "float32"), ("xl-2", dict(XL_WIDTH, n_layer=2), "bfloat16")])
def test_the_benchmark_layer_sizes_in_every_cutting(label, raw, dtype, tmp_path):
    """GPT-2 small's and XL's layer sizes (25 heads, a width of 1600, the vocabulary of 50,257) with random weights
    through whole / all-but-32 then singles / changing portions / mixed with page reuse, against the plain
    implementation in float64.  Logits are asked for at a fifth of the positions (each row is 50,257 numbers)."""
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import write_random_model
    folder = write_random_model(str(tmp_path / label), raw, seed=5, dtype=dtype)
    rng = np.random.default_rng(8)
    lengths = [200, 70, 33, 131, 2] if raw["n_layer"] <= 2 else [150, 40, 66]
    reqs = {f"r{i}": rng.integers(0, raw["vocab_size"], size=n).tolist() for i, n in enumerate(lengths)}
    oracle = plain.load_plain_model(folder)
    want = {r: plain.forward_logits(oracle, toks) for r, toks in reqs.items()}

    def keep(r, pos):
        return pos % 5 == 0 or pos >= len(reqs[r]) - 3

    n_rows = sum(1 for r, t in reqs.items() for pos in range(len(t)) if keep(r, pos))
    traces = {"whole": tt.whole(reqs), "tail": tt.tail_one_by_one(reqs, 32), "portions": tt.changing_portions(reqs, sizes=(64, 16, 8, 5, 3, 2, 2, 70, 2, 11)),
              "mixed": tt.mixed(reqs, max_live=4, seed=3, portion=40)}
    if raw["n_layer"] > 2:
        traces = {k: traces[k] for k in ("whole", "mixed")}
    results = {}
    for kind, steps in traces.items():
        steps = tt.thin(steps, keep)
        tokens = tt.peak_tokens(steps) if kind == "mixed" else 1024        # the mixed trace gets a pool for its own peak only
        engine = Replayer(folder, dtype, max_tokens=tokens, cuda_graphs=(kind == "mixed"), max_step_tokens=256,
                          fused_decode=(kind != "tail"))       # decode steps through the one kernel in all but one of the cuttings
        results[kind] = tt.collect(engine, steps)
        assert len(results[kind]) == n_rows
        if dtype == "bfloat16":
            stats = tt.check_rows(results[kind], want, BIG_REL_TOL[dtype], 1e-4, 0.99)
        else:
            stats = tt.check_rows(results[kind], want, BIG_REL_TOL[dtype])
        engine.close()
    if dtype == "float32":
        for kind in results:
            assert all(np.array_equal(row, results[kind][key]) for key, row in results["whole"].items()), f"{kind} differs from the whole run"


def test_the_one_kernel_step_is_taken_while_its_attention_fits_one_round(tmp_path):
    """Twelve heads: twelve decode tokens are 144 (token, head) pairs for 148 SMs and take the one-kernel step, fourteen
    would need a second round of its attention phase and go part by part (captured); both agree with the plain model."""
    from liyab_b200.engine import Replayer, StepEntry
    from liyab_b200.weights import write_random_model
    raw = dict(SMALL_WIDTH, n_layer=2)
    folder = write_random_model(str(tmp_path / "m"), raw, seed=9, dtype="bfloat16")
    oracle = plain.load_plain_model(folder)
    rng = np.random.default_rng(4)
    toks = {f"q{i}": rng.integers(0, raw["vocab_size"], size=5 + 3 * i).tolist() for i in range(14)}
    want = {r: plain.forward_logits(oracle, t) for r, t in toks.items()}
    for n, fused in ((12, True), (14, False)):
        engine = Replayer(folder, "bfloat16", max_tokens=16 * 128, max_requests=16, fused_decode=True)
        names = list(toks)[:n]
        for r in names:
            engine.cache.open(r)
            engine.step([StepEntry(r, toks[r][:-1], [])])
        out = engine.step([StepEntry(r, toks[r][-1:], [0]) for r in names]).logits
        assert (engine.counters()["fused_steps"] == 1) == fused
        for i, r in enumerate(names):
            assert np.abs(out[i] - want[r][-1]).max() <= BIG_REL_TOL["bfloat16"] * np.abs(want[r]).max(), (n, r)
        engine.close()
