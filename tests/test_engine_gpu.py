"""Generation through the Python entry point and the command line, against the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_gpt2 as plain
from tiny_models import CONFIGS, random_tokens, write_model

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = str(tmp_path_factory.mktemp("engine_models"))
    return {(n, d): write_model(base, n, d) for n in ("A", "B") for d in ("float32", "bfloat16")}


def plain_sampled(model, prompt, params, stream, n_new):
    """The plain sampler on the plain model's logits, with the engine's documented draws."""
    tokens, out = list(prompt), []
    for i in range(n_new):
        logits = plain.forward_logits(model, tokens)[-1].astype(np.float32)
        probs = plain.sampler_probabilities(logits, params.temperature, params.top_k, params.top_p)
        nxt = int(np.argmax(probs)) if params.temperature <= 0 else plain.sampler_draw(probs, plain.uniform_draw(params.seed, stream, i))
        out.append(nxt)
        tokens.append(nxt)
    return out


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_config_a(folders, graphs):
    """Workload A: two prompts of 7 and 13 ids, 16 greedy steps, 32-bit."""
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    folder = folders[("A", "float32")]
    prompts = [random_tokens(1, 7, 512), random_tokens(2, 13, 512)]
    engine = Engine(EngineConfig(model=folder, dtype="float32", max_requests=4, max_batched_tokens=64, num_pages=16,
                                 cuda_graphs=graphs))
    got = engine.generate_batch(prompts, SamplingParams(temperature=0.0, max_tokens=16))
    oracle = plain.load_plain_model(folder)
    for p, r in zip(prompts, got):
        assert r.tokens == plain.generate_greedy(oracle, p, 16) and r.finish_reason == "length"
        assert r.stats.prompt_tokens == len(p) and r.stats.generated_tokens == 16
    assert (engine.stats()["graph_steps"] > 0) == graphs
    assert engine.stats()["pages_in_use"] == 0


def test_sampled_generation_config_b(folders):
    """Workload B: prompts of 1, 5, 33 and 70 ids, prefilled in portions of 16 beside decoding,
    24 steps at temperature 0.8 with sampler seed 7."""
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    folder = folders[("B", "float32")]
    prompts = [random_tokens(10 + i, n, 1000) for i, n in enumerate((1, 5, 33, 70))]
    params = SamplingParams(temperature=0.8, top_k=40, top_p=0.95, seed=7, max_tokens=24)
    engine = Engine(EngineConfig(model=folder, dtype="float32", max_requests=4, max_batched_tokens=16, num_pages=64))
    got = engine.generate_batch(prompts, params)
    oracle = plain.load_plain_model(folder)
    for stream, (p, r) in enumerate(zip(prompts, got)):
        assert r.tokens == plain_sampled(oracle, p, params, stream, 24)
    assert engine.stats()["prefill_tokens"] == 1 + 5 + 33 + 70
    # the same requests one at a time give the same tokens: a draw belongs to (seed, stream, index), not to a batch
    engine2 = Engine(EngineConfig(model=folder, dtype="float32", max_requests=1, max_batched_tokens=2048, num_pages=64))
    for stream, (p, r) in enumerate(zip(prompts, got)):
        alone = engine2.generate_tokens(p, params)
        assert alone.tokens == r.tokens


def test_preemption_does_not_change_the_tokens(folders):
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    folder = folders[("A", "float32")]
    prompts = [random_tokens(20 + i, n, 512) for i, n in enumerate((30, 25, 20))]
    params = SamplingParams(temperature=0.7, top_k=0, top_p=1.0, seed=3, max_tokens=40)
    roomy = Engine(EngineConfig(model=folder, dtype="float32", max_requests=4, max_batched_tokens=32, num_pages=64))
    want = [r.tokens for r in roomy.generate_batch(prompts, params)]
    tight = Engine(EngineConfig(model=folder, dtype="float32", max_requests=4, max_batched_tokens=32, num_pages=9))
    got = tight.generate_batch(prompts, params)
    assert tight.stats()["preemptions"] >= 1
    assert [r.tokens for r in got] == want
    assert tight.stats()["pages_in_use"] == 0


def test_bfloat16_generation_stays_close(folders):
    """In bfloat16 a near-tie may flip a token, so the check is on the logits the engine's own
    tokens lead to: at every step the chosen token's plain logit is within rounding of the best."""
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    folder = folders[("B", "bfloat16")]
    prompt = random_tokens(5, 40, 1000)
    engine = Engine(EngineConfig(model=folder, dtype="bfloat16", max_requests=2, max_batched_tokens=64, num_pages=32, fused_decode=True))
    out = engine.generate_tokens(prompt, SamplingParams(temperature=0.0, max_tokens=20)).tokens
    logits = plain.forward_logits(plain.load_plain_model(folder), prompt + out)
    for i, tok in enumerate(out):
        row = logits[len(prompt) - 1 + i]
        assert row.max() - row[tok] <= 2.5e-2 * np.abs(row).max()


def test_callback_stop_and_eos(folders, tmp_path):
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    folder = folders[("A", "float32")]
    engine = Engine(EngineConfig(model=folder, dtype="float32", max_requests=2, num_pages=16))
    prompt = random_tokens(1, 7, 512)
    ref = engine.generate_tokens(prompt, SamplingParams(temperature=0.0, max_tokens=10)).tokens
    seen = []
    r = engine.generate_tokens(prompt, SamplingParams(temperature=0.0, max_tokens=10),
                               callback=lambda t: seen.append(t) or len(seen) < 3)
    assert r.tokens == ref[:3] and r.finish_reason == "stopped" and seen == ref[:3]
    # a model whose eos is the token it generates third stops there unless told to ignore it
    cfg = json.load(open(os.path.join(folder, "config.json")))
    cfg["eos_token_id"] = ref[2]
    eos_folder = tmp_path / "eos"
    eos_folder.mkdir()
    (eos_folder / "config.json").write_text(json.dumps(cfg))
    os.symlink(os.path.join(folder, "model.safetensors"), eos_folder / "model.safetensors")
    e2 = Engine(EngineConfig(model=str(eos_folder), dtype="float32", max_requests=2, num_pages=16))
    first = ref.index(ref[2])
    r = e2.generate_tokens(prompt, SamplingParams(temperature=0.0, max_tokens=10))
    assert r.tokens == ref[:first + 1] and r.finish_reason == "eos"
    r = e2.generate_tokens(prompt, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    assert r.tokens == ref


def test_command_line(folders):
    folder = folders[("A", "float32")]
    prompt = random_tokens(1, 7, 512)
    cmd = [os.path.join(ROOT, "bin", "liyab-cli"), "-m", folder, "-p", ",".join(map(str, prompt)),
           "-n", "6", "--temp", "0", "--dtype", "float32", "--num-pages", "16", "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    assert "load_ms" in lines[0] and lines[1]["generated_tokens"] == 6
    assert lines[1]["tokens"] == plain.generate_greedy(plain.load_plain_model(folder), prompt, 6)
    proc = subprocess.run(cmd[:5] + ["--tokenize"], capture_output=True, text=True, timeout=600)
    assert proc.stdout.split() == [str(t) for t in prompt]
    # the summary on stderr: prompt / decode / memory lines, the decode phases when asked for, the scheduler's counters
    proc = subprocess.run(cmd[:-1] + ["--phases"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [str(t) for t in lines[1]["tokens"]]
    for needle in ("prompt: 7 tokens", "decode: 6 tokens", "memory: KV", "decode phases (ms/token): embed", "scheduler: 6 steps"):
        assert needle in proc.stderr, proc.stderr
    # a model folder that does not fit its configuration is refused with the loader's one message
    proc = subprocess.run([cmd[0], "-m", os.path.join(folder, "nowhere"), "-p", "1"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 1 and "config.json" in proc.stderr


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "bfloat16")])
def test_pipelined_and_stepwise_loops_give_the_same_tokens(name, dtype, tmp_path):
    """The host running one step ahead (tokens stay on the device) against waiting for every step: same tokens,
    same reasons, with sampling, an end-of-sequence token, a callback that stops and a tight cache."""
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    folder = write_model(str(tmp_path), name, dtype)
    V = CONFIGS[name][0]["vocab_size"]
    prompts = [random_tokens(40 + i, n, V) for i, n in enumerate((21, 3, 34, 9, 15))]
    params = [SamplingParams(temperature=0.9, top_k=50, top_p=0.9, seed=11 + i, max_tokens=30 + 3 * i) for i in range(5)]
    probe = Engine(EngineConfig(model=folder, dtype=dtype, max_requests=5, max_batched_tokens=24, num_pages=40, pipeline=False))
    first = probe.generate_batch(prompts, params)
    eos = first[1].tokens[7]                     # make a token that really occurs the end-of-sequence token
    cfg = json.load(open(os.path.join(folder, "config.json")))
    cfg["eos_token_id"] = eos
    eos_folder = tmp_path / "eos"
    eos_folder.mkdir()
    (eos_folder / "config.json").write_text(json.dumps(cfg))
    os.symlink(os.path.join(folder, "model.safetensors"), eos_folder / "model.safetensors")
    outs = []
    for pipeline in (False, True):
        for pages in (40, 8):
            engine = Engine(EngineConfig(model=str(eos_folder), dtype=dtype, max_requests=5, max_batched_tokens=24,
                                         num_pages=pages, pipeline=pipeline))
            seen = []
            callbacks = [None, None, (lambda t: seen.append(t) or len(seen) < 5), None, None]
            res = engine.generate_batch(prompts, params, callbacks)
            outs.append([(r.tokens, r.finish_reason) for r in res])
            assert engine.stats()["pages_in_use"] == 0
            if pages == 8:
                assert engine.stats()["preemptions"] >= 1
    if dtype == "float32":
        # In 32-bit a token's logits do not depend on the batch or the cut, so every way of running agrees exactly.
        assert outs[0] == outs[1] == outs[2] == outs[3]
        assert outs[0][1][1] == "eos" and outs[0][2] == (first[2].tokens[:5], "stopped")
    else:
        # In bfloat16 a changed batch (a request that ends a step later) may round a near-tie the other way, so
        # only what does not depend on rounding is compared: every request ends, for a reason that fits its tokens.
        for run in outs:
            assert run[2][1] == "stopped" and len(run[2][0]) == 5
            for (tokens, reason), p in zip(run, params):
                assert reason in ("eos", "length", "stopped") and 1 <= len(tokens) <= p.max_tokens
                assert (reason == "eos") == (tokens[-1] == eos) or reason == "stopped"


def test_a_reported_wait_ends_the_step_with_an_error_and_the_engine_goes_on(tmp_path):
    """A kernel whose bounded wait ran out leaves a status word; the engine reads the words with every step's ids.
    Here the word of the fused step's barrier is written by hand: the requests of the step that meets it end with
    INTERNAL and a message, the words are cleared, the one-kernel step is switched off, and the next call generates
    as before (part by part)."""
    from liyab_b200 import Engine, EngineConfig, ErrorCode, SamplingParams
    from liyab_b200.engine import device_status, set_device_status, set_log
    folder = write_model(str(tmp_path), "D", "bfloat16")
    prompt = random_tokens(5, 30, CONFIGS["D"][0]["vocab_size"])
    params = SamplingParams(temperature=0.0, max_tokens=12)
    engine = Engine(EngineConfig(model=folder, dtype="bfloat16", max_requests=2, max_batched_tokens=64, num_pages=32, fused_decode=True))
    good = engine.generate_tokens(prompt, params)
    assert good.error is None and engine.stats()["fused_steps"] > 0 and engine.stats()["device_faults"] == 0
    seen = []
    set_log(3, lambda level, message: seen.append((level, message)))
    try:
        set_device_status(1, 0x51)
        bad = engine.generate_tokens(prompt, params)
    finally:
        set_log(2, None)
    assert bad.error is not None and bad.error.code == ErrorCode.INTERNAL and "bounded wait" in bad.error.message
    assert bad.finish_reason == "error" and len(bad.tokens) < 12
    assert seen and seen[0][0] == 3 and "0x51" in seen[0][1]
    st = engine.stats()
    # The step that was already in flight when the word was read met it too (the host runs one step ahead).
    assert 1 <= st["device_faults"] <= 2 and st["pages_in_use"] == 0 and device_status() == (0, 0)
    fused_before = st["fused_steps"]
    again = engine.generate_tokens(prompt, params)
    assert again.error is None and again.finish_reason == "length" and len(again.tokens) == 12
    assert engine.stats()["fused_steps"] == fused_before, "the one-kernel step stays off after it reported a fault"
    logits = plain.forward_logits(plain.load_plain_model(folder), prompt + again.tokens)
    for i, tok in enumerate(again.tokens):
        row = logits[len(prompt) - 1 + i]
        assert row.max() - row[tok] <= 2.5e-2 * np.abs(row).max()
