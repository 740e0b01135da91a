"""Each part alone against the plain functions, and the framework's generality: a toy mixer with state of its own
is registered from outside the framework (tests/toy_parts, a plug-in built against the host's headers), built into
a model beside attention layers (one layer run twice, one run reading another run's cache) and stepped, without a
change to the framework; and so are a feed-forward with routing, a position encoding without a table, a norm, two
arrangements of a block (one with a third norm) and a whole architecture with config.json keys of its own."""
from __future__ import annotations

import json
import os
import subprocess

import numpy as np
import pytest

import plain_gpt2 as plain
import trace_tools as tt

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def toy_plugin(tmp_path_factory):
    """Builds tests/toy_parts into a shared object and registers its parts with the library."""
    from liyab_b200.config import load_plugin
    from liyab_b200.csrc.build import cuda_include, find_cxx, find_nvcc
    out = str(tmp_path_factory.mktemp("toy_parts"))
    nvcc, cxx = find_nvcc(), find_cxx()
    arch = ["-gencode", "arch=compute_100a,code=sm_100a"]
    src = os.path.join(HERE, "toy_parts")
    subprocess.run([nvcc, *arch, "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-c", os.path.join(src, "toy_kernels.cu"), "-o",
                    os.path.join(out, "toy_kernels.o")], check=True)
    subprocess.run([cxx, "-std=c++20", "-O2", "-fPIC", "-I", os.path.join(ROOT, "liyab_b200", "host"), "-I", cuda_include(nvcc), "-c",
                    os.path.join(src, "toy_parts.cpp"), "-o", os.path.join(out, "toy_parts.o")], check=True)
    lib = os.path.join(out, "toy_parts.so")
    subprocess.run([nvcc, *arch, "-shared", "-o", lib, os.path.join(out, "toy_kernels.o"), os.path.join(out, "toy_parts.o")], check=True)
    load_plugin(lib)
    return lib


# ---- models as data ----------------------------------------------------------------------------------------------

def layernorm(size, eps=1e-5):
    return {"kind": "layernorm", "size": size, "eps": eps}


def attention(hidden, n_head, n_kv_head, head_dim, scale, window=0):
    return {"kind": "attention", "hidden": hidden, "n_head": n_head, "n_kv_head": n_kv_head, "head_dim": head_dim, "scale": scale, "window": window}


def dense(hidden, inner, activation):
    return {"kind": "dense", "hidden": hidden, "inner": inner, "activation": activation}


def layer(arrangement, **slots):
    roles = {"mixer": "mixer", "feed_forward": "feed_forward"}
    return {"arrangement": arrangement, "slots": [{"name": n, "role": roles.get(n, "norm"), "part": p} for n, p in slots.items()]}


def model_spec(vocab, hidden, position, layers, run_order, final_norm, max_positions, tied=True):
    return {"architecture": "toy", "embedding": {"vocab_size": vocab, "size": hidden}, "position": position, "layers": layers,
            "run_order": [{"layer": l, "cache": c} for l, c in run_order], "final_norm": final_norm,
            "head": {"vocab_size": vocab, "size": hidden, "tied": tied}, "max_positions": max_positions}


def build(folder, spec, seed, dtype="float32", num_pages=64, checkpoint=None, **options):
    """Writes the model as a folder (its description is the config.json), loads it; returns (replayer, parameters)."""
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import load_parameters, write_random_model
    config = {"model_type": "liyab_spec", "spec": spec, "init_std": 0.3}
    if checkpoint:
        config["checkpoint"] = checkpoint
    write_random_model(str(folder), config, seed, dtype)
    params = {k: v.astype(np.float64) for k, v in load_parameters(str(folder), "float32").items()}
    return Replayer(str(folder), dtype, max_tokens=0, num_pages=num_pages, max_requests=4, **options), params


def plain_attention_part(h, p, prefix, n_head, n_kv_head, scale, window=0, kv_from=None):
    """qkv projection [out, in] layout of the engine's parameters, attention, output projection."""
    w, b = p[prefix + "qkv.weight"], p[prefix + "qkv.bias"]
    hd = w.shape[0] // (n_head + 2 * n_kv_head)
    qd, kvd = n_head * hd, n_kv_head * hd
    qkv = h @ w.T + b
    src = qkv if kv_from is None else kv_from @ w.T + b
    att = plain.causal_attention(qkv[:, :qd], src[:, qd:qd + kvd], src[:, qd + kvd:], n_head, n_kv_head, scale, window)
    return att @ p[prefix + "out.weight"].T + p[prefix + "out.bias"]


def plain_ff_part(h, p, prefix, act):
    u = h @ p[prefix + "up.weight"].T + p[prefix + "up.bias"]
    u = plain.gelu_erf(u) if act == "gelu_erf" else plain.gelu_tanh(u)
    return u @ p[prefix + "down.weight"].T + p[prefix + "down.bias"]


def close(got, want, tol=2e-5):
    return np.abs(got - want).max() < tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("n_head,n_kv_head,window", [(3, 3, 0), (6, 2, 0), (4, 1, 5)])
def test_each_part_alone(n_head, n_kv_head, window, tmp_path):
    """Every part's output as the engine computed it, against the plain function of that part applied to the engine's
    own input of that part (so a fault shows at the part that has it, not downstream)."""
    from liyab_b200.engine import StepEntry
    H, eps = 96, 1e-4
    norm = layernorm(H, eps)
    spec = model_spec(50, H, {"kind": "learned_absolute", "size": H, "max_positions": 96},
                      [layer("pre_norm", mixer_norm=norm, mixer=attention(H, n_head, n_kv_head, H // n_head, 0.2, window), ff_norm=norm,
                             feed_forward=dense(H, 80, "gelu_erf"))], [(0, 0)], norm, 96)
    engine, p = build(tmp_path, spec, seed=n_head)
    tokens = np.random.default_rng(0).integers(0, 50, size=21).tolist()
    seen = {}
    engine.set_tap(lambda name, rows: seen.setdefault(name, rows.astype(np.float64)))
    engine.cache.open("a")
    out = engine.step([StepEntry("a", tokens, list(range(21)))])
    engine.set_tap(None)
    assert list(seen) == ["embed", "mixer_norm", "attention", "mixer", "ff_norm", "feed_forward", "final_norm"]
    # position encoding + embedding
    want_x = plain.add_positions(plain.embed(tokens, p["embedding.weight"]), p["position.weight"])
    assert np.abs(seen["embed"] - want_x).max() < 1e-6
    # norm, on the engine's own stream
    assert close(seen["mixer_norm"], plain.layernorm(seen["embed"], p["layers.0.mixer_norm.weight"], p["layers.0.mixer_norm.bias"], eps), 1e-5)
    # mixer: adds to the residual stream
    assert close(seen["mixer"], seen["embed"] + plain_attention_part(seen["mixer_norm"], p, "layers.0.mixer.", n_head, n_kv_head, 0.2, window))
    assert close(seen["ff_norm"], plain.layernorm(seen["mixer"], p["layers.0.ff_norm.weight"], p["layers.0.ff_norm.bias"], eps), 1e-5)
    # feed-forward
    assert close(seen["feed_forward"], seen["mixer"] + plain_ff_part(seen["ff_norm"], p, "layers.0.feed_forward.", "gelu_erf"))
    # the arrangement of all four, the final norm and the head: the whole chain from the tokens
    a = want_x + plain_attention_part(plain.layernorm(want_x, p["layers.0.mixer_norm.weight"], p["layers.0.mixer_norm.bias"], eps), p,
                                      "layers.0.mixer.", n_head, n_kv_head, 0.2, window)
    x = a + plain_ff_part(plain.layernorm(a, p["layers.0.ff_norm.weight"], p["layers.0.ff_norm.bias"], eps), p, "layers.0.feed_forward.", "gelu_erf")
    assert close(seen["feed_forward"], x)
    y = plain.layernorm(x, p["final_norm.weight"], p["final_norm.bias"], eps)
    assert close(seen["final_norm"], y) and close(out.logits, y @ p["embedding.weight"].T)
    # a step after the tap was removed runs as before
    assert engine.step([StepEntry("a", [1], [0])]).logits.shape == (1, 50)


# ---------------------------------------------------------------------------------------------------------
# A toy mixer with state of its own.  out_t = W . mean(h_0 .. h_t): the state is the running sum and count.

def toy_spec(host_loop=False):
    H = 32
    norm = layernorm(H)
    attn = layer("pre_norm", mixer_norm=norm, mixer=attention(H, 2, 1, 16, 0.25), ff_norm=norm, feed_forward=dense(H, 48, "gelu_tanh"))
    toy = layer("pre_norm", mixer_norm=norm, mixer={"kind": "toy_running_mean", "hidden": H, "host_loop": host_loop}, ff_norm=norm,
                feed_forward=dense(H, 40, "gelu_erf"))
    # Layer 0 runs twice; its second run reads the keys and values its first run wrote.
    return model_spec(40, H, {"kind": "learned_absolute", "size": H, "max_positions": 80}, [attn, toy], [(0, 0), (1, 1), (0, 0)], norm, 80)


def plain_toy_logits(p, tokens):
    x = plain.add_positions(plain.embed(tokens, p["embedding.weight"]), p["position.weight"])

    def ln(v, name):
        return plain.layernorm(v, p[name + ".weight"], p[name + ".bias"], 1e-5)

    h0 = ln(x, "layers.0.mixer_norm")                                    # first run of layer 0
    x = x + plain_attention_part(h0, p, "layers.0.mixer.", 2, 1, 0.25)
    x = x + plain_ff_part(ln(x, "layers.0.ff_norm"), p, "layers.0.feed_forward.", "gelu_tanh")
    h1 = ln(x, "layers.1.mixer_norm")                                    # the toy layer
    means = np.cumsum(h1, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
    x = x + means @ p["layers.1.mixer.w"].T
    x = x + plain_ff_part(ln(x, "layers.1.ff_norm"), p, "layers.1.feed_forward.", "gelu_erf")
    h2 = ln(x, "layers.0.mixer_norm")                                    # layer 0 again, on the first run's cache
    x = x + plain_attention_part(h2, p, "layers.0.mixer.", 2, 1, 0.25, kv_from=h0)
    x = x + plain_ff_part(ln(x, "layers.0.ff_norm"), p, "layers.0.feed_forward.", "gelu_tanh")
    return ln(x, "final_norm") @ p["embedding.weight"].T


@pytest.mark.parametrize("host_loop", [False, True])
def test_toy_mixer_with_state_is_registered_built_and_stepped(toy_plugin, tmp_path, host_loop):
    engine, p = build(tmp_path, toy_spec(host_loop), seed=5, num_pages=24, cuda_graphs=True, max_step_tokens=96)
    info = engine.info
    assert info["kv_units"] == [0] and info["state_units"] == [1] and info["capturable"] == (not host_loop)
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0]["units"] == [0]
    rng = np.random.default_rng(1)
    reqs = {f"t{i}": rng.integers(0, 40, size=n).tolist() for i, n in enumerate((37, 5, 80, 22, 9))}
    want = {r: plain_toy_logits(p, toks) for r, toks in reqs.items()}
    for steps in (tt.whole(reqs), tt.changing_portions(reqs), tt.tail_one_by_one(reqs, 20), tt.mixed(reqs, max_live=3, seed=2)):
        got = tt.collect(engine, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        for (r, pos), row in got.items():
            assert np.abs(row - want[r][pos]).max() < 5e-5 * max(1.0, np.abs(want[r]).max()), (r, pos)
    assert all(v == 0 for v in engine.cache.pages_in_use().values()) and engine.cache.state_slots_free() == 4
    # A mixer that keeps its state on the device only may be replayed from a captured graph (its state advances once
    # per step, in the replay); one that reads the host's copy of the layout is never captured.
    assert (engine.counters()["graph_steps"] > 0) == (not host_loop)


def test_windowed_layers_get_pages_of_their_own_and_give_them_back(tmp_path):
    """Two attention layers, one with a window: two cache groups; the windowed one frees pages as it goes."""
    H = 32
    norm, ff = layernorm(H), dense(H, 64, "gelu_tanh")
    full = layer("pre_norm", mixer_norm=norm, mixer=attention(H, 2, 2, 16, 0.25), ff_norm=norm, feed_forward=ff)
    win = layer("pre_norm", mixer_norm=norm, mixer=attention(H, 2, 2, 16, 0.25, window=20), ff_norm=norm, feed_forward=ff)
    spec = model_spec(40, H, {"kind": "learned_absolute", "size": H, "max_positions": 200}, [full, win], [(0, 0), (1, 1)], norm, 200)
    engine, p = build(tmp_path, spec, seed=9, num_pages=14)
    assert len(engine.cache.groups) == 2
    tokens = np.random.default_rng(3).integers(0, 40, size=200).tolist()
    x = plain.add_positions(plain.embed(tokens, p["embedding.weight"]), p["position.weight"])

    def ln(v, name):
        return plain.layernorm(v, p[name + ".weight"], p[name + ".bias"], 1e-5)

    for i, w in ((0, 0), (1, 20)):
        x = x + plain_attention_part(ln(x, f"layers.{i}.mixer_norm"), p, f"layers.{i}.mixer.", 2, 2, 0.25, window=w)
        x = x + plain_ff_part(ln(x, f"layers.{i}.ff_norm"), p, f"layers.{i}.feed_forward.", "gelu_tanh")
    want = ln(x, "final_norm") @ p["embedding.weight"].T
    steps = tt.changing_portions({"w": tokens}, sizes=(16, 3, 2, 30, 1, 1, 9))
    steps[-1] = (steps[-1][0], [])                       # keep the request open to look at what it still holds
    got = tt.collect(engine, steps)
    for (r, pos), row in got.items():
        assert np.abs(row - want[pos]).max() < 5e-5 * max(1.0, np.abs(want).max()), pos
    # 200 positions need 13 pages of 16; the windowed group holds what a window of 20 can still see
    gw = engine.cache.group_of_unit[1]
    assert engine.cache.groups[gw]["window"] == 20 and engine.cache.groups[gw]["num_pages"] == 14
    assert engine.cache.pages_in_use() == {engine.cache.group_of_unit[0]: 13, gw: 2}


def toy_parts_spec():
    H, V = 40, 33
    ln = layernorm(H)
    rms = {"kind": "toy_rms", "hidden": H, "eps": 1e-3}
    attn = attention(H, 5, 5, 8, 0.3)
    routed = {"kind": "toy_routed", "hidden": H, "experts": 3, "inner": 24, "top": 2}
    first = layer("pre_norm", mixer_norm=rms, mixer=attn, ff_norm=ln, feed_forward=routed)
    second = layer("toy_side_by_side", norm=rms, mixer=attn, feed_forward=dense(H, 56, "gelu_tanh"))
    third = layer("toy_third_norm", mixer_norm=ln, mixer=attn, ff_norm=rms, feed_forward=dense(H, 48, "gelu_erf"), out_norm=rms)
    return model_spec(V, H, {"kind": "toy_sinusoid", "hidden": H, "base": 50.0}, [first, second, third], [(0, 0), (1, 1), (2, 2)], rms, 128, tied=False)


def plain_toy_parts_logits(p, tokens):
    H = 40
    x = plain.embed(tokens, p["embedding.weight"])
    freq = 50.0 ** (-np.arange(0, H, 2) / H)
    angle = np.arange(len(tokens))[:, None] * freq
    x[:, 0::2] += np.sin(angle)
    x[:, 1::2] += np.cos(angle)

    def rms(v, name):
        return v / np.sqrt((v * v).mean(-1, keepdims=True) + 1e-3) * p[name + ".weight"]

    def ln(v, name):
        return plain.layernorm(v, p[name + ".weight"], p[name + ".bias"], 1e-5)

    x = x + plain_attention_part(rms(x, "layers.0.mixer_norm"), p, "layers.0.mixer.", 5, 5, 0.3)
    h = ln(x, "layers.0.ff_norm")
    logits = h @ p["layers.0.feed_forward.router"].T
    gate = np.exp(logits - logits.max(-1, keepdims=True))
    gate /= gate.sum(-1, keepdims=True)
    up = p["layers.0.feed_forward.up"].reshape(3, 24, H)
    down = p["layers.0.feed_forward.down"].reshape(3, H, 24)
    y = np.zeros_like(x)
    for t in range(len(tokens)):
        best = np.argsort(-gate[t], kind="stable")[:2]
        for e in best:
            y[t] += gate[t, e] / gate[t, best].sum() * (np.maximum(h[t] @ up[e].T, 0.0) @ down[e].T)
    x = x + y
    h = rms(x, "layers.1.norm")
    x = x + plain_attention_part(h, p, "layers.1.mixer.", 5, 5, 0.3) + plain_ff_part(h, p, "layers.1.feed_forward.", "gelu_tanh")
    x = x + plain_attention_part(ln(x, "layers.2.mixer_norm"), p, "layers.2.mixer.", 5, 5, 0.3)
    x = x + plain_ff_part(rms(x, "layers.2.ff_norm"), p, "layers.2.feed_forward.", "gelu_erf")
    x = rms(x, "layers.2.out_norm")
    return rms(x, "final_norm") @ p["head.weight"].T


def test_toy_feed_forward_with_routing_position_norm_and_arrangements(toy_plugin, tmp_path):
    """Parts of every other role, defined outside the framework, are registered, built beside the framework's own
    (attention over pages, the dense feed-forward, LayerNorm) and stepped in every cutting; one block has three slots,
    one has five (a third norm); one projection is joined from three tensors of the file."""
    from liyab_b200.config import describe_config
    spec = toy_parts_spec()
    ck = describe_config({"model_type": "liyab_spec", "spec": spec, "init_std": 0.3})["checkpoint"]
    qkv = "layers.2.mixer.qkv.weight"
    ck[qkv] = {"sources": [{"name": f"blk2.{n}", "shape": [40, 40]} for n in "qkv"], "transform": "transpose", "concat_axis": 0,
               "kind": "matrix", "init": [0.0, 0.3]}
    engine, p = build(tmp_path, spec, seed=9, num_pages=24, checkpoint=ck)
    from liyab_b200.weights import read_tensor
    stored = [read_tensor(str(tmp_path / "model.safetensors"), f"blk2.{n}").astype(np.float64) for n in "qkv"]
    assert np.array_equal(p[qkv], np.concatenate([s.T for s in stored], axis=0))
    assert engine.info["kv_units"] == [0, 1, 2] and not engine.info["state_units"]
    rng = np.random.default_rng(4)
    reqs = {f"t{i}": rng.integers(0, 33, size=n).tolist() for i, n in enumerate((41, 6, 90, 17))}
    want = {r: plain_toy_parts_logits(p, toks) for r, toks in reqs.items()}
    for steps in (tt.whole(reqs), tt.changing_portions(reqs), tt.mixed(reqs, max_live=3, seed=3)):
        got = tt.collect(engine, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        for (r, pos), row in got.items():
            assert np.abs(row - want[r][pos]).max() < 5e-5 * max(1.0, np.abs(want[r]).max()), (r, pos)
    assert all(v == 0 for v in engine.cache.pages_in_use().values())


def test_head_with_bias_scale_and_soft_cap(tmp_path):
    """An untied head with a bias, a factor on the logits and a soft cap: the slots exist and are applied."""
    H, V = 32, 37
    norm = layernorm(H)
    spec = model_spec(V, H, {"kind": "none"}, [layer("pre_norm", mixer_norm=norm, mixer=attention(H, 2, 2, 16, 0.25), ff_norm=norm,
                                                      feed_forward=dense(H, 48, "gelu_tanh"))], [(0, 0)], norm, 64, tied=False)
    spec["head"].update(bias=True, logit_scale=0.5, soft_cap=3.0)
    engine, p = build(tmp_path, spec, seed=2)
    assert "head.bias" in p and p["head.bias"].shape == (V,)
    tokens = np.random.default_rng(5).integers(0, V, size=19).tolist()
    x = plain.embed(tokens, p["embedding.weight"])

    def ln(v, name):
        return plain.layernorm(v, p[name + ".weight"], p[name + ".bias"], 1e-5)

    x = x + plain_attention_part(ln(x, "layers.0.mixer_norm"), p, "layers.0.mixer.", 2, 2, 0.25)
    x = x + plain_ff_part(ln(x, "layers.0.ff_norm"), p, "layers.0.feed_forward.", "gelu_tanh")
    raw = ln(x, "final_norm") @ p["head.weight"].T + p["head.bias"]
    want = 3.0 * np.tanh(raw * 0.5 / 3.0)
    assert np.abs(raw * 0.5).max() > 3.0, "the cap must bite for the test to mean something"
    got = tt.collect(engine, tt.changing_portions({"h": tokens}, sizes=(7, 1, 11)))
    for (r, pos), row in got.items():
        assert np.abs(row - want[pos]).max() < 5e-5, pos


@pytest.mark.parametrize("host_loop", [False, True])
def test_an_architecture_from_outside_runs_through_the_engine_with_graphs_on(toy_plugin, tmp_path, host_loop):
    """`toy_stack` has config.json keys of its own and a layer with state; generation through the public entry point
    (scheduler, captured graphs, pipelined loop) gives the plain implementation's greedy tokens.  Where the state
    mixer reads the host's copy of the layout the engine must not capture a step; it still generates correctly."""
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    from liyab_b200.weights import load_parameters, write_random_model
    raw = dict(model_type="toy_stack", width=32, depth=3, vocab=48, positions=96, host_loop=host_loop)
    folder = write_random_model(str(tmp_path / "toy"), raw, seed=11, dtype="float32")
    p = {k: v.astype(np.float64) for k, v in load_parameters(folder, "float32").items()}

    def logits(tokens):
        x = plain.add_positions(plain.embed(tokens, p["embedding.weight"]), p["position.weight"])
        for i in range(3):
            h = plain.layernorm(x, p[f"layers.{i}.mixer_norm.weight"], p[f"layers.{i}.mixer_norm.bias"], 1e-5)
            if i % 2 == 0:
                x = x + plain_attention_part(h, p, f"layers.{i}.mixer.", 2, 1, 0.25)
            else:
                x = x + (np.cumsum(h, axis=0) / np.arange(1, len(tokens) + 1)[:, None]) @ p[f"layers.{i}.mixer.w"].T
            x = x + plain_ff_part(plain.layernorm(x, p[f"layers.{i}.ff_norm.weight"], p[f"layers.{i}.ff_norm.bias"], 1e-5), p,
                                  f"layers.{i}.feed_forward.", "gelu_tanh")
        return plain.layernorm(x, p["final_norm.weight"], p["final_norm.bias"], 1e-5) @ p["embedding.weight"].T

    def greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(np.argmax(logits(toks)[-1])))
        return toks[len(prompt):]

    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, 48, size=n).tolist() for n in (9, 3, 21)]
    engine = Engine(EngineConfig(model=folder, dtype="float32", max_requests=3, max_batched_tokens=16, num_pages=24, cuda_graphs=True))
    got = engine.generate_batch(prompts, SamplingParams(temperature=0.0, max_tokens=20))
    for prompt, r in zip(prompts, got):
        assert r.tokens == greedy(prompt, 20) and r.finish_reason == "length"
    st = engine.stats()
    assert (st["graph_steps"] > 0) == (not host_loop) and st["pages_in_use"] == 0
