"""Each part alone against the plain functions, and the framework's generality: a toy mixer with
state of its own, defined here, is registered, built into a model beside attention layers (one layer
run twice, one run reading another run's cache) and stepped, without a change to the framework; and so are
a feed-forward with routing, a position encoding without a table, a norm and an arrangement of a block."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_gpt2 as plain

pytestmark = pytest.mark.gpu


def _np(t):
    return t.detach().double().cpu().numpy()


def build(spec, seed, dtype="float32", num_pages=64, page_size=16, max_requests=4):
    from liyab_b200.cache import CacheManager
    from liyab_b200.engine import Stepper
    from liyab_b200.models import DecoderModel, parameter_shapes
    from liyab_b200.parts import Runtime
    from liyab_b200.weights import COMPUTE_DTYPES, random_parameters
    dev = torch.device("cuda:0")
    params = random_parameters(parameter_shapes(spec), seed, dtype, dev, std=0.3)
    model = DecoderModel(spec, params, Runtime(dtype=COMPUTE_DTYPES[dtype], device=dev))
    cache = CacheManager(model.kv_needs(), model.state_needs(), page_size, num_pages, max_requests,
                         dtype=model.runtime.dtype, device=dev)
    return model, params, cache, Stepper(model, cache)


def context_for(stepper, cache, entries):
    """Opens requests, reserves their pages and lays the step out: what `Stepper.step` does before the model runs."""
    from liyab_b200.engine import StepEntry
    batch = [StepEntry(request=r, tokens=t, want=list(range(len(t)))) for r, t in entries]
    for e in batch:
        if not cache.is_open(e.request):
            cache.open(e.request)
    rows, q_len, tokens = stepper.validate(batch)
    cache.reserve_rows(rows, q_len)
    ctx, _ = stepper._layout(batch, rows, q_len, tokens)
    return ctx


def one_layer_spec(hidden=48, n_head=3, n_kv_head=3, inner=80, vocab=50, positions=96, act="gelu_erf", eps=1e-4,
                   scale=0.2, window=0):
    from liyab_b200.config import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec,
                                   NormSpec, PositionSpec, RunEntry)
    norm = NormSpec(kind="layernorm", size=hidden, eps=eps)
    layer = LayerSpec("pre_norm", norm,
                      AttentionSpec(kind="attention", hidden=hidden, n_head=n_head, n_kv_head=n_kv_head,
                                    head_dim=hidden // n_head, scale=scale, window=window),
                      norm, DenseFeedForwardSpec(kind="dense", hidden=hidden, inner=inner, activation=act))
    return ModelSpec("toy", EmbeddingSpec(vocab, hidden), PositionSpec(kind="learned_absolute", size=hidden, max_positions=positions),
                     (layer,), (RunEntry(0, 0),), norm, HeadSpec(vocab, hidden, tied=True), positions)


def plain_attention_part(h, p, prefix, n_head, n_kv_head, scale, window=0, kv_from=None):
    """qkv projection [out, in] layout of the engine's parameters, attention, output projection."""
    w, b = _np(p[prefix + "qkv.weight"]), _np(p[prefix + "qkv.bias"])
    qd = h.shape[1] // n_head * n_head
    hd = qd // n_head
    kvd = n_kv_head * hd
    qkv = h @ w.T + b
    src = qkv if kv_from is None else kv_from @ w.T + b
    att = plain.causal_attention(qkv[:, :qd], src[:, qd:qd + kvd], src[:, qd + kvd:], n_head, n_kv_head, scale, window)
    return att @ _np(p[prefix + "out.weight"]).T + _np(p[prefix + "out.bias"])


def plain_ff_part(h, p, prefix, act):
    u = h @ _np(p[prefix + "up.weight"]).T + _np(p[prefix + "up.bias"])
    u = plain.gelu_erf(u) if act == "gelu_erf" else plain.gelu_tanh(u)
    return u @ _np(p[prefix + "down.weight"]).T + _np(p[prefix + "down.bias"])


@pytest.mark.parametrize("n_head,n_kv_head,window", [(3, 3, 0), (6, 2, 0), (4, 1, 5)])
def test_each_part_alone(n_head, n_kv_head, window):
    spec = one_layer_spec(hidden=96, n_head=n_head, n_kv_head=n_kv_head, window=window)
    model, p, cache, stepper = build(spec, seed=n_head)
    tokens = np.random.default_rng(0).integers(0, 50, size=21).tolist()
    ctx = context_for(stepper, cache, [("a", tokens)])
    T = len(tokens)
    dev = model.runtime.device
    # position encoding + embedding
    x = torch.empty((T, 96), dtype=torch.float32, device=dev)
    model.position.embed(ctx, model.embedding, 1.0, x)
    want_x = plain.add_positions(plain.embed(tokens, _np(p["embedding.weight"])), _np(p["position.weight"]))
    assert np.abs(_np(x) - want_x).max() < 1e-6
    # norm
    parts = model.layers[0].parts
    h = torch.empty_like(x)
    parts.mixer_norm.forward(ctx, x, h, T)
    want_h = plain.layernorm(want_x, _np(p["layers.0.mixer_norm.weight"]), _np(p["layers.0.mixer_norm.bias"]), 1e-4)
    assert np.abs(_np(h) - want_h).max() < 1e-5
    # mixer: adds to the residual stream
    from liyab_b200.parts import CacheUnit
    x1 = x.clone()
    parts.mixer.forward(ctx, h, x1, CacheUnit(read=0, write=True))
    want_x1 = want_x + plain_attention_part(want_h, p, "layers.0.mixer.", n_head, n_kv_head, 0.2, window)
    assert np.abs(_np(x1) - want_x1).max() < 2e-5 * max(1.0, np.abs(want_x1).max())
    # feed-forward
    x2 = x1.clone()
    parts.feed_forward.forward(ctx, h, x2)
    want_x2 = want_x1 + plain_ff_part(want_h, p, "layers.0.feed_forward.", "gelu_erf")
    assert np.abs(_np(x2) - want_x2).max() < 2e-5 * max(1.0, np.abs(want_x2).max())
    # the arrangement of all four
    x3 = x.clone()
    model.layers[0].forward(ctx, x3, CacheUnit(read=0, write=True))
    a = want_x + plain_attention_part(want_h, p, "layers.0.mixer.", n_head, n_kv_head, 0.2, window)
    h2 = plain.layernorm(a, _np(p["layers.0.ff_norm.weight"]), _np(p["layers.0.ff_norm.bias"]), 1e-4)
    want_x3 = a + plain_ff_part(h2, p, "layers.0.feed_forward.", "gelu_erf")
    assert np.abs(_np(x3) - want_x3).max() < 2e-5 * max(1.0, np.abs(want_x3).max())


# ---------------------------------------------------------------------------------------------------------
# A toy mixer with state of its own.  out_t = W . mean(h_0 .. h_t): the state is the running sum and count.

def register_toy_mixer():
    from liyab_b200.cache import StateNeed
    from liyab_b200.parts import MIXERS

    @MIXERS.register("toy_running_mean")
    class RunningMeanMixer:
        def __init__(self, spec, params, runtime):
            self.spec, self.w = spec, params["w"]

        @classmethod
        def parameters(cls, spec):
            return {"w": ((spec.hidden, spec.hidden), "matrix")}

        def kv_need(self):
            return None

        def state_need(self):
            return StateNeed(shape=(self.spec.hidden + 1,), dtype=torch.float32)

        def forward(self, ctx, h, x, unit):
            state = ctx.state(unit.read)
            slots = ctx.state_slots.tolist()
            for i in range(ctx.n_seq):
                lo, hi = ctx.host_q_start[i], ctx.host_q_start[i + 1]
                s = state[slots[i]]
                sums = s[:-1] + torch.cumsum(h[lo:hi].float(), dim=0)
                counts = s[-1] + torch.arange(1, hi - lo + 1, device=h.device, dtype=torch.float32)
                x[lo:hi] += (sums / counts[:, None]) @ self.w.float().t()
                if unit.write:
                    s[:-1] = sums[-1]
                    s[-1] = counts[-1]

    return RunningMeanMixer


def toy_spec():
    from liyab_b200.config import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, GenericSpec, HeadSpec, LayerSpec,
                                   ModelSpec, NormSpec, PositionSpec, RunEntry)
    H = 32
    norm = NormSpec(kind="layernorm", size=H, eps=1e-5)
    attn = LayerSpec("pre_norm", norm, AttentionSpec(kind="attention", hidden=H, n_head=2, n_kv_head=1, head_dim=16, scale=0.25),
                     norm, DenseFeedForwardSpec(kind="dense", hidden=H, inner=48, activation="gelu_tanh"))
    toy = LayerSpec("pre_norm", norm, GenericSpec(kind="toy_running_mean", hidden=H),
                    norm, DenseFeedForwardSpec(kind="dense", hidden=H, inner=40, activation="gelu_erf"))
    # Layer 0 runs twice; its second run reads the keys and values its first run wrote.
    order = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 0))
    return ModelSpec("toy", EmbeddingSpec(40, H), PositionSpec(kind="learned_absolute", size=H, max_positions=80),
                     (attn, toy), order, norm, HeadSpec(40, H, tied=True), 80)


def plain_toy_logits(p, tokens):
    x = plain.add_positions(plain.embed(tokens, _np(p["embedding.weight"])), _np(p["position.weight"]))

    def ln(v, name):
        return plain.layernorm(v, _np(p[name + ".weight"]), _np(p[name + ".bias"]), 1e-5)

    h0 = ln(x, "layers.0.mixer_norm")                                    # first run of layer 0
    x = x + plain_attention_part(h0, p, "layers.0.mixer.", 2, 1, 0.25)
    x = x + plain_ff_part(ln(x, "layers.0.ff_norm"), p, "layers.0.feed_forward.", "gelu_tanh")
    h1 = ln(x, "layers.1.mixer_norm")                                    # the toy layer
    means = np.cumsum(h1, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
    x = x + means @ _np(p["layers.1.mixer.w"]).T
    x = x + plain_ff_part(ln(x, "layers.1.ff_norm"), p, "layers.1.feed_forward.", "gelu_erf")
    h2 = ln(x, "layers.0.mixer_norm")                                    # layer 0 again, on the first run's cache
    x = x + plain_attention_part(h2, p, "layers.0.mixer.", 2, 1, 0.25, kv_from=h0)
    x = x + plain_ff_part(ln(x, "layers.0.ff_norm"), p, "layers.0.feed_forward.", "gelu_tanh")
    return ln(x, "final_norm") @ _np(p["embedding.weight"]).T


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    import trace_tools as tt
    register_toy_mixer()
    model, p, cache, stepper = build(toy_spec(), seed=5, num_pages=24)
    assert sorted(model.kv_needs()) == [0] and sorted(model.state_needs()) == [1]
    assert len(cache.groups) == 1 and cache.groups[0].units == [0]
    rng = np.random.default_rng(1)
    reqs = {f"t{i}": rng.integers(0, 40, size=n).tolist() for i, n in enumerate((37, 5, 80, 22, 9))}
    want = {r: plain_toy_logits(p, toks) for r, toks in reqs.items()}
    for steps in (tt.whole(reqs), tt.changing_portions(reqs), tt.mixed(reqs, max_live=3, seed=2)):
        got = tt.collect(stepper, cache, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        for (r, pos), row in got.items():
            assert np.abs(row - want[r][pos]).max() < 5e-5 * max(1.0, np.abs(want[r]).max()), (r, pos)
    assert all(v == 0 for v in cache.pages_in_use().values()) and cache.states.pool.free_count == 4


def test_windowed_layers_get_pages_of_their_own_and_give_them_back():
    """Two attention layers, one with a window: two cache groups; the windowed one frees pages as it goes."""
    import trace_tools as tt
    from liyab_b200.config import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec,
                                   NormSpec, PositionSpec, RunEntry)
    H = 32
    norm = NormSpec(kind="layernorm", size=H, eps=1e-5)
    ff = DenseFeedForwardSpec(kind="dense", hidden=H, inner=64, activation="gelu_tanh")
    full = LayerSpec("pre_norm", norm, AttentionSpec(kind="attention", hidden=H, n_head=2, n_kv_head=2, head_dim=16, scale=0.25), norm, ff)
    win = LayerSpec("pre_norm", norm, AttentionSpec(kind="attention", hidden=H, n_head=2, n_kv_head=2, head_dim=16, scale=0.25, window=20), norm, ff)
    spec = ModelSpec("toy", EmbeddingSpec(40, H), PositionSpec(kind="learned_absolute", size=H, max_positions=200),
                     (full, win), (RunEntry(0, 0), RunEntry(1, 1)), norm, HeadSpec(40, H, tied=True), 200)
    model, p, cache, stepper = build(spec, seed=9, num_pages=14)
    assert len(cache.groups) == 2
    tokens = np.random.default_rng(3).integers(0, 40, size=200).tolist()
    x = plain.add_positions(plain.embed(tokens, _np(p["embedding.weight"])), _np(p["position.weight"]))

    def ln(v, name):
        return plain.layernorm(v, _np(p[name + ".weight"]), _np(p[name + ".bias"]), 1e-5)

    for i, w in ((0, 0), (1, 20)):
        x = x + plain_attention_part(ln(x, f"layers.{i}.mixer_norm"), p, f"layers.{i}.mixer.", 2, 2, 0.25, window=w)
        x = x + plain_ff_part(ln(x, f"layers.{i}.ff_norm"), p, f"layers.{i}.feed_forward.", "gelu_tanh")
    want = ln(x, "final_norm") @ _np(p["embedding.weight"]).T
    got = tt.collect(stepper, cache, tt.changing_portions({"w": tokens}, sizes=(16, 3, 2, 30, 1, 1, 9)))
    for (r, pos), row in got.items():
        assert np.abs(row - want[pos]).max() < 5e-5 * max(1.0, np.abs(want).max()), pos
    # 200 positions need 13 pages of 16; the windowed group never held more than a window and a portion's worth
    gw = cache.groups[cache.group_of_unit[1]]
    assert gw.need.window == 20 and gw.pool.num_pages == 14


def register_toy_parts():
    """A feed-forward with routing, a position encoding without a table, a norm without a mean and a
    block that runs its two parts side by side: each defined here, in plain torch, on the parts' interfaces."""
    from liyab_b200 import ops
    from liyab_b200.parts import ARRANGEMENTS, FEED_FORWARDS, NORMS, POSITIONS

    @FEED_FORWARDS.register("toy_routed")
    class RoutedFeedForward:
        """Every token goes to its best `top` experts of `experts` small ungated ones; router in 32-bit."""
        def __init__(self, spec, params, runtime):
            self.spec, self.p = spec, params

        @classmethod
        def parameters(cls, spec):
            E, I, H = spec.options["experts"], spec.options["inner"], spec.hidden
            return {"router": ((E, H), "matrix"), "up": ((E * I, H), "matrix"), "down": ((E * H, I), "matrix")}

        def forward(self, ctx, h, x):
            E, I, H, top = self.spec.options["experts"], self.spec.options["inner"], self.spec.hidden, self.spec.options["top"]
            hf = h[:ctx.n_tokens].float()
            gate = torch.softmax(hf @ self.p["router"].float().t(), dim=-1)
            weight, chosen = torch.topk(gate, top, dim=-1)
            weight = weight / weight.sum(-1, keepdim=True)
            up, down = self.p["up"].float().view(E, I, H), self.p["down"].float().view(E, H, I)
            for e in range(E):
                share = (weight * (chosen == e)).sum(-1)
                rows = torch.nonzero(share > 0).flatten()
                if rows.numel():
                    y = torch.relu(hf[rows] @ up[e].t()) @ down[e].t()
                    x[rows] += share[rows, None] * y

    @POSITIONS.register("toy_sinusoid")
    class SinusoidPosition:
        """sin / cos of the position at geometric frequencies, added to the embedding; nothing learned."""
        def __init__(self, spec, params, runtime):
            self.spec = spec

        @classmethod
        def parameters(cls, spec):
            return {}

        @property
        def max_positions(self):
            return 1 << 20

        def embed(self, ctx, table, scale, x):
            ops.embed_positions(ctx.tokens, ctx.positions, table, None, x, scale)
            H = self.spec.hidden
            freq = self.spec.options["base"] ** (-torch.arange(0, H, 2, device=x.device, dtype=torch.float32) / H)
            angle = ctx.positions[:ctx.n_tokens].float()[:, None] * freq
            x[:ctx.n_tokens, 0::2] += torch.sin(angle)
            x[:ctx.n_tokens, 1::2] += torch.cos(angle)
            return x

    @NORMS.register("toy_rms")
    class RmsNorm:
        def __init__(self, spec, params, runtime):
            self.spec, self.weight = spec, params["weight"]

        @classmethod
        def parameters(cls, spec):
            return {"weight": ((spec.hidden,), "vector")}

        def forward(self, ctx, x, out, n_rows, rows=None):
            v = x[:n_rows] if rows is None else x[rows[:n_rows].long()]
            v = v.float()
            y = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + self.spec.options["eps"]) * self.weight.float()
            out[:n_rows] = y.to(out.dtype)
            return out

    @ARRANGEMENTS.register("toy_side_by_side")
    class SideBySideBlock:
        """x += mixer(norm(x)) + feed_forward(norm(x)): both parts read the same normalised input."""
        def __init__(self, spec, parts, runtime):
            self.spec, self.parts, self.runtime = spec, parts, runtime

        def forward(self, ctx, x, unit):
            h = ctx.workspace.get("block.normed", ctx.n_tokens, x.shape[1], self.runtime.dtype)
            self.parts.mixer_norm.forward(ctx, x, h, ctx.n_tokens)
            self.parts.mixer.forward(ctx, h, x, unit)
            self.parts.feed_forward.forward(ctx, h, x)


def toy_parts_spec():
    from liyab_b200.config import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, GenericSpec, HeadSpec, LayerSpec,
                                   ModelSpec, NormSpec, RunEntry)
    H, V = 40, 33
    ln = NormSpec(kind="layernorm", size=H, eps=1e-5)
    rms = GenericSpec(kind="toy_rms", hidden=H, options={"eps": 1e-3})
    attn = AttentionSpec(kind="attention", hidden=H, n_head=5, n_kv_head=5, head_dim=8, scale=0.3)
    routed = GenericSpec(kind="toy_routed", hidden=H, options={"experts": 3, "inner": 24, "top": 2})
    first = LayerSpec("pre_norm", rms, attn, ln, routed)
    second = LayerSpec("toy_side_by_side", rms, attn, rms,
                       DenseFeedForwardSpec(kind="dense", hidden=H, inner=56, activation="gelu_tanh"))
    return ModelSpec("toy", EmbeddingSpec(V, H), GenericSpec(kind="toy_sinusoid", hidden=H, options={"base": 50.0}),
                     (first, second), (RunEntry(0, 0), RunEntry(1, 1)), rms, HeadSpec(V, H, tied=False), 128)


def plain_toy_parts_logits(p, tokens):
    H = 40
    x = plain.embed(tokens, _np(p["embedding.weight"]))
    freq = 50.0 ** (-np.arange(0, H, 2) / H)
    angle = np.arange(len(tokens))[:, None] * freq
    x[:, 0::2] += np.sin(angle)
    x[:, 1::2] += np.cos(angle)

    def rms(v, name):
        return v / np.sqrt((v * v).mean(-1, keepdims=True) + 1e-3) * _np(p[name + ".weight"])

    x = x + plain_attention_part(rms(x, "layers.0.mixer_norm"), p, "layers.0.mixer.", 5, 5, 0.3)
    h = plain.layernorm(x, _np(p["layers.0.ff_norm.weight"]), _np(p["layers.0.ff_norm.bias"]), 1e-5)
    logits = h @ _np(p["layers.0.feed_forward.router"]).T
    gate = np.exp(logits - logits.max(-1, keepdims=True))
    gate /= gate.sum(-1, keepdims=True)
    up = _np(p["layers.0.feed_forward.up"]).reshape(3, 24, H)
    down = _np(p["layers.0.feed_forward.down"]).reshape(3, H, 24)
    y = np.zeros_like(x)
    for t in range(len(tokens)):
        best = np.argsort(-gate[t], kind="stable")[:2]
        for e in best:
            y[t] += gate[t, e] / gate[t, best].sum() * (np.maximum(h[t] @ up[e].T, 0.0) @ down[e].T)
    x = x + y
    h = rms(x, "layers.1.mixer_norm")
    x = x + plain_attention_part(h, p, "layers.1.mixer.", 5, 5, 0.3) + plain_ff_part(h, p, "layers.1.feed_forward.", "gelu_tanh")
    return rms(x, "final_norm") @ _np(p["head.weight"]).T


def test_toy_feed_forward_with_routing_position_norm_and_arrangement():
    """Parts of every other role, defined in this file, are registered, built beside the framework's own
    (attention over pages, the dense feed-forward, LayerNorm) and stepped in every cutting."""
    import trace_tools as tt
    register_toy_parts()
    model, p, cache, stepper = build(toy_parts_spec(), seed=9, num_pages=24)
    assert sorted(model.kv_needs()) == [0, 1] and not model.state_needs()
    rng = np.random.default_rng(4)
    reqs = {f"t{i}": rng.integers(0, 33, size=n).tolist() for i, n in enumerate((41, 6, 90, 17))}
    want = {r: plain_toy_parts_logits(p, toks) for r, toks in reqs.items()}
    for steps in (tt.whole(reqs), tt.changing_portions(reqs), tt.mixed(reqs, max_live=3, seed=3)):
        got = tt.collect(stepper, cache, steps)
        assert len(got) == sum(len(t) for t in reqs.values())
        for (r, pos), row in got.items():
            assert np.abs(row - want[r][pos]).max() < 5e-5 * max(1.0, np.abs(want[r]).max()), (r, pos)
    assert all(v == 0 for v in cache.pages_in_use().values())
