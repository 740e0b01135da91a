"""The plain implementation itself: against logits that the reference's own C++ forward pass produced
(tests/golden/, made by make_golden.py), and against simple facts about its parts."""
import json
import os

import numpy as np
import pytest

import plain_gpt2 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["gpt2_ref_a", "gpt2_ref_b", "gpt2_ref_c"])
def test_plain_matches_the_reference_engine(name):
    """a and b: GPT-2 as the reference runs it.  c: `scale_attn_weights: false`, which the reference computes from
    its per-model factor on the scores (gpt2.attention.scale = 1)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = json.loads(bytes(z["config_json"]).decode())
    tensors = {k[len("tensor:"):]: z[k].astype(np.float64) for k in z.files if k.startswith("tensor:")}
    logits = plain.forward_logits(plain.PlainModel(cfg, tensors), z["tokens"].tolist())
    ref = z["logits"].astype(np.float64)
    # The reference keeps keys and values in 16-bit; 1e-4 of the logits' scale covers that rounding.
    assert np.abs(logits - ref).max() <= 1e-4 * np.abs(ref).max()
    assert (logits.argmax(axis=1) == ref.argmax(axis=1)).all()


def test_layernorm_and_gelu_facts():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    y = plain.layernorm(x, None, None, 0.0)
    assert np.allclose(y.mean(), 0) and np.allclose((y * y).mean(), 1)
    assert np.allclose(plain.gelu_erf(np.array([0.0, 1.0])), [0.0, 0.8413447460685429])
    assert np.allclose(plain.gelu_tanh(np.array([1.0])), [0.8411919906082768])


def test_causal_attention_sees_only_the_past_and_the_window():
    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((3, 6, 8))
    full = plain.causal_attention(q, k, v, 2, 2, 0.5)
    k2, v2 = k.copy(), v.copy()
    k2[4:], v2[4:] = 99.0, -99.0
    assert np.allclose(plain.causal_attention(q, k2, v2, 2, 2, 0.5)[:4], full[:4])     # the future does not matter
    win = plain.causal_attention(q, k, v, 2, 2, 0.5, window=2)
    assert np.allclose(win[:2], full[:2]) and not np.allclose(win[3], full[3])
    assert np.allclose(plain.causal_attention(q, k[:, :4], v[:, :4], 2, 1, 0.5)[:, 4:],
                       plain.causal_attention(q[:, 4:], k[:, :4], v[:, :4], 1, 1, 0.5))  # grouped heads share keys


def test_sampler_follows_the_reference_rules():
    logits = np.array([1.0, 3.0, 2.0, 3.0, -1.0], dtype=np.float32)
    assert plain.sampler_probabilities(logits, 0.0, 40, 0.95).tolist() == [0, 1, 0, 0, 0]      # first maximum
    p = plain.sampler_probabilities(logits, 1.0, 2, 1.0)
    assert (p > 0).tolist() == [False, True, False, True, False] and np.allclose(p[[1, 3]], 0.5)
    p = plain.sampler_probabilities(logits, 1.0, 0, 0.5)          # shortest prefix reaching 0.5
    assert (p > 0).sum() == 2
    assert plain.sampler_draw(np.array([0.25, 0.0, 0.75], dtype=np.float32), 0.2) == 0
    assert plain.sampler_draw(np.array([0.25, 0.0, 0.75], dtype=np.float32), 0.3) == 2
    u = [plain.uniform_draw(7, 1, i) for i in range(1000)]
    assert 0 <= min(u) and max(u) < 1 and abs(np.mean(u) - 0.5) < 0.05
