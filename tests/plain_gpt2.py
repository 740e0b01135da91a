"""A plain, slow GPT-2 in NumPy float64: the oracle of the tests.

Whole sequences, no cache, one function for each part, written from the
formulas of the reference (andrei-borcea/liyab); every function cites the file
and lines it restates.  Nothing here imports the engine: the model folder is
read with the `safetensors` package and plain `json`, tensors keep the file's
own names and layouts (projection matrices [in, out]).

Anchoring: `tests/golden/` holds logits that the reference's own C++ forward
pass produced for a tiny random GPT-2, and a test compares this file with them.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np


# --------------------------------------------------------------------------- model folder

@dataclass
class PlainModel:
    config: Dict
    tensors: Dict[str, np.ndarray]      # float64, names as in the file, without a "transformer." prefix

    @property
    def n_layer(self) -> int:
        return int(self.config["n_layer"])

    @property
    def n_head(self) -> int:
        return int(self.config["n_head"])

    @property
    def n_embd(self) -> int:
        return int(self.config["n_embd"])


def load_plain_model(model_dir: str) -> PlainModel:
    import torch
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        config = json.load(f)
    raw = load_file(os.path.join(model_dir, "model.safetensors"))
    tensors = {}
    for name, t in raw.items():
        if name.startswith("transformer."):
            name = name[len("transformer."):]
        tensors[name] = t.to(torch.float64).numpy()
    return PlainModel(config=config, tensors=tensors)


# --------------------------------------------------------------------------- parts

def embed(tokens: Sequence[int], wte: np.ndarray) -> np.ndarray:
    """x_t = wte[token_t]; no embedding scale for this architecture
    (src/core/transformer.cpp:5495-5512)."""
    return wte[np.asarray(tokens, dtype=np.int64)].copy()


def add_positions(x: np.ndarray, wpe: np.ndarray, first_position: int = 0) -> np.ndarray:
    """x_t += wpe[pos_t], pos_t = n_past + index in the segment; a position at or
    past the table's rows is ContextFull (src/core/transformer.cpp:2791-2808)."""
    n = x.shape[0]
    if first_position + n > wpe.shape[0]:
        raise ValueError("context full: position beyond the position table")
    return x + wpe[first_position:first_position + n]


def layernorm(x: np.ndarray, w: Optional[np.ndarray], b: Optional[np.ndarray], eps: float) -> np.ndarray:
    """mean = sum(x)/n, var = sum((x-mean)^2)/n (population), y = (x-mean) /
    sqrt(var+eps) * w + b (src/core/transformer.cpp:74-106)."""
    mean = x.mean(axis=-1, keepdims=True)
    dev = x - mean
    var = (dev * dev).mean(axis=-1, keepdims=True)
    y = dev * (1.0 / np.sqrt(var + eps))
    if w is not None:
        y = y * w
    if b is not None:
        y = y + b
    return y


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
    (src/core/transformer.cpp:123-130)."""
    return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def gelu_erf(x: np.ndarray) -> np.ndarray:
    """0.5 x (1 + erf(x / sqrt 2)) (src/core/transformer.cpp:134-142)."""
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return 0.5 * x * (1.0 + erf(x * 0.70710678118654752440))


def linear_in_out(x: np.ndarray, w_in_out: np.ndarray, bias: Optional[np.ndarray]) -> np.ndarray:
    """y = x W + b for a matrix stored [in, out]: the reference's matmul is
    y[n][rows] = x[n][cols] . w^T over its [out][in] rows (include/liyab/backend.h:35-43)
    with the optional bias added to each output row before anything consumes it
    (src/core/transformer.cpp:111-118)."""
    y = x @ w_in_out
    if bias is not None:
        y = y + bias
    return y


def causal_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, n_head: int, n_kv_head: int, scale: float,
                     window: int = 0) -> np.ndarray:
    """Scores s_j = (q_h . k_j,h) * scale for the visible keys j in [0, pos]
    (or the `window` latest), softmax with the maximum subtracted, weighted sum
    of the values; query head h reads key/value head h // (n_head / n_kv_head)
    (src/core/transformer.cpp:2303-2313 scores, 2327-2341 softmax, 2344-2358
    values, 2367-2385 merge; causal range 497-510, 2235-2242)."""
    n, qd = q.shape
    hd = qd // n_head
    group = n_head // n_kv_head
    out = np.zeros((n, n_head * hd), dtype=np.float64)
    for h in range(n_head):
        g = h // group
        qh = q[:, h * hd:(h + 1) * hd]
        kh = k[:, g * hd:(g + 1) * hd]
        vh = v[:, g * hd:(g + 1) * hd]
        for t in range(n):
            first = 0 if window <= 0 else max(0, t - window + 1)
            s = (kh[first:t + 1] @ qh[t]) * scale
            e = np.exp(s - s.max())
            out[t, h * hd:(h + 1) * hd] = (e[:, None] * vh[first:t + 1]).sum(axis=0) / e.sum()
    return out


def attention_mixer(x: np.ndarray, m: PlainModel, layer: int) -> np.ndarray:
    """Fused projection, split [q | k | v] with the bias split the same way, no
    rotation, attention, output projection + bias
    (src/core/transformer.cpp:2657-2673, 3083-3126, 3139-3140; bias split 1266-1273)."""
    t, d, H = m.tensors, m.n_embd, m.n_head
    qkv = linear_in_out(x, t[f"h.{layer}.attn.c_attn.weight"], t[f"h.{layer}.attn.c_attn.bias"])
    q, k, v = qkv[:, :d], qkv[:, d:2 * d], qkv[:, 2 * d:]
    att = causal_attention(q, k, v, H, H, attention_scale(m.config, layer))
    return linear_in_out(att, t[f"h.{layer}.attn.c_proj.weight"], t[f"h.{layer}.attn.c_proj.bias"])


def attention_scale(config: Dict, layer: int) -> float:
    """1/sqrt(head_dim) unless the file overrides it (src/compat/architecture.cpp:975-985).
    GPT-2's own options: `scale_attn_weights` false leaves scores unscaled and
    `scale_attn_by_inverse_layer_idx` divides by (layer + 1); the reference has
    no such rule, these two follow the meaning of GPT-2's configuration keys."""
    hd = int(config["n_embd"]) // int(config["n_head"])
    scale = 1.0 / math.sqrt(hd) if config.get("scale_attn_weights", True) else 1.0
    if config.get("scale_attn_by_inverse_layer_idx", False):
        scale /= layer + 1
    return scale


def dense_ffn(x: np.ndarray, m: PlainModel, layer: int) -> np.ndarray:
    """down(act(up x + b_up)) + b_down, ungated (src/core/transformer.cpp:4903-4913)."""
    t = m.tensors
    h = linear_in_out(x, t[f"h.{layer}.mlp.c_fc.weight"], t[f"h.{layer}.mlp.c_fc.bias"])
    act = m.config.get("activation_function", "gelu_new")
    h = gelu_erf(h) if act == "gelu" else gelu_tanh(h)
    return linear_in_out(h, t[f"h.{layer}.mlp.c_proj.weight"], t[f"h.{layer}.mlp.c_proj.bias"])


def block(x: np.ndarray, m: PlainModel, layer: int) -> np.ndarray:
    """norm -> mixer -> +residual -> norm -> feed-forward -> +residual
    (src/core/transformer.cpp:5574-5577, 5633-5637, 5647, 5663-5666, 5684-5685, 5692)."""
    t, eps = m.tensors, float(m.config.get("layer_norm_epsilon", 1e-5))
    x = x + attention_mixer(layernorm(x, t[f"h.{layer}.ln_1.weight"], t[f"h.{layer}.ln_1.bias"], eps), m, layer)
    x = x + dense_ffn(layernorm(x, t[f"h.{layer}.ln_2.weight"], t[f"h.{layer}.ln_2.bias"], eps), m, layer)
    return x


def final_logits(x: np.ndarray, m: PlainModel) -> np.ndarray:
    """Final norm, then the tied head: logits = y . wte^T, no bias, no scale
    (src/core/transformer.cpp:6564-6579, 2613-2620; tie 1100-1104)."""
    t, eps = m.tensors, float(m.config.get("layer_norm_epsilon", 1e-5))
    y = layernorm(x, t["ln_f.weight"], t["ln_f.bias"], eps)
    head = t["wte.weight"] if m.config.get("tie_word_embeddings", True) else t["lm_head.weight"]
    return y @ head.T


def hidden_states(m: PlainModel, tokens: Sequence[int]) -> np.ndarray:
    """The residual stream after the last block for a whole sequence
    (src/core/transformer.cpp:6181-6293: embed, positions, every block)."""
    x = add_positions(embed(tokens, m.tensors["wte.weight"]), m.tensors["wpe.weight"], 0)
    for layer in range(m.n_layer):
        x = block(x, m, layer)
    return x


def forward_logits(m: PlainModel, tokens: Sequence[int]) -> np.ndarray:
    """Logits [len(tokens), vocab] of a whole sequence, float64."""
    return final_logits(hidden_states(m, tokens), m)


# --------------------------------------------------------------------------- sampling

def sampler_probabilities(logits: np.ndarray, temperature: float, top_k: int, top_p: float) -> np.ndarray:
    """temperature -> top-k -> sort -> softmax (maximum subtracted, exp in
    float, sum in double) -> top-p over the sorted candidates -> renormalise by
    the kept mass; greedy (temperature <= 0) is one-hot at the first maximum
    (src/core/sampling.cpp:12-61).  Ties are ordered by index, lowest first."""
    n = logits.shape[0]
    probs = np.zeros(n, dtype=np.float32)
    logits = logits.astype(np.float32)
    if temperature <= 0.0:
        probs[int(np.argmax(logits))] = 1.0
        return probs
    ids = np.lexsort((np.arange(n), -logits.astype(np.float64)))        # by logit descending, then index
    if 0 < top_k < n:
        ids = ids[:top_k]
    inv_t = np.float32(1.0) / np.float32(temperature)
    mx = logits[ids[0]]
    p = np.exp(((logits[ids] - mx) * inv_t).astype(np.float32)).astype(np.float32)
    total = float(p.astype(np.float64).sum())
    keep = len(ids)
    if top_p < 1.0:
        cumulative = 0.0
        for i in range(len(ids)):
            cumulative += float(p[i]) / total
            if cumulative >= top_p:
                keep = i + 1
                break
    kept = float(p[:keep].astype(np.float64).sum())
    probs[ids[:keep]] = (p[:keep].astype(np.float64) / kept).astype(np.float32)
    return probs


def sampler_draw(probs: np.ndarray, u: float) -> int:
    """r = u * total, walk the ids in index order subtracting p_i until r < 0,
    else the last id with mass (src/core/sampling.cpp:66-79)."""
    total = float(probs.astype(np.float64).sum())
    if total <= 0.0:
        return int(np.argmax(probs))
    r = u * total
    for i in range(probs.shape[0]):
        r -= float(probs[i])
        if r < 0.0:
            return i
    nz = np.nonzero(probs > 0)[0]
    return int(nz[-1]) if len(nz) else 0


def uniform_draw(seed: int, stream: int, counter: int) -> float:
    """The engine's own uniform in [0, 1): SplitMix64 of a key built from the
    sampler seed, the request's stream number and the draw's index; the top 53
    bits scaled by 2^-53.  (The reference draws from mt19937_64, which a GPU
    sampler cannot share; the distribution it draws from is the reference's.)"""
    mask = 0xFFFFFFFFFFFFFFFF
    x = (seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + counter * 0x8CB92BA72F3D8DD7) & mask
    z = (x + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 11) * (1.0 / 9007199254740992.0)


def generate_greedy(m: PlainModel, prompt: Sequence[int], n_new: int) -> List[int]:
    """Greedy generation by recomputing the whole sequence at every step."""
    tokens = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(np.argmax(forward_logits(m, tokens)[-1].astype(np.float32)))
        out.append(nxt)
        tokens.append(nxt)
    return out
