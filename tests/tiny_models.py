"""The tests' small configurations and helpers that write them as model folders.

A and B differ in every size and option GPT-2 has: layers, width, heads (so head
size), inner width (4x and not), vocabulary (a power of two and not even a
multiple of 64), positions, the norms' eps, the activation, and the per-layer
attention factor.  C is a third, odd one used for kernels' corner sizes.
"""
from __future__ import annotations

import json
import os

import numpy as np

CONFIG_A = dict(model_type="gpt2", n_layer=2, n_embd=64, n_head=4, n_inner=256, vocab_size=512, n_positions=128,
                layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
                tie_word_embeddings=True)
CONFIG_B = dict(model_type="gpt2", n_layer=3, n_embd=96, n_head=3, n_inner=320, vocab_size=1000, n_positions=256,
                layer_norm_epsilon=1e-6, activation_function="gelu", scale_attn_by_inverse_layer_idx=True,
                tie_word_embeddings=True)
CONFIG_C = dict(model_type="gpt2", n_layer=1, n_embd=240, n_head=5, n_inner=136, vocab_size=777, n_positions=320,
                layer_norm_epsilon=1e-3, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=True,
                scale_attn_weights=True, tie_word_embeddings=True)
# Head sizes 64 and 128: the shapes the fused decode step takes.
CONFIG_D = dict(model_type="gpt2", n_layer=3, n_embd=128, n_head=2, n_inner=328, vocab_size=777, n_positions=300,
                layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False,
                tie_word_embeddings=True)
CONFIG_E = dict(model_type="gpt2", n_layer=2, n_embd=384, n_head=3, n_inner=1000, vocab_size=1031, n_positions=200,
                layer_norm_epsilon=1e-6, activation_function="gelu", scale_attn_by_inverse_layer_idx=True,
                tie_word_embeddings=True)
CONFIGS = {"A": (CONFIG_A, 0), "B": (CONFIG_B, 1), "C": (CONFIG_C, 2), "D": (CONFIG_D, 3), "E": (CONFIG_E, 4)}


def write_model(folder: str, name: str, dtype: str = "float32") -> str:
    """Writes configuration `name` with its seed into `folder`/<name>_<dtype> and returns that path."""
    from liyab_b200.weights import write_random_model
    raw, seed = CONFIGS[name]
    path = os.path.join(folder, f"{name}_{dtype}")
    if not os.path.isfile(os.path.join(path, "model.safetensors")):
        write_random_model(path, raw, seed, dtype)
    return path


def random_tokens(seed: int, n: int, vocab: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, size=n).astype(int).tolist()
