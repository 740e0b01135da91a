"""Random-weights mode: a model folder from a configuration and a seed.

The reference's tests write tiny models on the fly from a seed and a weight
scale (tests/test_model.h:64-318).  Here the folder holds config.json and
model.safetensors in the architecture's own tensor names and layouts, so it is
read back through the ordinary loader.  Values come from a counter-based
generator (SplitMix64 of a key made of the seed and the tensor's name, plus the
element's index, then Box-Muller in 64-bit), so a tensor's values depend on
nothing but (seed, name, index): not on the order tensors are written in, nor
on a library's normal distribution.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import numpy as np
import torch

from ..config.registry import ArchitectureConfig
from ..status import invalid_argument
from .safetensors_io import write_safetensors

_MASK = np.uint64(0xFFFFFFFFFFFFFFFF)
_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _fnv1a64(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def normal_values(seed: int, name: str, count: int, mean: float, std: float) -> np.ndarray:
    """`count` float64 draws of N(mean, std) for the tensor `name` under `seed`."""
    key = np.uint64((_fnv1a64(name) ^ ((seed * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF)) & 0xFFFFFFFFFFFFFFFF)
    out = np.empty(count, dtype=np.float64)
    chunk = 1 << 22
    for start in range(0, count, chunk):
        n = min(chunk, count - start)
        with np.errstate(over="ignore"):
            idx = np.arange(start, start + n, dtype=np.uint64) + key
        bits = _splitmix64(idx)
        hi = (bits >> np.uint64(32)).astype(np.float64)
        lo = (bits & np.uint64(0xFFFFFFFF)).astype(np.float64)
        u1 = (hi + 1.0) / 4294967296.0          # (0, 1]
        u2 = lo / 4294967296.0                  # [0, 1)
        out[start:start + n] = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return mean + std * out


def random_tensors(config: ArchitectureConfig, seed: int, dtype: str = "float32") -> Dict[str, torch.Tensor]:
    """Every tensor of the model file, in the file's names and layouts."""
    if dtype not in _STORE:
        raise invalid_argument(f"cannot store weights as {dtype!r}; choose one of {', '.join(_STORE)}")
    tensors: Dict[str, torch.Tensor] = {}
    for spec in config.checkpoint_map().values():
        count = int(np.prod(spec.shape, dtype=np.int64))
        values = normal_values(seed, spec.name, count, spec.init[0], spec.init[1]).astype(np.float32)
        tensors[spec.name] = torch.from_numpy(values).reshape(spec.shape).to(_STORE[dtype])
    return tensors


def write_random_model(model_dir: str, config: ArchitectureConfig, seed: int, dtype: str = "float32") -> str:
    """Writes `model_dir`/config.json and model.safetensors; returns the folder."""
    os.makedirs(model_dir, exist_ok=True)
    raw = dict(config.to_dict())
    raw["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(raw, f, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), random_tensors(config, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
