"""Weights by tensor name, checked as a whole before any is used.

Every parameter the configuration asks for is looked up by its name in the
model file; a file that lacks a tensor, holds one nobody asked for, or has one
of the wrong shape is refused with ONE error that lists all three kinds, in the
words of the reference's loader ("missing tensor 'X'", "tensor 'X' has shape
[..], expected [..]": src/core/transformer.cpp:1052-1072).

Storage types.  In the 32-bit mode every floating tensor is widened to float32.
In the bfloat16 mode matrices and embedding tables (the operands of matrix
products) are kept in bfloat16, while vectors (norm gains, biases) stay or
become float32, which the kernels add in 32-bit anyway; integer tensors become
int32.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Mapping

import torch

from ..config.registry import ArchitectureConfig
from ..status import invalid_argument, invalid_model
from .safetensors_io import SafetensorsFile

COMPUTE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_ALIASES = {"fp32": "float32", "f32": "float32", "bf16": "bfloat16", "float32": "float32", "bfloat16": "bfloat16"}


def canonical_dtype(name: str) -> str:
    if name not in _ALIASES:
        raise invalid_argument(f"unknown dtype {name!r}; choose bfloat16 or float32")
    return _ALIASES[name]


def _storage_dtype(kind: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32 or kind == "vector":
        return torch.float32
    return compute


def load_parameters(model_dir: str, config: ArchitectureConfig, dtype: str, device: str | torch.device
                    ) -> Dict[str, torch.Tensor]:
    """Reads model.safetensors of `model_dir` into {parameter path: tensor}."""
    compute = COMPUTE_DTYPES[canonical_dtype(dtype)]
    path = os.path.join(model_dir, "model.safetensors")
    wanted = config.checkpoint_map()
    prefixes = getattr(config, "name_prefixes", lambda: ("",))()
    with SafetensorsFile(path) as f:
        names = set(f.names())
        prefix = max(prefixes, key=lambda p: sum((p + s.name) in names for s in wanted.values()))
        missing: List[str] = []
        wrong: List[str] = []
        used = set()
        for spec in wanted.values():
            full = prefix + spec.name
            if full not in names:
                missing.append(f"missing tensor '{full}'")
                continue
            used.add(full)
            entry = f.entries[full]
            if tuple(entry.shape) != tuple(spec.shape):
                wrong.append(f"tensor '{full}' has shape {list(entry.shape)}, expected {list(spec.shape)}")
            elif not entry.dtype.is_floating_point and spec.kind != "index":
                wrong.append(f"tensor '{full}' has dtype {entry.dtype}, expected a floating type")
        # A tensor that carries no weights may sit under the file's prefix or outside it
        # (a stored copy of a tied head usually does not carry the body's prefix).
        ignored = [re.compile("^(?:" + re.escape(prefix) + ")?" + p + "$") for p in config.ignored_tensors()]
        unexpected = sorted(n for n in names - used if not any(p.match(n) for p in ignored))
        if missing or wrong or unexpected:
            parts = []
            if missing:
                parts.append(f"{len(missing)} missing: " + "; ".join(missing))
            if unexpected:
                parts.append(f"{len(unexpected)} unexpected: " + "; ".join(f"unexpected tensor '{n}'" for n in unexpected))
            if wrong:
                parts.append(f"{len(wrong)} of the wrong shape: " + "; ".join(wrong))
            raise invalid_model(f"{path} does not fit the configuration. " + " | ".join(parts))
        params: Dict[str, torch.Tensor] = {}
        for dest, spec in wanted.items():
            t = f.read(prefix + spec.name).to(device)
            if spec.transform == "transpose":
                t = t.t()
            elif spec.transform != "none":
                raise invalid_model(f"unknown transform {spec.transform!r} for tensor '{spec.name}'")
            params[dest] = t.to(_storage_dtype(spec.kind, t.dtype, compute)).contiguous()
    return params


def random_parameters(spec_map: Mapping[str, tuple], seed: int, dtype: str, device: str | torch.device,
                      std: float = 0.05) -> Dict[str, torch.Tensor]:
    """Seeded parameters for a model that has no file format of its own (toy
    parts in tests): `spec_map` is {parameter path: (shape, kind)}."""
    from .random_init import normal_values
    compute = COMPUTE_DTYPES[canonical_dtype(dtype)]
    out = {}
    for dest, (shape, kind) in spec_map.items():
        n = 1
        for s in shape:
            n *= s
        mean = 1.0 if dest.endswith("norm.weight") else 0.0
        v = torch.from_numpy(normal_values(seed, dest, n, mean, std)).to(torch.float32).reshape(shape)
        out[dest] = v.to(device).to(_storage_dtype(kind, torch.float32, compute)).contiguous()
    return out
