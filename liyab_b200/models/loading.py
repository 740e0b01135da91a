"""From a model folder to a model on the device.

config.json chooses the architecture through the registry; the architecture's
typed configuration gives the `ModelSpec` and the names of the file's tensors;
the loader reads them; the generic decoder is built from spec and parameters.
The reference's load runs the same stages: describe, bind by name, size the
cache, build (src/core/transformer.cpp:712-1046).
"""
from __future__ import annotations

from typing import Tuple

import torch

from ..config.registry import ArchitectureConfig, read_config
from ..parts.base import Runtime
from ..status import backend_error
from ..weights.loader import COMPUTE_DTYPES, canonical_dtype, load_parameters
from .decoder import DecoderModel


def load_model(model_dir: str, dtype: str = "bfloat16", device: str = "cuda:0") -> Tuple[DecoderModel, ArchitectureConfig]:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise backend_error(f"the engine runs on a CUDA device only (asked for {device})")
    if not torch.cuda.is_available():
        raise backend_error("no CUDA device is available; the engine has no CPU path")
    config = read_config(model_dir)
    name = canonical_dtype(dtype)
    params = load_parameters(model_dir, config, name, dev)
    model = DecoderModel(config.model_spec(), params, Runtime(dtype=COMPUTE_DTYPES[name], device=dev))
    return model, config
