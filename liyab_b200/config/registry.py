"""The one registry from an architecture's name to its configuration and model.

The reference keeps a table of `ArchSpec` rows keyed by `general.architecture`
and answers an unknown name with `Unsupported` plus the list of names it knows
(src/compat/architecture.cpp:19-426, 578-585).  Here a row is an `Architecture`
whose `parse` turns the dictionary of config.json into a typed configuration;
that configuration yields the `ModelSpec` and the map from parameters to the
tensor names of the model file.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Protocol, Sequence

from ..status import ErrorCode, LiyabError, invalid_model, unsupported
from .spec import CheckpointTensor, ModelSpec


class ArchitectureConfig(Protocol):
    """What every architecture's typed configuration offers the framework."""

    def to_dict(self) -> Dict[str, Any]: ...
    def model_spec(self) -> ModelSpec: ...
    def checkpoint_map(self) -> Mapping[str, CheckpointTensor]: ...
    def ignored_tensors(self) -> Sequence[str]: ...


@dataclass(frozen=True)
class Architecture:
    name: str                               # config.json "model_type"
    class_names: Sequence[str]              # config.json "architectures" entries
    parse: Callable[[Mapping[str, Any]], ArchitectureConfig]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def supported_architectures() -> Sequence[str]:
    return sorted(_ARCHITECTURES)


def find_architecture(config: Mapping[str, Any]) -> Architecture:
    """Chooses the row by `model_type`, else by the first of `architectures`."""
    name = config.get("model_type")
    if isinstance(name, str) and name in _ARCHITECTURES:
        return _ARCHITECTURES[name]
    for cls in config.get("architectures") or []:
        for arch in _ARCHITECTURES.values():
            if cls in arch.class_names:
                return arch
    shown = name if name is not None else (config.get("architectures") or "nothing")
    raise unsupported(
        f"architecture {shown!r} is not supported; supported: {', '.join(supported_architectures())}")


def parse_config(config: Mapping[str, Any]) -> ArchitectureConfig:
    return find_architecture(config).parse(config)


def read_config(model_dir: str) -> ArchitectureConfig:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except OSError as e:
        raise LiyabError(ErrorCode.IO_ERROR, f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise invalid_model(f"{path} is not valid JSON: {e}") from e
    if not isinstance(raw, dict):
        raise invalid_model(f"{path} does not hold a JSON object")
    return parse_config(raw)
