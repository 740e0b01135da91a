"""Typed configurations and the architecture registry, as the library describes them.

`describe_config(raw)` parses the dictionary of a config.json through the registry
and returns {"architecture", "config": the typed configuration, "spec": the model
as data (layers of named slots, run order, head), "checkpoint": parameter path ->
tensors of the model file}.  Errors carry the library's status code and name the key.
"""
from __future__ import annotations

import json
from typing import Any, Dict, List, Mapping

from .. import _capi


def describe_config(raw: Mapping[str, Any]) -> Dict[str, Any]:
    return _capi.json_of(_capi.lib().lb_config_describe, _capi.b(json.dumps(raw)))


def parse_config(raw: Mapping[str, Any]) -> Dict[str, Any]:
    """The typed configuration (every key with its default applied)."""
    return describe_config(raw)["config"]


def read_config(model_dir: str) -> Dict[str, Any]:
    return _capi.json_of(_capi.lib().lb_config_describe_folder, _capi.b(model_dir))


def supported_architectures() -> List[str]:
    return _capi.json_of(_capi.lib().lb_supported_architectures)


def load_plugin(path: str) -> None:
    """Registers the parts and architectures of a shared object built against the library's headers."""
    _capi.check(_capi.lib().lb_load_plugin(_capi.b(path)))


def slot(layer: Mapping[str, Any], name: str) -> Dict[str, Any]:
    """The part in the slot `name` of a layer of a described spec."""
    for s in layer["slots"]:
        if s["name"] == name:
            return s["part"]
    raise KeyError(name)


__all__ = ["describe_config", "parse_config", "read_config", "supported_architectures", "load_plugin", "slot"]
