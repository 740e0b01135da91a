"""Model files: the safetensors container, the by-name loader and the random-weights mode.

All of it is the library's (host/safetensors.cpp, host/weights.cpp); tensors cross
as NumPy arrays (bfloat16 as uint16 bit patterns, see `bf16_to_f32`).
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Any, Dict, Mapping, Optional

import numpy as np

from .. import _capi

_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32,
       "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
_NAMES = {"float32": np.float32, "bfloat16": np.uint16, "int32": np.int32}


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round to nearest even, as the library does."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_random_model(model_dir: str, raw_config: Mapping[str, Any], seed: int, dtype: str = "float32") -> str:
    """Writes `model_dir`/config.json and model.safetensors from a configuration and a seed; returns the folder."""
    _capi.check(_capi.lib().lb_write_random_model(_capi.b(json.dumps(raw_config)), seed, _capi.b(dtype), _capi.b(model_dir)))
    return model_dir


def normal_values(seed: int, name: str, count: int, mean: float, std: float, first: int = 0) -> np.ndarray:
    out = np.empty(count, dtype=np.float64)
    _capi.check(_capi.lib().lb_normal_values(seed, _capi.b(name), first, count, mean, std, out.ctypes.data_as(C.POINTER(C.c_double))))
    return out


def safetensors_describe(path: str) -> Dict[str, Any]:
    """{"metadata": {...}, "tensors": {name: {"dtype", "shape", "bytes"}}}; raises on a malformed file."""
    return _capi.json_of(_capi.lib().lb_safetensors_describe, _capi.b(path))


def read_tensor(path: str, name: str, info: Optional[Mapping[str, Any]] = None) -> np.ndarray:
    info = info or safetensors_describe(path)["tensors"][name]
    out = np.empty(info["shape"], dtype=_NP[info["dtype"]])
    _capi.check(_capi.lib().lb_safetensors_read(_capi.b(path), _capi.b(name), out.ctypes.data, out.nbytes))
    return out


def write_safetensors(path: str, tensors: Mapping[str, np.ndarray], metadata: Optional[Mapping[str, str]] = None,
                      tags: Optional[Mapping[str, str]] = None) -> None:
    """Writes NumPy arrays in the order given; `tags` overrides a tensor's stored type (e.g. "BF16" for uint16 bits)."""
    rev = {np.dtype(v): k for k, v in _NP.items() if k != "BF16"}
    names, dts, ranks, shapes, ptrs, keep = [], [], [], [], [], []
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        keep.append(a)
        names.append(_capi.b(name))
        dts.append(_capi.b((tags or {}).get(name) or rev[a.dtype]))
        ranks.append(a.ndim)
        shapes.extend(a.shape)
        ptrs.append(a.ctypes.data)
    n = len(names)
    _capi.check(_capi.lib().lb_safetensors_write(
        _capi.b(path), n, (C.c_char_p * n)(*names), (C.c_char_p * n)(*dts), (C.c_int32 * n)(*ranks),
        (C.c_int64 * max(1, len(shapes)))(*shapes), (C.c_void_p * n)(*ptrs), _capi.b(json.dumps(dict(metadata or {})))))


def load_parameters(model_dir: str, dtype: str = "float32") -> Dict[str, np.ndarray]:
    """The model's parameters as the engine would hold them for `dtype`: {path: array}, matrices [out, in]."""
    l = _capi.lib()
    handle = C.c_void_p()
    _capi.check(l.lb_weights_load(_capi.b(model_dir), _capi.b(dtype), C.byref(handle)))
    try:
        out = {}
        for name, info in _capi.json_of(l.lb_weights_describe, handle).items():
            data, n = C.c_void_p(), C.c_size_t()
            _capi.check(l.lb_weights_data(handle, _capi.b(name), C.byref(data), C.byref(n)))
            raw = C.string_at(data.value, n.value) if n.value else b""
            out[name] = np.frombuffer(raw, dtype=_NAMES[info["dtype"]]).reshape(info["shape"]).copy()
        return out
    finally:
        l.lb_weights_free(handle)


__all__ = ["bf16_to_f32", "f32_to_bf16", "write_random_model", "normal_values", "safetensors_describe", "read_tensor",
           "write_safetensors", "load_parameters"]
