"""Reading and writing the safetensors container.

The format: eight bytes of little-endian header length, a JSON object mapping
each tensor's name to {"dtype", "shape", "data_offsets": [begin, end)} (offsets
relative to the end of the header), then the raw little-endian data.  The
header is parsed and checked before any data is touched, as the reference
describes a model from metadata and tensor shapes alone
(src/compat/architecture.h:30-32) and rejects malformed files with the tensor
named (src/core/transformer.cpp:1052-1072).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch

from ..status import ErrorCode, LiyabError, invalid_model

_DTYPES: Dict[str, Tuple[torch.dtype, int]] = {
    "F64": (torch.float64, 8),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int      # absolute byte offsets in the file
    end: int


def _no_duplicates(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise invalid_model(f"tensor '{k}' appears twice in the header")
        seen[k] = v
    return seen


class SafetensorsFile:
    """A model file opened for reading: header checked, data mapped on demand."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise LiyabError(ErrorCode.IO_ERROR, f"cannot open {path}: {e}") from e
        if size < 8:
            raise invalid_model(f"{path}: file of {size} bytes is too short for a safetensors header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen < 2 or 8 + hlen > size:
            raise invalid_model(f"{path}: header length {hlen} does not fit a file of {size} bytes")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise invalid_model(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise invalid_model(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        base = 8 + hlen
        data_size = size - base
        self.entries: Dict[str, TensorEntry] = {}
        spans = []
        for name, info in header.items():
            try:
                dt, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise invalid_model(f"{path}: malformed header entry for tensor '{name}'") from ex
            if dt not in _DTYPES:
                raise invalid_model(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            tdt, isz = _DTYPES[dt]
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if any(s < 0 for s in shape) or not (0 <= b <= e) or e - b != count * isz:
                raise invalid_model(f"{path}: tensor '{name}' has the wrong size: shape {list(shape)} of {dt} "
                                    f"needs {count * isz} bytes, offsets give {e - b}")
            if e > data_size:
                raise invalid_model(f"{path}: tensor '{name}' ends at byte {e} but the file holds {data_size} "
                                    f"bytes of data (truncated file)")
            self.entries[name] = TensorEntry(name, tdt, shape, base + b, base + e)
            if e > b:
                spans.append((b, e, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise invalid_model(f"{path}: tensors '{n0}' and '{n1}' overlap in the file")
        self._map = None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def read(self, name: str) -> torch.Tensor:
        """The tensor's data as a CPU tensor (a copy, so the file may close)."""
        e = self.entries[name]
        if self._map is None:
            self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        n = e.end - e.begin
        if n == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=n, offset=e.begin).copy()
        return torch.from_numpy(raw).view(e.dtype).reshape(e.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    """Writes tensors in the order given; data starts 8-byte aligned."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise LiyabError(ErrorCode.INVALID_ARGUMENT, f"tensor '{name}' has dtype {t.dtype}, which cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for t in blobs:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
