"""A small reader and writer for the safetensors container.

Layout of a file: 8 bytes little-endian header length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``, then
the raw little-endian tensor data; offsets are relative to the end of the header.
The reader maps the file and hands out zero-copy torch views.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped file: ``entries`` lists name -> (dtype string, shape); ``tensor(name)``
    returns a CPU tensor that views the mapping (copy before the file object dies)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            dt, shape = info["dtype"], tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            if dt in _DTYPES:
                want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dt][1] if shape else _DTYPES[dt][1]
                if e - b != want:
                    raise SafetensorsError(
                        f"{path}: tensor {name!r} spans {e - b} bytes, its shape {shape} and dtype {dt} need {want}")
            if self._data_start + e > size:
                raise SafetensorsError(f"{path}: tensor {name!r} reaches beyond the end of the file")
            self._entries[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    @property
    def entries(self) -> Dict[str, Tuple[str, Tuple[int, ...]]]:
        return {k: (v[0], v[1]) for k, v in self._entries.items()}

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, e = self._entries[name]
        if dt not in _DTYPES:
            raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dt}")
        tdt, _ = _DTYPES[dt]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self._data_start + b:self._data_start + e]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the mapping is read-only; callers copy
            return torch.frombuffer(buf, dtype=tdt).view(shape)

    def close(self):
        # views handed out keep the mapping alive through their buffer; only drop our handles
        self._mm = None
        self._f.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] = None) -> None:
    """Write ``tensors`` (CPU, contiguous) in name order."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order: List[str] = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def open_model_files(folder: str) -> List[SafetensorsFile]:
    """All ``*.safetensors`` of a model folder (one file, or shards named by an index)."""
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
    else:
        names = sorted(n for n in os.listdir(folder) if n.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"no .safetensors file in {folder}")
    return [SafetensorsFile(os.path.join(folder, n)) for n in names]
