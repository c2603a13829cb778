"""
Reader and writer of the safetensors container: an 8-byte little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the tensors' raw little-endian bytes.

The reference reads checkpoints with the safetensors package (model/loader.py:41-60); this file
is the engine's own reader so that a model folder is all it needs.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass

import torch

_DTYPES = {
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F32": torch.float32,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int          # byte offsets into the data section
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are materialised one at a time."""

    def __init__(self, path: str) -> None:
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than its 8-byte header length")
        self._file = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len > size - 8:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file ({size} bytes): truncated?")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not JSON ({exc})") from None
        self._data_start = 8 + header_len
        data_len = size - self._data_start
        self.metadata = header.pop("__metadata__", None) or {}
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {info['dtype']!r}")
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(d) for d in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            count = 1
            for d in shape:
                count *= d
            if end - begin != count * dtype.itemsize:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans {end - begin} bytes but shape {shape} of {info['dtype']} "
                    f"needs {count * dtype.itemsize}")
            if begin < 0 or end > data_len:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} ends at byte {end} of a {data_len}-byte data section: truncated?")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor holding a copy of the named tensor's data, in its stored dtype."""
        entry = self.entries[name]
        count = 1
        for d in entry.shape:
            count *= d
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        view = memoryview(self._map)[self._data_start + entry.begin: self._data_start + entry.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)       # the map is read-only; the data is cloned right away
            flat = torch.frombuffer(view, dtype=entry.dtype, count=count)
        return flat.reshape(entry.shape).clone()

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass                      # a view is still alive; the map goes with the process
            self._map = None
        self._file.close()

    def __enter__(self) -> "SafetensorsFile":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Write CPU tensors (contiguous copies are made) under their names, in the order given."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)       # keep the data section 8-byte aligned
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for t in tensors.values():
            t = t.detach().to("cpu").contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
