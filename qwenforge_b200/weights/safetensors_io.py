"""Reader and writer of the safetensors container: 8 bytes little-endian header length, a JSON
header {name: {dtype, shape, data_offsets}}, then the tensors' bytes. Tensors are read through a
memory map, one at a time, so a file larger than host memory can be loaded tensor by tensor."""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path
from typing import Mapping

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One opened file: `names()`, `info(name)` -> (dtype, shape), `tensor(name)` -> CPU tensor (a copy)."""

    def __init__(self, path):
        self.path = Path(path)
        self._file = open(self.path, "rb")
        head = self._file.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: too short to be a safetensors file")
        (header_len,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if header_len <= 0 or 8 + header_len > size:
            raise ValueError(f"{self.path}: header length {header_len} does not fit the file ({size} bytes)")
        header = json.loads(self._file.read(header_len).decode("utf-8"))
        header.pop("__metadata__", None)
        self._entries = header
        self._data_start = 8 + header_len
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for name, entry in header.items():
            if entry["dtype"] not in _DTYPES:
                raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {entry['dtype']}")
            begin, end = entry["data_offsets"]
            if not (0 <= begin <= end and self._data_start + end <= size):
                raise ValueError(f"{self.path}: tensor {name!r} lies outside the file")

    def names(self) -> list[str]:
        return list(self._entries)

    def info(self, name: str):
        entry = self._entries[name]
        return _DTYPES[entry["dtype"]], tuple(entry["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        entry = self._entries[name]
        dtype, shape = _DTYPES[entry["dtype"]], tuple(entry["shape"])
        begin, end = entry["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)  # the read-only map is copied at once, never written
            flat = torch.frombuffer(view, dtype=dtype, count=count)
        return flat.reshape(shape).clone()

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass  # a tensor view is still alive; the map goes with it
            self._map = None
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def save_safetensors(path, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write `tensors` (CPU or device tensors) as one safetensors file, names sorted."""
    header = {}
    offset = 0
    ordered = sorted(tensors)
    for name in ordered:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise ValueError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in ordered:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
