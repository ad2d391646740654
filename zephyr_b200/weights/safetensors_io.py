"""Reading and writing the safetensors container, with the reference's checks.

Format: an 8-byte little-endian header length, a JSON header mapping tensor
names to ``{"dtype", "shape", "data_offsets"}``, then the raw data.  The
checks follow ``ParseSafetensorsFile`` (src/weight/checkpoint.cpp:502-630):
the header lies within the file, every range lies within the data section,
byte counts equal ``numel * itemsize``, names are unique, non-empty ranges do
not overlap, ``__metadata__`` is a map of strings, and only the dtypes of
src/weight/checkpoint.cpp:121-161 are known.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Mapping

import torch

from ..config.errors import WeightError

_DTYPES: dict[str, torch.dtype] = {
    "BOOL": torch.bool,
    "U8": torch.uint8,
    "I32": torch.int32,
    "I64": torch.int64,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "F32": torch.float32,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int          # absolute byte offset in the file
    end: int
    file: Path

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


class SafetensorsFile:
    """One memory-mapped file; tensors are read as views of the map."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        try:
            with open(self.path, "rb") as handle:
                size = handle.seek(0, 2)
                if size < 8:
                    raise WeightError(f"{self.path}: too short to hold a safetensors header")
                # A private copy-on-write map: nothing reaches the file, and the buffer counts as writable,
                # which torch.frombuffer wants.
                self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY)
        except OSError as error:
            raise WeightError(f"cannot open checkpoint file {self.path}: {error.strerror}") from error
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > size - 8:
            raise WeightError(f"{self.path}: header length {header_len} exceeds the file size {size}")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"),
                                object_pairs_hook=self._no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise WeightError(f"{self.path}: the header is not valid JSON: {error}") from error
        if not isinstance(header, dict):
            raise WeightError(f"{self.path}: the header must be a JSON object")
        data_start = 8 + header_len
        data_size = size - data_start
        self.metadata: dict[str, str] = {}
        self.records: dict[str, TensorRecord] = {}
        ranges = []
        for name, entry in header.items():
            if name == "__metadata__":
                if not isinstance(entry, dict) or any(not isinstance(v, str) for v in entry.values()):
                    raise WeightError(f"{self.path}: __metadata__ must map strings to strings")
                self.metadata = dict(entry)
                continue
            if not isinstance(entry, dict) or not {"dtype", "shape", "data_offsets"} <= set(entry):
                raise WeightError(f"{self.path}: tensor '{name}' lacks dtype, shape or data_offsets")
            if entry["dtype"] not in _DTYPES:
                raise WeightError(f"{self.path}: tensor '{name}' has the unsupported dtype {entry['dtype']!r}")
            dtype = _DTYPES[entry["dtype"]]
            shape = entry["shape"]
            offsets = entry["data_offsets"]
            if (not isinstance(shape, list) or any(isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape)
                    or not isinstance(offsets, list) or len(offsets) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) or o < 0 for o in offsets)):
                raise WeightError(f"{self.path}: tensor '{name}' has a malformed shape or data_offsets")
            begin, end = offsets
            if begin > end or end > data_size:
                raise WeightError(f"{self.path}: tensor '{name}' data range [{begin}, {end}) lies outside the file")
            numel = 1
            for d in shape:
                numel *= d
            if end - begin != numel * _itemsize(dtype):
                raise WeightError(
                    f"{self.path}: tensor '{name}' has {end - begin} bytes but shape {shape} of "
                    f"{entry['dtype']} needs {numel * _itemsize(dtype)}")
            self.records[name] = TensorRecord(name, dtype, tuple(shape), data_start + begin, data_start + end,
                                              self.path)
            if end > begin:
                ranges.append((begin, end, name))
        ranges.sort()
        for (b0, e0, n0), (b1, _e1, n1) in zip(ranges, ranges[1:]):
            if b1 < e0:
                raise WeightError(f"{self.path}: tensors '{n0}' and '{n1}' overlap in the data section")

    def _no_duplicates(self, pairs):
        out = {}
        for key, value in pairs:
            if key in out:
                raise WeightError(f"{self.path}: the header names '{key}' twice")
            out[key] = value
        return out

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (read-only: clone or convert before writing)."""
        record = self.records[name]
        if record.numel == 0:
            return torch.empty(record.shape, dtype=record.dtype)
        flat = torch.frombuffer(self._map, dtype=record.dtype, count=record.numel, offset=record.begin)
        return flat.view(record.shape)


def save_safetensors(path: str | Path, tensors: Mapping[str, torch.Tensor],
                     metadata: Mapping[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU or CUDA, contiguous or not) as one safetensors file, names sorted."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise WeightError(f"cannot store tensor '{name}' of dtype {tensor.dtype}")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)     # keeps the data section 8-byte aligned
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in order:
            tensor = tensors[name].detach().contiguous().cpu()
            if tensor.numel():
                handle.write(tensor.view(torch.uint8).numpy().tobytes() if tensor.dim() else
                             tensor.reshape(1).view(torch.uint8).numpy().tobytes())
