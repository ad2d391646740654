"""A model folder's tensors by name.

Discovery follows the reference's ``Checkpoint`` (src/weight/checkpoint.cpp:
233-276, 286-369, 371-500): one ``*.safetensors.index.json`` names the files
to open (and every tensor must live in the file the index says); without an
index the folder holds ``model.safetensors``, ``consolidated.safetensors``, a
complete ``model-0000i-of-0000n.safetensors`` family, or a single file.
"""

from __future__ import annotations

import json
import re
from pathlib import Path

import torch

from ..config.errors import WeightError
from .safetensors_io import SafetensorsFile, TensorRecord

_SHARD = re.compile(r"^(?P<stem>.+)-(?P<index>\d{5})-of-(?P<total>\d{5})\.safetensors$")


class Checkpoint:
    def __init__(self, model_dir: str | Path):
        self.model_dir = Path(model_dir)
        if not self.model_dir.is_dir():
            raise WeightError(f"model folder does not exist: {self.model_dir}")
        self._files: dict[Path, SafetensorsFile] = {}
        self.records: dict[str, TensorRecord] = {}
        indexes = sorted(self.model_dir.glob("*.safetensors.index.json"))
        if len(indexes) > 1:
            raise WeightError(f"{self.model_dir}: several safetensors index files; keep one")
        if indexes:
            self._load_with_index(indexes[0])
        else:
            self._load_without_index()

    # ---------------------------------------------------------------- discovery
    def _open(self, path: Path) -> SafetensorsFile:
        if path not in self._files:
            self._files[path] = SafetensorsFile(path)
        return self._files[path]

    def _load_with_index(self, index_path: Path) -> None:
        try:
            index = json.loads(index_path.read_text(encoding="utf-8"))
        except (OSError, json.JSONDecodeError) as error:
            raise WeightError(f"{index_path}: cannot read the index: {error}") from error
        weight_map = index.get("weight_map") if isinstance(index, dict) else None
        if not isinstance(weight_map, dict) or not weight_map:
            raise WeightError(f"{index_path}: 'weight_map' must be a non-empty object")
        for name, relative in weight_map.items():
            if (not isinstance(relative, str) or not relative.endswith(".safetensors")
                    or Path(relative).is_absolute() or ".." in Path(relative).parts):
                raise WeightError(f"{index_path}: tensor '{name}' maps to the invalid file {relative!r}")
            file = self._open(self.model_dir / relative)
            if name not in file.records:
                raise WeightError(f"{index_path}: tensor '{name}' is not in {relative} as the index says")
            self.records[name] = file.records[name]

    def _load_without_index(self) -> None:
        for fixed in ("model.safetensors", "consolidated.safetensors"):
            if (self.model_dir / fixed).is_file():
                self._take_all(self._open(self.model_dir / fixed))
                return
        candidates = sorted(self.model_dir.glob("*.safetensors"))
        families: dict[tuple[str, int], dict[int, Path]] = {}
        for path in candidates:
            match = _SHARD.match(path.name)
            if match:
                families.setdefault((match["stem"], int(match["total"])), {})[int(match["index"])] = path
        if families:
            if len(families) > 1:
                raise WeightError(f"{self.model_dir}: several shard families; add an index file")
            (stem, total), shards = next(iter(families.items()))
            if sorted(shards) != list(range(1, total + 1)):
                raise WeightError(f"{self.model_dir}: shard family '{stem}' is incomplete "
                                  f"({len(shards)} of {total} files)")
            for index in sorted(shards):
                self._take_all(self._open(shards[index]))
            return
        if len(candidates) == 1:
            self._take_all(self._open(candidates[0]))
            return
        if not candidates:
            raise WeightError(f"{self.model_dir}: no safetensors file found")
        raise WeightError(f"{self.model_dir}: several safetensors files and no index; cannot choose")

    def _take_all(self, file: SafetensorsFile) -> None:
        for name, record in file.records.items():
            if name in self.records:
                raise WeightError(f"tensor '{name}' appears in {self.records[name].file} and {file.path}")
            self.records[name] = record

    # ------------------------------------------------------------------- access
    def names(self) -> tuple[str, ...]:
        return tuple(self.records)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.records[name].shape

    def dtype(self, name: str) -> torch.dtype:
        return self.records[name].dtype

    def read(self, name: str) -> torch.Tensor:
        record = self.records[name]
        return self._files[record.file].read(name)
