"""Reads tensors by name from a model folder's safetensors files.

As the reference's ``CheckpointReader`` (utils/weights.py:15-55): a sharded checkpoint is found
through ``model.safetensors.index.json``'s ``weight_map``, else the single ``model.safetensors`` is
used; files are opened lazily and memory-mapped.  Only local folders are read; nothing is downloaded.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Tuple

INDEX_FILE = "model.safetensors.index.json"
SINGLE_FILE = "model.safetensors"


class CheckpointReader:
    def __init__(self, folder: str):
        self.folder = folder
        self._handles: Dict[str, object] = {}
        index_path = os.path.join(folder, INDEX_FILE)
        single_path = os.path.join(folder, SINGLE_FILE)
        if os.path.isfile(index_path):
            with open(index_path) as handle:
                self.file_of: Dict[str, str] = dict(json.load(handle)["weight_map"])
        elif os.path.isfile(single_path):
            self.file_of = {name: SINGLE_FILE for name in self._open(SINGLE_FILE).keys()}
        else:
            raise FileNotFoundError(f"{folder!r} has neither {INDEX_FILE} nor {SINGLE_FILE}")

    def _open(self, file_name: str):
        if file_name not in self._handles:
            from safetensors import safe_open

            self._handles[file_name] = safe_open(os.path.join(self.folder, file_name), framework="pt", device="cpu")
        return self._handles[file_name]

    def names(self) -> List[str]:
        return sorted(self.file_of)

    def has(self, name: str) -> bool:
        return name in self.file_of

    def shape_and_dtype(self, name: str) -> Tuple[Tuple[int, ...], str]:
        piece = self._open(self.file_of[name]).get_slice(name)
        return tuple(piece.get_shape()), str(piece.get_dtype())

    def get(self, name: str):
        return self._open(self.file_of[name]).get_tensor(name)

    def close(self) -> None:
        self._handles.clear()
