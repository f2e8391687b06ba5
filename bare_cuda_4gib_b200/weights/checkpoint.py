"""A model folder's tensors: one `model.safetensors`, or shards named by `model.safetensors.index.json`.

A sharded checkpoint lists every tensor's file in the index's `weight_map`; each shard is opened
once.  What is wrong with the folder as a whole is collected in `problems` (a shard file that is
missing or unreadable, a tensor the index places in a shard that does not hold it, a tensor that
two shards hold), so that the loader can report it in its one error beside missing and unexpected
tensors.  (cuongvng/bare-cuda-4gib converts any Hugging Face checkpoint offline through
`from_pretrained`, tools/convert/convert_weights.py:17-24, which reads shards the same way.)
"""

from __future__ import annotations

import json
import pathlib
from typing import Dict, List, Tuple

from ..errors import WeightError
from .safetensors_io import SafetensorsFile, TensorEntry

WEIGHT_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


class Checkpoint:
    """`entries`: tensor name -> (open file, its entry); `problems`: what is wrong with the folder."""

    def __init__(self, folder):
        self.folder = pathlib.Path(folder)
        self.files: Dict[str, SafetensorsFile] = {}
        self.entries: Dict[str, Tuple[SafetensorsFile, TensorEntry]] = {}
        self.problems: List[str] = []
        index = self.folder / INDEX_FILE
        try:
            if index.exists():
                self.where = str(index)
                self._open_shards(index)
            else:
                self.where = str(self.folder / WEIGHT_FILE)
                f = self._open(WEIGHT_FILE)
                self.entries = {name: (f, e) for name, e in f.entries.items()}
        except BaseException:
            self.close()
            raise

    def _open(self, name: str) -> SafetensorsFile:
        f = SafetensorsFile(self.folder / name)
        self.files[name] = f
        return f

    def _open_shards(self, index: pathlib.Path) -> None:
        try:
            doc = json.loads(index.read_text())
            weight_map = doc["weight_map"]
            if not isinstance(weight_map, dict) or not all(isinstance(v, str) for v in weight_map.values()):
                raise TypeError("weight_map must map tensor names to file names")
        except (OSError, ValueError, KeyError, TypeError) as e:
            raise WeightError(f"{index}: not a usable shard index: {e}") from e
        for shard in sorted(set(weight_map.values())):
            if "/" in shard or "\\" in shard:
                self.problems.append(f"shard name '{shard}' leaves the model folder")
                continue
            try:
                self._open(shard)
            except WeightError as e:
                self.problems.append(f"shard {shard}: {e}")
        holders: Dict[str, List[str]] = {}
        for shard, f in self.files.items():
            for name in f.entries:
                holders.setdefault(name, []).append(shard)
        for name, shards in sorted(holders.items()):
            if len(shards) > 1:
                self.problems.append(f"tensor '{name}' is held by {len(shards)} shards: {', '.join(sorted(shards))}")
        for name, shard in sorted(weight_map.items()):
            f = self.files.get(shard)
            if f is None:
                continue                      # the shard itself is already reported
            if name not in f.entries:
                self.problems.append(f"tensor '{name}' is listed in shard {shard}, which does not hold it")
                continue
            self.entries[name] = (f, f.entries[name])
        for name, shards in holders.items():       # held by a shard but not listed: still a tensor of the folder
            if name not in weight_map and name not in self.entries:
                self.entries[name] = (self.files[shards[0]], self.files[shards[0]].entries[name])

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {name: e.shape for name, (_f, e) in self.entries.items()}

    def close(self) -> None:
        for f in self.files.values():
            f.close()
        self.files = {}

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
