"""Reader and writer for the safetensors container, written against the format itself: 8 bytes
of little-endian header length, a JSON header {name: {dtype, shape, data_offsets}}, then raw
little-endian tensor data.  (cuongvng/bare-cuda-4gib reads a private container instead,
engine/src/loader.cpp:55-148; its failure cases - cannot open, truncated file, data range
exceeds file - have their counterparts here.)
"""

from __future__ import annotations

import json
import mmap
import pathlib
import struct
from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np
import torch

from ..errors import WeightError

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """An open file: `entries` by name, `tensor(name)` as a CPU tensor that views the mapping."""

    def __init__(self, path):
        self.path = pathlib.Path(path)
        try:
            self._file = open(self.path, "rb", buffering=0)
        except OSError as e:
            raise WeightError(f"cannot open {self.path}: {e}") from e
        size = self.path.stat().st_size
        head = self._file.read(8)
        if len(head) < 8:
            raise WeightError(f"{self.path}: truncated file (no header length)")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise WeightError(f"{self.path}: header length {n} exceeds the file ({size} bytes)")
        def no_duplicates(pairs):
            seen = {}
            for key, value in pairs:
                if key in seen:
                    raise WeightError(f"{self.path}: tensor '{key}' is listed twice in the header")
                seen[key] = value
            return seen

        try:
            header = json.loads(self._file.read(n).decode("utf-8"), object_pairs_hook=no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightError(f"{self.path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise WeightError(f"{self.path}: header must be a JSON object")
        self.data_start = 8 + n
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise WeightError(f"{self.path}: malformed header entry for '{name}'") from e
            if dtype_name not in _DTYPES:
                raise WeightError(f"{self.path}: tensor '{name}' has unknown dtype '{dtype_name}'")
            dtype, width = _DTYPES[dtype_name]
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if end - begin != count * width:
                raise WeightError(f"{self.path}: tensor '{name}' of shape {shape} and dtype {dtype_name} "
                                  f"needs {count * width} bytes, its data range holds {end - begin}")
            if begin < 0 or self.data_start + end > size:
                raise WeightError(f"{self.path}: data range of tensor '{name}' exceeds the file")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=e.end - e.begin,
                            offset=self.data_start + e.begin)
        return torch.from_numpy(raw.copy()).view(e.dtype).reshape(e.shape)

    def read_into(self, name: str, out: np.ndarray, begin: int = 0) -> None:
        """Reads `out.nbytes` bytes of the tensor's data, from byte `begin` of it, straight into
        `out` (a contiguous uint8 array, for instance a view of pinned memory): no copy in between."""
        e = self.entries[name]
        if begin < 0 or begin + out.nbytes > e.end - e.begin:
            raise WeightError(f"{self.path}: read of {out.nbytes} bytes at {begin} exceeds tensor '{name}'")
        self._file.seek(self.data_start + e.begin + begin)
        view = memoryview(out).cast("B")
        got = 0
        while got < out.nbytes:
            n = self._file.readinto(view[got:])
            if not n:
                raise WeightError(f"{self.path}: file ended inside tensor '{name}'")
            got += n

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: Dict[str, torch.Tensor]) -> None:
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise WeightError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
