"""Binds the tensors of a model folder to the parts of a model, by tensor name.

Element types: in a bfloat16 run 16-bit floating tensors are kept in bfloat16 and a tensor stored
in 32-bit stays 32-bit; in a float32 run every floating tensor is widened to float32 (exact).
Integer tensors are kept as int32.  All problems of a folder are reported in ONE `WeightError`
that lists missing tensors, unexpected tensors, wrong shapes and what is wrong with the shards
(the reference stops at the first: engine/src/model.cpp:24-32, engine/src/loader.cpp:142-148).

Placement: every tensor goes into ONE device allocation at an offset aligned to 1,024 bytes, as the
reference does (engine/src/model.cpp:382-395).  Tensors that a part multiplies as one matrix
([Wq; Wk; Wv], [Wgate; Wup]: the model's `adjacent` groups) are placed back to back in that order,
so the part's fused matrix is a view of the arena and nothing is concatenated afterwards.  File
bytes are read straight into one of two pinned staging buffers and copied to the device
asynchronously, so that reading the next piece overlaps the copy of this one; a tensor whose stored
type differs from its kept type is converted on the device.
"""

from __future__ import annotations

import fnmatch
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import WeightError
from ..parts.spec import WeightSpec
from .checkpoint import WEIGHT_FILE, Checkpoint  # noqa: F401  (WEIGHT_FILE is part of this module's surface)

ARENA_ALIGN = 1024
STAGING_BYTES = 128 << 20


def storage_dtype(stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32 or stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def _ignorable(name: str, patterns: Sequence[str]) -> bool:
    return any(name == p or fnmatch.fnmatchcase(name, p) for p in patterns)


def check_names_and_shapes(expected: Dict[str, WeightSpec], present: Dict[str, Tuple[int, ...]],
                           aliases: Dict[str, str], ignorable=(), where: str = "",
                           problems: Sequence[str] = ()) -> Dict[str, str]:
    """Returns {expected name: name to read from the file}; raises one error for every problem.
    `ignorable` holds names or shell-style patterns of tensors a file may hold unbound."""
    missing, wrong, resolved = [], [], {}
    for name, spec in sorted(expected.items()):
        source = name if name in present else aliases.get(name)
        if source is None or source not in present:
            missing.append(name)
            continue
        if tuple(present[source]) != tuple(spec.shape):
            wrong.append(f"{name}: file has {list(present[source])}, the model needs {list(spec.shape)}")
        resolved[name] = source
    used = set(resolved.values())
    unexpected = sorted(n for n in present if n not in used and n not in expected and not _ignorable(n, ignorable))
    if missing or wrong or unexpected or problems:
        lines = [f"weights in {where} do not match the model:" if where else "weights do not match the model:"]
        if problems:
            lines.append(f"  shards ({len(problems)}): " + "; ".join(problems))
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))
    return resolved


class Arena:
    """One allocation that holds every weight: `place` hands out aligned offsets, `allocate` makes
    the storage, `view` returns a tensor inside it."""

    def __init__(self, device: torch.device):
        self.device = device
        self.size = 0
        self.offsets: Dict[str, Tuple[int, Tuple[int, ...], torch.dtype]] = {}
        self.storage: Optional[torch.Tensor] = None

    def place(self, key: str, shape: Tuple[int, ...], dtype: torch.dtype, packed: bool = False) -> None:
        """`packed`: directly behind the tensor placed before it (no alignment gap), for tensors
        that are later seen as one matrix."""
        if key in self.offsets:
            return
        if not packed:
            self.size = -(-self.size // ARENA_ALIGN) * ARENA_ALIGN
        self.offsets[key] = (self.size, tuple(shape), dtype)
        self.size += int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()

    def allocate(self) -> None:
        self.storage = torch.empty(max(self.size, 1), dtype=torch.uint8, device=self.device)

    def view(self, key: str) -> torch.Tensor:
        offset, shape, dtype = self.offsets[key]
        n = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
        return self.storage[offset: offset + n].view(dtype).view(shape)


def plan_arena(arena: Arena, kept: Dict[str, Tuple[Tuple[int, ...], torch.dtype]],
               adjacent: Sequence[Sequence[str]]) -> None:
    """Places every tensor of `kept` (name -> (shape, kept dtype)); each group of `adjacent` whose
    members are all present, distinct, of one dtype and one row width goes back to back."""
    grouped = set()
    for group in adjacent:
        members = [n for n in group]
        ok = (len(set(members)) == len(members) and all(n in kept and n not in grouped for n in members)
              and len({kept[n][1] for n in members}) == 1 and len({kept[n][0][1:] for n in members}) == 1)
        if not ok:
            continue
        for i, n in enumerate(members):
            arena.place(n, kept[n][0], kept[n][1], packed=i > 0)
            grouped.add(n)
    for n in sorted(kept):
        arena.place(n, kept[n][0], kept[n][1])


def fused_rows(tensors: Sequence[torch.Tensor]) -> torch.Tensor:
    """[t0; t1; ...] along the rows.  Tensors that lie back to back in one storage (the loader
    places a model's `adjacent` groups so) become one view of it; anything else is concatenated."""
    first = tensors[0]
    same = all(t.dtype == first.dtype and t.device == first.device and t.is_contiguous()
               and t.shape[1:] == first.shape[1:] for t in tensors)
    if same:
        at = first.data_ptr()
        base = first.untyped_storage().data_ptr()
        for t in tensors:
            if t.untyped_storage().data_ptr() != base or t.data_ptr() != at:
                same = False
                break
            at += t.numel() * t.element_size()
    if same:
        rows = sum(t.shape[0] for t in tensors)
        return torch.as_strided(first, (rows, *first.shape[1:]), first.stride(), first.storage_offset())
    widest = torch.float32 if any(t.dtype == torch.float32 for t in tensors) else first.dtype
    return torch.cat([t.to(widest) for t in tensors], dim=0)


class _Staging:
    """Two pinned buffers taken in turn; a buffer is reused only after the copy that read it ran."""

    def __init__(self, device: torch.device, nbytes: int):
        self.device = device
        self.cuda = device.type == "cuda"
        self.buffers = [torch.empty(nbytes, dtype=torch.uint8, pin_memory=self.cuda) for _ in range(2 if self.cuda else 1)]
        self.events: List[Optional[torch.cuda.Event]] = [None] * len(self.buffers)
        self.turn = 0

    def take(self) -> Tuple[torch.Tensor, int]:
        i = self.turn
        self.turn = (self.turn + 1) % len(self.buffers)
        if self.events[i] is not None:
            self.events[i].synchronize()
        return self.buffers[i], i

    def sent(self, i: int) -> None:
        if self.cuda:
            if self.events[i] is None:
                self.events[i] = torch.cuda.Event()
            self.events[i].record()


def _fill_from_file(f, entry, dest: torch.Tensor, staging: _Staging) -> None:
    """Reads one tensor's bytes through the staging buffers into `dest` (a view of the arena),
    converting on the device when the stored type is not the kept one."""
    total = entry.end - entry.begin
    if total == 0:
        return
    same = entry.dtype == dest.dtype
    src_size = torch.empty((), dtype=entry.dtype).element_size()
    dest_flat = dest.reshape(-1)
    dest_bytes = dest_flat.view(torch.uint8) if same else None
    chunk = staging.buffers[0].numel() // 64 * 64
    for begin in range(0, total, chunk):
        n = min(chunk, total - begin)
        buffer, turn = staging.take()
        f.read_into(entry.name, buffer[:n].numpy(), begin)
        if same:
            dest_bytes[begin: begin + n].copy_(buffer[:n], non_blocking=True)
        else:
            piece = buffer[:n].to(dest.device, non_blocking=True).view(entry.dtype)
            dest_flat[begin // src_size: (begin + n) // src_size].copy_(piece)
        staging.sent(turn)


def load_weights(folder, expected: Dict[str, WeightSpec], aliases: Dict[str, str], ignorable,
                 run_dtype: torch.dtype, device: torch.device,
                 adjacent: Sequence[Sequence[str]] = ()) -> Dict[str, torch.Tensor]:
    """Reads every expected tensor into one arena on `device`; a tensor reached through an alias
    shares storage.  `adjacent`: groups of expected names to place back to back."""
    device = torch.device(device)
    with Checkpoint(folder) as ckpt:
        resolved = check_names_and_shapes(expected, ckpt.shapes(), aliases, ignorable, ckpt.where, ckpt.problems)
        kept = {}
        for name, source in resolved.items():
            _f, e = ckpt.entries[source]
            kept[source] = (tuple(e.shape), storage_dtype(e.dtype, run_dtype))
        arena = Arena(device)
        plan_arena(arena, kept, [[resolved[n] for n in group if n in resolved] for group in adjacent])
        arena.allocate()
        staging = _Staging(device, min(STAGING_BYTES, max(64, max((e.end - e.begin for _f, e in ckpt.entries.values()),
                                                                  default=64))))
        for source in kept:
            f, e = ckpt.entries[source]
            _fill_from_file(f, e, arena.view(source), staging)
        if device.type == "cuda":
            torch.cuda.current_stream(device).synchronize()
    return {name: arena.view(source) for name, source in resolved.items()}


def random_weights(expected: Dict[str, WeightSpec], aliases: Dict[str, str], seed: int, run_dtype: torch.dtype,
                   device: torch.device, adjacent: Sequence[Sequence[str]] = (),
                   stored: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """The tensors `load_weights` would return for a folder that `write_random_model` wrote with
    this seed and stored type - generated straight into the arena on `device`, with no file."""
    from .random_init import fill_random

    device = torch.device(device)
    kept = {name: (tuple(spec.shape), storage_dtype(stored, run_dtype)) for name, spec in expected.items()}
    arena = Arena(device)
    plan_arena(arena, kept, adjacent)
    arena.allocate()
    out = {}
    for name, spec in sorted(expected.items()):
        out[name] = arena.view(name)
        fill_random(out[name], spec, seed, name, stored)
    return out
