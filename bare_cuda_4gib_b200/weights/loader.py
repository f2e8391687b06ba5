"""Binds the tensors of a model folder to the parts of a model, by tensor name.

Element types: in a bfloat16 run 16-bit floating tensors are kept in bfloat16 and a tensor stored
in 32-bit stays 32-bit; in a float32 run every floating tensor is widened to float32 (exact).
Integer tensors are kept as int32.  All problems of a file are reported in ONE `WeightError`
that lists missing tensors, unexpected tensors and wrong shapes (the reference stops at the
first: engine/src/model.cpp:24-32, engine/src/loader.cpp:142-148).
"""

from __future__ import annotations

import pathlib
from typing import Dict, Tuple

import torch

from ..errors import WeightError
from ..parts.spec import WeightSpec
from .safetensors_io import SafetensorsFile

WEIGHT_FILE = "model.safetensors"


def storage_dtype(stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32 or stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_names_and_shapes(expected: Dict[str, WeightSpec], present: Dict[str, Tuple[int, ...]],
                           aliases: Dict[str, str], ignorable=(), where: str = "") -> Dict[str, str]:
    """Returns {expected name: name to read from the file}; raises one error for every problem."""
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
    unexpected = sorted(n for n in present if n not in used and n not in expected and n not in ignorable)
    if missing or wrong or unexpected:
        lines = [f"weights in {where} do not match the model:" if where else "weights do not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))
    return resolved


def load_weights(folder, expected: Dict[str, WeightSpec], aliases: Dict[str, str], ignorable,
                 run_dtype: torch.dtype, device: torch.device) -> Dict[str, torch.Tensor]:
    """Reads every expected tensor onto `device`; a tensor reached through an alias shares storage."""
    path = pathlib.Path(folder) / WEIGHT_FILE
    with SafetensorsFile(path) as f:
        present = {n: e.shape for n, e in f.entries.items()}
        resolved = check_names_and_shapes(expected, present, aliases, ignorable, str(path))
        by_source: Dict[str, torch.Tensor] = {}
        out: Dict[str, torch.Tensor] = {}
        for name, source in resolved.items():
            if source not in by_source:
                t = f.tensor(source)
                by_source[source] = t.to(device=device, dtype=storage_dtype(t.dtype, run_dtype))
            out[name] = by_source[source]
    return out
