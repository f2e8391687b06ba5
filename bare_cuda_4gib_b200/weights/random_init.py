"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Matrices and tables ~ N(0, 0.02), norm weights ~ 1 + N(0, 0.01).  Every tensor has a generator
of its own, seeded from the seed and the tensor's name, so a tensor's values do not depend on
which other tensors exist.  (cuongvng/bare-cuda-4gib has random weights only in its torch
fixture: tools/references/reference_forward.py:301-321.)
"""

from __future__ import annotations

import hashlib
import json
import pathlib
from typing import Dict

import torch

from ..parts.spec import WeightSpec
from .checkpoint import WEIGHT_FILE
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.01


def _generator(seed: int, name: str, device) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensor(spec: WeightSpec, seed: int, name: str, dtype: torch.dtype, device) -> torch.Tensor:
    g = _generator(seed, name, device)
    x = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
    x = 1.0 + NORM_STD * x if spec.init == "norm" else MATRIX_STD * x
    return x.to(dtype)


def random_tensors(expected: Dict[str, WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu") -> Dict[str, torch.Tensor]:
    return {name: random_tensor(spec, seed, name, dtype, device) for name, spec in sorted(expected.items())}


def fill_random(dest: torch.Tensor, spec: WeightSpec, seed: int, name: str, stored: torch.dtype) -> None:
    """Writes into `dest` what a folder written with this seed and stored type would load as
    (generated on dest's device, rounded to the stored type first)."""
    dest.copy_(random_tensor(spec, seed, name, stored, dest.device))


def write_random_model(folder, config, seed: int, dtype: torch.dtype = torch.bfloat16, device="cpu") -> pathlib.Path:
    """`config` is a typed configuration of a registered architecture (it has `to_dict`)."""
    from ..config.registry import resolve_architecture
    from ..engine.model import expected_weights

    folder = pathlib.Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg_dict = config.to_dict()
    cfg_dict["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    arch = resolve_architecture(cfg_dict)
    spec = arch.build_spec(config)
    expected, _ = expected_weights(spec)
    tensors = random_tensors(expected, seed, dtype, device)
    write_safetensors(folder / WEIGHT_FILE, tensors)
    (folder / "config.json").write_text(json.dumps(cfg_dict, indent=2) + "\n")
    return folder
