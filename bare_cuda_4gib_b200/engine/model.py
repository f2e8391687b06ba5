"""The generic model: parts built from a `ModelSpec`, weights bound by name, one `forward` that
runs the tokens of a step.

The layer graph is the reference's (cuongvng/bare-cuda-4gib engine/src/model.cpp:522-615):
embedding, the layers in run order, final norm and head - except that the head runs only on
the rows whose logits are wanted.  Nothing here is specific to one architecture: the spec says
which parts to build and in which order layers run.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.manager import CacheDemand
from ..config.reader import read_config_json
from ..config.registry import resolve_architecture
from ..errors import ConfigError
from ..parts.base import Part
from ..parts.registry import build_part, lookup
from ..parts.spec import ModelSpec, WeightSpec
from ..weights.loader import load_weights, random_weights

RUN_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def run_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"dtype {name} is not supported (float32 or bfloat16)")
        return name
    if name not in RUN_DTYPES:
        raise ConfigError(f"dtype '{name}' is not supported (float32 or bfloat16)")
    return RUN_DTYPES[name]


def _walk(part) -> List[Part]:
    out = [part]
    for child in part.children():
        out.extend(_walk(child))
    return out


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embed = build_part("embedding", spec.embed)
        self.blocks = [lookup("block", layer.block)(layer) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        self.order = list(spec.order)
        for i, call in enumerate(self.order):
            if not (0 <= call.layer < len(self.blocks)):
                raise ConfigError(f"run order entry {i} names layer {call.layer}; the model has {len(self.blocks)}")
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        self._planners = [p for p in self.all_parts() if hasattr(p, "plan_step")]
        # a part whose forward does host-dependent work sets `graph_safe = False`; steps of such a
        # model are never captured as CUDA graphs
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in self.all_parts())

    # ------------------------------------------------------------------ structure
    def all_parts(self) -> List[Part]:
        parts: List[Part] = _walk(self.embed)
        for block in self.blocks:
            for p in block.parts():
                parts.extend(_walk(p))
        parts.extend(_walk(self.final_norm))
        parts.extend(_walk(self.head))
        return parts

    def cache_demands(self) -> List[List[CacheDemand]]:
        """Per entry of the run order, what its block keeps per request (the block says; a block
        with one mixer states one demand)."""
        return [[CacheDemand(kv, state, call.cache_from) for kv, state in self.blocks[call.layer].cache_demands()]
                for call in self.order]

    # ------------------------------------------------------------------ weights
    def adjacent_weights(self) -> List[List[str]]:
        """File names of tensors that some part multiplies as one matrix, in stacking order."""
        out = []
        for part in self.all_parts():
            specs = part.weight_specs()
            for group in part.adjacent_weights():
                if all(local in specs for local in group):
                    out.append([specs[local].name for local in group])
        return out

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """`tensors` by file name (see `expected_weights`)."""
        self.dtype, self.device = dtype, torch.device(device)
        for part in self.all_parts():
            specs = part.weight_specs()
            part.bind({local: tensors[ws.name] for local, ws in specs.items()}, dtype)
        for part in self.all_parts():
            part.prepare(dtype, self.device)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for obj in self._weight_tensors():
            key = obj.data_ptr()
            if key not in seen:
                seen.add(key)
                total += obj.numel() * obj.element_size()
        return total

    def _weight_tensors(self):
        from ..parts.linear import Linear
        for part in self.all_parts():
            for t in part.tensors.values():
                yield t
            for v in vars(part).values():
                if isinstance(v, Linear):
                    yield v.weight

    # ------------------------------------------------------------------ one step
    def plan_step(self, ctx) -> None:
        """Host-side planning of the parts that need it (never captured in a CUDA graph)."""
        for part in self._planners:
            part.plan_step(ctx)

    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs ctx's tokens; returns float32 logits [wanted rows, vocab] (None if none is wanted)."""
        x = self.embed.forward(ctx)
        pending = None
        for i, call in enumerate(self.order):
            # the norm that reads the residual stream after this layer: the next layer's first, or the final one
            if i + 1 < len(self.order):
                entry = getattr(self.blocks[self.order[i + 1].layer], "entry_norm", None)
                ctx.norm_after_layer = entry() if entry else None
            else:
                ctx.norm_after_layer = self.final_norm if ctx.n_want > 0 else None
            pending = self.blocks[call.layer].forward(ctx, ctx.calls[i], x, pending)
        ctx.norm_after_layer = None
        if ctx.n_want == 0:
            return None
        normed = self.final_norm.forward(ctx, x, pending, ctx.n_want, ctx.want_rows, buffer="final_normed",
                                         lazy=getattr(self.head, "takes_lazy_input", False))
        return self.head.forward(ctx, normed, ctx.n_want)


def expected_weights(spec: ModelSpec) -> Tuple[Dict[str, WeightSpec], Model]:
    """Every tensor the model's parts bind, by file name (a name bound twice must agree in shape)."""
    model = Model(spec)
    expected: Dict[str, WeightSpec] = {}
    for part in model.all_parts():
        for ws in part.weight_specs().values():
            if ws.name in expected and expected[ws.name].shape != ws.shape:
                raise ConfigError(f"tensor '{ws.name}' is bound with shapes {expected[ws.name].shape} and {ws.shape}")
            expected.setdefault(ws.name, ws)
    return expected, model


def load_model(folder, dtype="bfloat16", device="cuda") -> Tuple[Model, object]:
    """Reads config.json, picks the architecture from the registry, builds and binds the model."""
    from .. import models  # noqa: F401  (registers the architectures)

    cfg_dict = read_config_json(folder)
    arch = resolve_architecture(cfg_dict)
    config = arch.config_class.from_dict(cfg_dict)
    return load_model_with_spec(folder, arch.build_spec(config), dtype, device), config


def load_model_with_spec(folder, spec: ModelSpec, dtype="bfloat16", device="cuda") -> Model:
    """Builds the model a spec describes and binds the folder's tensors to it (the spec need not come
    from a registered architecture)."""
    expected, model = expected_weights(spec)
    dt = run_dtype(dtype)
    tensors = load_weights(folder, expected, spec.aliases, spec.ignorable, dt, torch.device(device),
                           model.adjacent_weights())
    model.bind(tensors, dt, device)
    return model


def random_model(config, seed: int, dtype="bfloat16", device="cuda", stored: torch.dtype = torch.bfloat16) -> Model:
    """The model `load_model` would return for the folder that `write_random_model(folder, config,
    seed)` writes, with the weights generated straight on the device and no file in between."""
    from .. import models  # noqa: F401  (registers the architectures)

    arch = resolve_architecture(config.to_dict())
    spec = arch.build_spec(config)
    expected, model = expected_weights(spec)
    dt = run_dtype(dtype)
    tensors = random_weights(expected, spec.aliases, seed, dt, torch.device(device), model.adjacent_weights(), stored)
    model.bind(tensors, dt, device)
    return model
