"""Data that describes a model: which parts each layer is made of, with which sizes and
constants, which tensors of the weight file each part binds, and in which order layers run.

A `ModelSpec` is plain data.  An architecture's builder (see `config.registry`) turns its typed
configuration into one; the generic `Model` (see `engine.model`) turns it into parts through the
part registries.  Nothing in the parts knows which model they are in.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """One part: `kind` is its key in the registry of its family (mixer, feed-forward, norm,
    position encoding, block); `params` holds its sizes and constants; `weights` maps the part's
    own tensor names to names in the weight file."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: an arrangement (`block`) of a mixer and a feed-forward with their norms."""

    mixer_norm: PartSpec
    mixer: PartSpec
    ffn_norm: PartSpec
    ffn: PartSpec
    block: str = "prenorm"


@dataclass
class LayerCall:
    """One entry of the run order: run layer `layer`; if `cache_from` is given, this run reads the
    keys and values (or state) that the earlier run with that index wrote and writes none itself."""

    layer: int
    cache_from: Optional[int] = None


@dataclass
class WeightSpec:
    """A tensor a part expects in the weight file."""

    name: str                 # name in the file
    shape: Tuple[int, ...]
    init: str = "matrix"      # random-weights mode: "matrix" ~ N(0, 0.02); "norm" ~ 1 + N(0, 0.01)
    integer: bool = False     # integer tables are kept as int32


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embed: PartSpec
    layers: List[LayerSpec]
    order: List[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    # file tensor -> file tensor to use in its place when the first is absent (tied embeddings)
    aliases: Dict[str, str] = field(default_factory=dict)
    # tensors that may be present in the file without being bound
    ignorable: Tuple[str, ...] = ()
