"""Interfaces of the part families, and what a step hands to them.

Families and the one method each must have besides `weight_specs` / `bind`:

* norm          `forward(ctx, residual, delta, rows, row_index=None, buffer=..., lazy=False) -> activations`
                adds `delta` (a `Partials`, or None) into the float32 residual stream, then
                normalises; returns [rows, hidden] in the step's activation type.  With `lazy`
                it may return a `LazyNorm` (see kernels.lib) instead, which the consumer either
                hands to a `Linear` or turns into a matrix with `materialize()`; the block asks
                for that only of consumers that declare `takes_lazy_input = True`.
* position      `fused_rotation()` -> float32 inverse frequencies [head_dim / 2] that the attention
                kernels apply themselves (rotate_half pairing), or None; a part that also defines
                `apply(ctx, q, k)` gets q [tokens, heads, head_dim] and k [tokens, kv_heads,
                head_dim] as views of the finished projection and changes them in place (row t is
                at position `ctx.positions[t]`) before k and v are written to the cache.
* mixer         `forward(ctx, call, h) -> Partials` (the mixer's contribution to the residual), or
                None if it has added the contribution into `ctx.residual` itself;
                `cache_request()` -> `KVCacheRequest` or None; `state_request()` ->
                `StateRequest` or None.  The cache manager serves both.
* feed_forward  `forward(ctx, h) -> Partials`, or None as for a mixer
* block         `forward(ctx, call, residual, pending) -> Partials`: runs one layer; `pending` is
                the previous layer's contribution that has not been added to the residual yet.
                `parts()` lists its parts; `cache_demands()` -> [(KVCacheRequest or None,
                StateRequest or None), ...], one pair per part that keeps something per request
                (`call.caches[j]` / `call.states[j]` belong to pair j).
* embedding     `forward(ctx) -> residual [tokens, hidden] float32`
* head          `forward(ctx, normed) -> logits [rows, vocab] float32`

A part gets its sizes and constants from `spec.params` only.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .spec import PartSpec, WeightSpec


@dataclass(frozen=True)
class KVCacheRequest:
    """Keys and values per token that a mixer wants paged: `window` None keeps every key, a
    number keeps the last `window` positions (older pages are given back)."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """Per-request state of fixed size: one tensor of `shape` and `dtype` per request slot,
    zeroed when a request takes the slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Common ground of all parts: the spec, expected tensors, binding of loaded tensors."""

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params = spec.params
        self.tensors: Dict[str, torch.Tensor] = {}

    # local tensor name -> (shape, init kind); subclasses fill this in
    def local_weights(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {}

    def weight_specs(self) -> Dict[str, WeightSpec]:
        out = {}
        for local, (shape, init) in self.local_weights().items():
            if local not in self.spec.weights:
                raise KeyError(f"part '{self.spec.kind}' needs a file name for its tensor '{local}'")
            out[local] = WeightSpec(self.spec.weights[local], tuple(shape), init)
        return out

    def adjacent_weights(self) -> List[Tuple[str, ...]]:
        """Groups of local tensor names that this part multiplies as one matrix, rows stacked in
        this order: the loader places such tensors back to back, so that `weights.fused_rows` of
        them is a view and not a copy."""
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        """Receives the loaded tensors by local name; `dtype` is the step's activation type."""
        self.tensors = dict(tensors)

    def children(self) -> List["Part"]:
        return []

    def prepare(self, dtype: torch.dtype, device: torch.device) -> None:
        """Called once after binding, on the device: fuse tensors, build tables, compile kernels."""

    # A part that must look at the batch on the host before its kernels run (to build work lists
    # and upload them) defines `plan_step(ctx)`; it is called once per step before `forward`, and
    # is NOT part of a captured CUDA graph, while `forward` may be.


class CallContext:
    """One run of a layer inside a step: its index in the run order, the caches it reads (and
    whether it also writes them) and its per-request states, one of each per demand the block
    stated (`None` where a demand asked for none).  `cache` and `state` are the first ones: all a
    block with a single mixer needs."""

    __slots__ = ("index", "caches", "writes_cache", "states")

    def __init__(self, index, caches, writes_cache, states):
        if not isinstance(caches, (list, tuple)):
            caches, states = [caches], [states]
        self.index, self.caches, self.writes_cache, self.states = index, list(caches), writes_cache, list(states)

    @property
    def cache(self):
        return self.caches[0] if self.caches else None

    @property
    def state(self):
        return self.states[0] if self.states else None
