"""Registries from a part's `kind` to its class, one per family.

Adding a part is: write a class with the family's interface (see `parts.base`), decorate it with
`register_mixer("name")` (or the family's decorator), and name it in a `PartSpec`.  Tests
register toy parts this way without touching the package.
"""

from __future__ import annotations

from typing import Callable, Dict

from ..errors import ConfigError

_FAMILIES: Dict[str, Dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}, "embedding": {}, "head": {},
}


def _register(family: str, kind: str) -> Callable[[type], type]:
    def deco(cls: type) -> type:
        _FAMILIES[family][kind] = cls
        return cls
    return deco


def register_mixer(kind: str): return _register("mixer", kind)
def register_feed_forward(kind: str): return _register("feed_forward", kind)
def register_norm(kind: str): return _register("norm", kind)
def register_position(kind: str): return _register("position", kind)
def register_block(kind: str): return _register("block", kind)
def register_embedding(kind: str): return _register("embedding", kind)
def register_head(kind: str): return _register("head", kind)


def lookup(family: str, kind: str) -> type:
    table = _FAMILIES[family]
    if kind not in table:
        raise ConfigError(f"no {family.replace('_', '-')} part named '{kind}' is registered "
                          f"(registered: {sorted(table)})")
    return table[kind]


def build_part(family: str, spec, **extra):
    """Instantiates the part a `PartSpec` names."""
    return lookup(family, spec.kind)(spec, **extra)
