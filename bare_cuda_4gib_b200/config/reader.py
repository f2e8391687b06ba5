"""Reading a model folder's `config.json` into a plain dictionary, before any architecture is
known: the registry picks the typed configuration class from its `architectures` entry."""

from __future__ import annotations

import json
import pathlib
from typing import Any, Dict

from ..errors import ConfigError


def read_config_json(folder) -> Dict[str, Any]:
    path = pathlib.Path(folder) / "config.json"
    try:
        text = path.read_text()
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    try:
        d = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d
