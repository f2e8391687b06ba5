"""Typed configuration and the architecture registry."""

from .llama import LlamaConfig  # noqa: F401
from .reader import read_config_json  # noqa: F401
from .registry import (Architecture, register_architecture, registered_architectures,  # noqa: F401
                       resolve_architecture)
