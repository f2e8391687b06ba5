"""Architectures.  Importing this package registers them."""

from . import llama  # noqa: F401
