"""Weights: the safetensors container, binding by tensor name, and the random-weights mode."""

from .checkpoint import Checkpoint  # noqa: F401
from .loader import check_names_and_shapes, fused_rows, load_weights, random_weights, storage_dtype  # noqa: F401
from .random_init import random_tensors, write_random_model  # noqa: F401
from .safetensors_io import SafetensorsFile, write_safetensors  # noqa: F401
