"""A small, whole inference engine for the Llama dense decoder on one NVIDIA B200 (sm_100a)."""

__version__ = "0.1.0"
