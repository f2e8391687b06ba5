"""Sampling: parameters, the host sampler and the device sampler."""

from .params import SamplingParams, check_sampling, rng_for  # noqa: F401
from .sampler import host_sample  # noqa: F401
