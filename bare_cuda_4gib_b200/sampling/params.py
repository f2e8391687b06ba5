"""Sampling parameters with the names, defaults and meanings of cuongvng/bare-cuda-4gib
(engine/include/llm/sampler.h:9-16; validation engine/src/sampler.cpp:20-27)."""

from __future__ import annotations

import math
import os
import random
from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 0.0   # 0 is greedy
    top_p: float = 1.0         # keep the fewest likeliest tokens whose probability reaches top_p
    top_k: int = 0             # keep the k likeliest tokens; 0 keeps all
    seed: int = -1             # -1 draws a random seed

    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    def filtered(self) -> bool:
        """True if top-k or top-p cuts the distribution (such rows are drawn on the host)."""
        return self.top_k > 0 or self.top_p < 1.0


def check_sampling(p: SamplingParams) -> str:
    """Empty if the parameters are valid, else why not."""
    if not (isinstance(p.temperature, (int, float)) and p.temperature >= 0.0 and math.isfinite(p.temperature)):
        return "temperature must be a finite number >= 0"
    if not (0.0 < p.top_p <= 1.0):
        return "top_p must be in (0, 1]"
    if p.top_k < 0:
        return "top_k must be >= 0"
    return ""


def rng_for(p: SamplingParams) -> random.Random:
    """One generator per request, so a seed gives the same tokens alone or in a batch
    (engine/include/llm/scheduler.h:103, engine/src/sampler.cpp:29-33)."""
    seed = p.seed if p.seed >= 0 else int.from_bytes(os.urandom(8), "little")
    return random.Random(seed)
