"""Rotary position encoding with the rotate_half pairing (element p with p + head_dim / 2).

inv_freq[p] = 1 / theta^(2p / head_dim); the angle of position pos is the float32 product
float(pos) * inv_freq[p]; lo' = lo cos - hi sin, hi' = hi cos + lo sin
(cuongvng/bare-cuda-4gib engine/kernels/rope.cu:44-53; tools/references/reference_forward.py:89-104).
The frequencies are computed once on the host in float32 and kept on the device; the attention
kernels rotate q and k with them while they write the cache, so this part launches nothing.

params: `head_dim`, `theta`.  No tensors.
"""

from __future__ import annotations

import torch

from .base import Part
from .registry import register_position


@register_position("rope")
class RotaryPositions(Part):
    def prepare(self, dtype, device) -> None:
        d, theta = int(self.params["head_dim"]), float(self.params["theta"])
        exponent = torch.arange(d // 2, dtype=torch.float32) * 2.0 / d
        self.inv_freq = (1.0 / (theta ** exponent)).to(device)

    def fused_rotation(self):
        """Inverse frequencies for kernels that rotate q and k themselves."""
        return self.inv_freq


@register_position("none")
class NoPositions(Part):
    """No position information inside the mixer (keys and queries are used as projected)."""

    def fused_rotation(self):
        return None
