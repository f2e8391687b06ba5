"""RMSNorm, fused with the residual add that precedes it.

out = x * rsqrt(mean(x^2) + eps) * w with eps inside the root, on the mean, and the weight
multiplied last (cuongvng/bare-cuda-4gib engine/kernels/rmsnorm.cu:26-40).  The reference adds
the residual in a kernel of its own (engine/kernels/residual_add.cu:20); here the add of the
previous part's contribution and the norm are one kernel, and the residual stream stays float32.

params: `size` (width), `eps`.  tensors: `weight` [size].
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import lib as K
from .base import Part
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    prenormable = True      # the norm's factor is one number per row (see kernels.lib.AddTo)

    def local_weights(self):
        return {"weight": ((self.params["size"],), "norm")}

    def forward(self, ctx, residual: torch.Tensor, delta: Optional[K.Partials], rows: int,
                row_index: Optional[torch.Tensor] = None, buffer: str = "normed", lazy: bool = False):
        """With `lazy` (the consumer takes a `LazyNorm`) and nothing to add, a few-token bfloat16
        step gets the norm as a description that the consuming product computes in its own kernel."""
        left = getattr(ctx, "prenormed", None)       # what the last adding product may have left for this norm
        ctx.prenormed = None
        if lazy and delta is None and ctx.dtype == torch.bfloat16 and ctx.use_fast_gemm:
            from ..kernels import gemv
            mine = left if left is not None and left.norm is self else None
            # a few-token step norms inside the consuming product; a many-token step only where the
            # product before this norm has prepared it
            if (gemv.takes(rows, int(self.params["size"])) or mine is not None) and self.tensors["weight"].is_cuda:
                return K.LazyNorm(ctx, residual, self.tensors["weight"], float(self.params["eps"]), rows,
                                  row_index, buffer, mine)
        out = ctx.ws.get(buffer, (rows, self.params["size"]), ctx.dtype)
        K.add_rmsnorm(residual, delta, self.tensors["weight"], out, float(self.params["eps"]), rows,
                      row_index, ctx.stream)
        return out
