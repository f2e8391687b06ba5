"""Dense SwiGLU feed-forward: down(silu(gate(h)) * up(h)), no biases, silu(g) = g / (1 + exp(-g))
(cuongvng/bare-cuda-4gib engine/src/model.cpp:589-598, engine/kernels/swiglu.cu:22-23).
gate and up are one matrix product against [Wgate; Wup], fused at load; where the fast kernel
runs, silu(gate) * up is its epilogue.

params: `hidden`, `intermediate`.  tensors: `gate`, `up`, `down`.
"""

from __future__ import annotations

import torch

from ..kernels import lib as K
from .base import Part
from .linear import Linear
from .registry import register_feed_forward
from ..weights.loader import fused_rows


@register_feed_forward("swiglu")
class SwiGLUFeedForward(Part):
    def local_weights(self):
        h, i = int(self.params["hidden"]), int(self.params["intermediate"])
        return {"gate": ((i, h), "matrix"), "up": ((i, h), "matrix"), "down": ((h, i), "matrix")}

    def adjacent_weights(self):
        return [("gate", "up")]

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.gate_up = Linear(fused_rows([t.pop("gate"), t.pop("up")]), "gate_up")
        self.down = Linear(t.pop("down"), "down")
        self.gate_up.prepare(dtype)
        self.down.prepare(dtype)

    takes_lazy_input = True

    def forward(self, ctx, h):
        n = ctx.n_tokens
        act = self.gate_up.forward(ctx, h, n, ctx.dtype, "ffn_act", swiglu=True)
        residual = getattr(ctx, "residual", None)
        return self.down.forward(ctx, act.tensor, n, torch.float32, "ffn_out", allow_partials=True,
                                 epilogue=K.AddTo(residual, getattr(ctx, "following_norm", None)) if residual is not None else None)
