"""Token embedding and output head.

Embedding: x[t, :] = E[ids[t], :], no scale and no position term
(cuongvng/bare-cuda-4gib engine/kernels/embedding_lookup.cu:22-30), widened into the float32
residual stream.  Head: logits = normed lm_head^T in float32, only for the rows that were asked
for (the reference computes every row: engine/src/model.cpp:612-615).
"""

from __future__ import annotations

import torch

from ..kernels import lib as K
from .base import Part
from .linear import Linear
from .registry import register_embedding, register_head


@register_embedding("table")
class TokenEmbedding(Part):
    """params: `vocab`, `hidden`.  tensors: `weight` [vocab, hidden]."""

    def local_weights(self):
        return {"weight": ((int(self.params["vocab"]), int(self.params["hidden"])), "matrix")}

    def forward(self, ctx) -> torch.Tensor:
        x = ctx.ws.get("residual", (ctx.n_tokens, int(self.params["hidden"])), torch.float32)
        K.embed_gather(self.tensors["weight"], ctx.token_ids, x, ctx.n_tokens, ctx.stream)
        return x


@register_head("linear")
class OutputHead(Part):
    """params: `vocab`, `hidden`.  tensors: `weight` [vocab, hidden] (may be the embedding's)."""

    def local_weights(self):
        return {"weight": ((int(self.params["vocab"]), int(self.params["hidden"])), "matrix")}

    def prepare(self, dtype, device) -> None:
        self.linear = Linear(self.tensors["weight"], "lm_head")
        self.linear.prepare(dtype)

    takes_lazy_input = True

    def forward(self, ctx, normed, rows: int) -> torch.Tensor:
        return self.linear.forward(ctx, normed, rows, torch.float32, "logits").tensor
