"""Causal grouped-query attention over the paged cache.

q = h Wq^T, k = h Wk^T, v = h Wv^T (no bias); q and k rotated by position; k and v appended to
the request's cache pages; scores (q . k) / sqrt(head_dim) over the keys at positions
<= the query's (and, with `window`, newer than position - window); softmax; weighted values;
output projection (cuongvng/bare-cuda-4gib engine/src/model.cpp:540-572,
engine/kernels/attention_qk.cu:49-68, softmax.cu:28-42, attention_av.cu:24-44).
The three projections are one matrix product against [Wq; Wk; Wv], fused at load.

params: `hidden`, `heads`, `kv_heads`, `head_dim`, `window` (None = every key), `position`
(a `PartSpec` of the position family).  tensors: `q`, `k`, `v`, `o`.
"""

from __future__ import annotations

import math

import torch

from ..errors import ConfigError
from ..kernels import lib as K
from .base import KVCacheRequest, Part
from .linear import Linear
from .registry import build_part, register_mixer
from ..weights.loader import fused_rows


@register_mixer("attention")
class Attention(Part):
    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden, self.heads, self.kv_heads, self.head_dim = (
            int(p["hidden"]), int(p["heads"]), int(p["kv_heads"]), int(p["head_dim"]))
        self.window = p.get("window")
        if self.heads % self.kv_heads:
            raise ConfigError(f"attention: {self.heads} heads cannot share {self.kv_heads} key/value heads")
        self.position = build_part("position", p["position"])
        self.scale = 1.0 / math.sqrt(self.head_dim)

    def children(self):
        return [self.position]

    def local_weights(self):
        qd, kvd = self.heads * self.head_dim, self.kv_heads * self.head_dim
        return {"q": ((qd, self.hidden), "matrix"), "k": ((kvd, self.hidden), "matrix"),
                "v": ((kvd, self.hidden), "matrix"), "o": ((self.hidden, qd), "matrix")}

    def adjacent_weights(self):
        return [("q", "k", "v")]

    def cache_request(self):
        return KVCacheRequest(self.kv_heads, self.head_dim, self.window)

    def state_request(self):
        return None

    def prepare(self, dtype, device) -> None:
        t = self.tensors
        self.qkv = Linear(fused_rows([t.pop("q"), t.pop("k"), t.pop("v")]), "qkv")
        self.o = Linear(t.pop("o"), "o")
        self.qkv.prepare(dtype)
        self.o.prepare(dtype)
        self.position.prepare(dtype, device)
        if dtype == torch.bfloat16 and device.type == "cuda":
            from ..kernels import attention as fast
            self.fast = fast.plan_for(self.head_dim, self.heads, self.kv_heads)
        else:
            self.fast = None

    def plan_step(self, ctx) -> None:
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.step_tiles(ctx, self.fast)

    takes_lazy_input = True

    def forward(self, ctx, call, h):
        n = ctx.n_tokens
        qd = self.heads * self.head_dim
        # few rows: float32 partial results let the product split its inner dimension over more SMs
        qkv_dtype = torch.float32 if n <= 256 else ctx.dtype
        q = ctx.ws.get("q", (n, qd), ctx.dtype)
        inv_freq = self.position.fused_rotation()
        apply = getattr(self.position, "apply", None)
        if apply is not None:
            # a position encoding with kernels of its own: it changes q and k in place, as [tokens, heads,
            # head_dim] views of the finished projection, before k and v go into the cache
            qkv = self.qkv.forward(ctx, h, n, ctx.dtype, "qkv")
            kvd = self.kv_heads * self.head_dim
            apply(ctx, qkv.tensor[:, :qd].unflatten(1, (self.heads, self.head_dim)),
                  qkv.tensor[:, qd: qd + kvd].unflatten(1, (self.kv_heads, self.head_dim)))
        else:
            rotate = K.RotateAndCache(q, call.cache, ctx.positions, ctx.row_seq, inv_freq, self.heads, call.writes_cache)
            qkv = self.qkv.forward(ctx, h, n, qkv_dtype, "qkv", allow_partials=True, epilogue=rotate)
        if qkv is not None:
            K.rope_cache_write(qkv, q, call.cache, ctx.positions, ctx.row_seq, inv_freq, self.heads,
                               call.writes_cache, n, ctx.stream)
        out = ctx.ws.get("attn_out", (n, qd), ctx.dtype)
        window = int(self.window) if self.window else 0
        if self.fast is not None and ctx.use_fast_attention:
            from ..kernels import attention as fast
            fast.run(ctx, self.fast, q, out, call.cache, self.scale, window)
        else:
            K.attention_plain(q, out, call.cache, ctx.positions, ctx.row_seq, self.heads, n,
                              self.scale, window, ctx.stream)
        residual = getattr(ctx, "residual", None)
        return self.o.forward(ctx, out, n, torch.float32, "attn_proj", allow_partials=True,
                              epilogue=K.AddTo(residual, getattr(ctx, "following_norm", None)) if residual is not None else None)
