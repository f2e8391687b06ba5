"""Arrangement of a mixer and a feed-forward in one layer.

"prenorm": x += mixer(norm(x)); x += feed_forward(norm(x))
(cuongvng/bare-cuda-4gib engine/src/model.cpp:526-604).  Each add is carried out by the norm
that follows it, so a layer hands its last contribution on, not yet added, as `pending` - unless
the part's last kernel added it into the residual stream itself (`ctx.residual`), in which case the
part returns None.
"""

from __future__ import annotations

from .registry import build_part, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, layer_spec):
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.ffn_norm = build_part("norm", layer_spec.ffn_norm)
        self.ffn = build_part("feed_forward", layer_spec.ffn)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def cache_demands(self):
        """What this layer keeps per request: its mixer's paged cache and state."""
        return [(self.mixer.cache_request(), self.mixer.state_request())]

    def forward(self, ctx, call, residual, pending):
        n = ctx.n_tokens
        ctx.residual = residual      # a part may add its contribution here itself and return None
        after = getattr(ctx, "norm_after_layer", None)
        h = self.mixer_norm.forward(ctx, residual, pending, n, lazy=getattr(self.mixer, "takes_lazy_input", False))
        ctx.following_norm = self.ffn_norm     # the norm that reads the stream after the part that runs now
        mixed = self.mixer.forward(ctx, call, h)
        h = self.ffn_norm.forward(ctx, residual, mixed, n, lazy=getattr(self.ffn, "takes_lazy_input", False))
        ctx.following_norm = after
        out = self.ffn.forward(ctx, h)
        ctx.following_norm = None
        return out

    def entry_norm(self):
        """The norm that reads the residual stream first when this layer runs."""
        return self.mixer_norm
