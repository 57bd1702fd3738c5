"""Block arrangements.  ``prenorm``: x += mixer(norm(x)); x += ffn(norm(x))
(src/llm/model.c:743-796)."""
from __future__ import annotations

from .base import Block
from .registry import register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, ctx, x, pending, cache):
        # the add of what the previous part produced is fused into the norm
        h = self.mixer_norm.apply(x, ctx.dtype, delta=pending)
        d = self.mixer.forward(ctx, h, cache)
        h = self.ffn_norm.apply(x, ctx.dtype, delta=d)
        return x, self.feed_forward.forward(ctx, h)
