"""Pre-norm residual block: h += mixer(norm(h)); h += feed_forward(norm(h))
(src/model.py:113-127 of the reference). Each add is fused with the norm that follows it, so a
branch output travels to the next norm as `pending`."""
from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    def forward(self, h, pending, ctx, unit, owns_cache):
        x = self.mixer_norm.forward(h, pending)
        mixed = self.mixer.forward(x, ctx, unit, owns_cache)
        x = self.feed_forward_norm.forward(h, mixed)
        return h, self.feed_forward.forward(x, ctx)


register_block("pre_norm", PreNormBlock)
