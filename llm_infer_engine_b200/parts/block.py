"""Pre-norm residual block: h += mixer(norm(h)); h += feed_forward(norm(h))
(src/model.py:113-127 of the reference). Each add is fused with the norm that follows it, so a
branch output travels to the next norm as `pending`."""
from __future__ import annotations

from ..kernels import trace
from .base import Block, call_branch, register_block


class PreNormBlock(Block):
    """Roles: mixer, feed_forward and a norm in front of each. A branch whose part declares
    `accepts_deferred_norm` gets the norm as a promise and folds it into its first kernel; one that declares
    `adds_to_residual` gets the residual stream and may add its output there itself (parts/base.py)."""
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}

    def forward(self, h, pending, ctx, unit, owns_cache):
        tracing = trace.active()
        if tracing:
            trace.push(f"Attn_{ctx.entry}")           # the reference's range names (src/model.py:112,126)
        x = None
        if pending is None and self.mixer.accepts_deferred_norm:
            x = self.mixer_norm.defer(h)              # the mixer's first kernel applies the norm
        if x is None:
            x = self.mixer_norm.forward(h, pending)
        mixed = call_branch(self.mixer, x, ctx, unit, owns_cache, residual=h)
        if tracing:
            trace.pop()
            trace.push(f"FFN_{ctx.entry}")
        x = None
        if mixed is None and self.feed_forward.accepts_deferred_norm:
            x = self.feed_forward_norm.defer(h)
        if x is None:
            x = self.feed_forward_norm.forward(h, mixed)
        out = call_branch(self.feed_forward, x, ctx, residual=h)
        if tracing:
            trace.pop()
        return h, out


register_block("pre_norm", PreNormBlock)
