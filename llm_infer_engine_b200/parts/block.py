"""Pre-norm residual block: h += mixer(norm(h)); h += feed_forward(norm(h))
(src/model.py:113-127 of the reference). Each add is fused with the norm that follows it, so a
branch output travels to the next norm as `pending`."""
from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    """A part that sets `adds_to_residual = True` accepts `residual=h` and may add its output into
    h itself (in float32, inside its last kernel); it then returns None instead of a branch output.
    A part that sets `accepts_deferred_norm = True` may be handed a `DeferredNorm` instead of the
    normalised tensor and folds the norm into its first kernel."""

    def forward(self, h, pending, ctx, unit, owns_cache):
        x = None
        if pending is None and getattr(self.mixer, "accepts_deferred_norm", False):
            x = self.mixer_norm.defer(h)              # the mixer's first kernel applies the norm
        if x is None:
            x = self.mixer_norm.forward(h, pending)
        if getattr(self.mixer, "adds_to_residual", False):
            mixed = self.mixer.forward(x, ctx, unit, owns_cache, residual=h)
        else:
            mixed = self.mixer.forward(x, ctx, unit, owns_cache)
        x = None
        if mixed is None and getattr(self.feed_forward, "accepts_deferred_norm", False):
            x = self.feed_forward_norm.defer(h)
        if x is None:
            x = self.feed_forward_norm.forward(h, mixed)
        if getattr(self.feed_forward, "adds_to_residual", False):
            return h, self.feed_forward.forward(x, ctx, residual=h)
        return h, self.feed_forward.forward(x, ctx)

    def stack_view(self):
        views = {role: part.stack_view() for role, part in self.parts().items()}
        if any(v is None for v in views.values()):
            return None
        return dict(kind="pre_norm", **views)


register_block("pre_norm", PreNormBlock)
