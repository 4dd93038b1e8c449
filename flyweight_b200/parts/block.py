"""The pre-norm residual arrangement: x += mixer(norm(x)); x += ffn(norm(x))
(native/src/v2_runtime.cpp:4164-4175).  A residual sum is folded either into the product that
makes the delta (a part with ``adds_residual`` adds into x in its last epilogue) or into the
norm that follows (the delta is handed on as ``pending``); a norm whose input needs no sum is
handed to its consumer unapplied when that consumer can fold it into its first product."""
from __future__ import annotations

from .base import Arrangement, register_arrangement


def _normed(norm, consumer, ctx, x, pending):
    if pending is None and consumer.takes_deferred_norm:
        deferred = norm.defer(ctx, x)
        if deferred is not None:
            return deferred
    return norm.forward(ctx, x, delta=pending)


@register_arrangement("prenorm_residual")
class PreNormResidual(Arrangement):
    def forward(self, ctx, x, pending, cache):
        mixer, ffn = self.mixer, self.feed_forward
        h = _normed(self.mixer_norm, mixer, ctx, x, pending)
        delta = mixer.forward(ctx, h, cache, residual=x) if mixer.adds_residual else mixer.forward(ctx, h, cache)
        h = _normed(self.ffn_norm, ffn, ctx, x, delta)
        return x, (ffn.forward(ctx, h, residual=x) if ffn.adds_residual else ffn.forward(ctx, h))

    def plan(self, builder, cache):
        """This block's operations for the native step plan: the mixer behind its norm, the
        feed-forward behind its norm; the residual sums ride on the products."""
        from ..engine.plan import NotPlannable
        for part in (self.mixer, self.feed_forward):
            if getattr(part, "plan", None) is None:
                raise NotPlannable(f"part {part.kind!r} has no native form")
        self.mixer.plan(builder, self.mixer_norm, cache)
        self.feed_forward.plan(builder, self.ffn_norm)
