"""The pre-norm residual arrangement: x += mixer(norm(x)); x += ffn(norm(x))
(native/src/v2_runtime.cpp:4164-4175).  Every residual sum is folded into the norm that
follows it, so the delta a block's feed-forward produces is handed on as ``pending``."""
from __future__ import annotations

from .base import Arrangement, register_arrangement


@register_arrangement("prenorm_residual")
class PreNormResidual(Arrangement):
    def forward(self, ctx, x, pending, cache):
        h = self.mixer_norm.forward(ctx, x, delta=pending)
        delta = self.mixer.forward(ctx, h, cache)
        h = self.ffn_norm.forward(ctx, x, delta=delta)
        return x, self.feed_forward.forward(ctx, h)
