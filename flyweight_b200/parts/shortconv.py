"""Gated short-convolution mixer.

in_proj to 3H split B | C | x (native/include/flyweight_v2_native_kernels.hpp:1295-1299);
u = B*x; causal depthwise FIR of L taps, oldest first, over u with the request's rolling
state standing for the positions before this step (:1301-1345); optional bias after the
taps; z = C*y; out_proj.  The state, [H][L-1] fp32 per request, lives in a slot that the
cache manager owns (native/src/v2_runtime.cpp:3501-3505 for its size).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import FixedState, Mixer, Precision, register_mixer


@register_mixer("gated_short_conv")
class GatedShortConv(Mixer):
    """params: hidden_size, taps (L >= 2), bias (bool).
    tensors: in_proj [3H][H], taps [H][L] (also stored as [H][1][L]), out_proj [H][H], bias [H]."""
    graph_safe = True
    takes_deferred_norm = True
    adds_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.taps_len = int(self.params["taps"])
        self.has_bias = bool(self.params.get("bias", False))
        if self.taps_len < 2:
            raise ValueError("a short convolution needs at least 2 taps")
        self.w_in = self.w_out = self.taps = self.bias = None

    def declare(self):
        n, H, L = self.names, self.hidden, self.taps_len
        out = {n["in_proj"]: TensorDecl((3 * H, H)),
               n["taps"]: TensorDecl((H, L), "taps", also=((H, 1, L),)),
               n["out_proj"]: TensorDecl((H, H))}
        if self.has_bias:
            out[n["bias"]] = TensorDecl((H,), "bias")
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        self.w_in = precision.matrix(get(n["in_proj"]), device)
        self.w_out = precision.matrix(get(n["out_proj"]), device)
        self.taps = precision.vector(get(n["taps"]).reshape(self.hidden, self.taps_len), device)
        self.bias = precision.vector(get(n["bias"]), device) if self.has_bias else None

    def weight_bytes(self):
        return (self.w_in.numel() * self.w_in.element_size()
                + self.w_out.numel() * self.w_out.element_size() + self.taps.numel() * 4)

    def flops_per_token(self):
        return 2.0 * (self.w_in.numel() + self.w_out.numel() + self.taps.numel())

    def state_spec(self):
        return FixedState((self.hidden, self.taps_len - 1))

    def forward(self, ctx, h, cache, residual=None):
        batch = ctx.batch
        # B|C|x in the activation dtype: the conv kernel widens them and multiplies in fp32
        p = ops.linear(h, self.w_in, ctx.precision.act_dtype)
        z = ops.shortconv(p, self.taps, self.bias, cache.state, batch.seg_start, batch.seg_slot,
                          batch.tok_seg, batch.n_segments, ctx.precision.act_dtype)
        return ops.linear_into_residual(z, self.w_out, residual)

    def plan(self, builder, norm, cache):
        """The same three operations for the native step plan (``engine/plan.py``)."""
        from ..engine.plan import EPI_ACT
        act = builder.act_dtype
        p = builder.tokens(3 * self.hidden, act)
        builder.norm_linear(norm, self.w_in, EPI_ACT, p, "conv in_proj")
        z = builder.tokens(self.hidden, act)
        builder.shortconv(p, self.taps, self.bias, cache.state, z)
        builder.free(p)
        builder.linear_residual(z, self.w_out, "conv out_proj")
        builder.free(z)
