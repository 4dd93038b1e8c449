"""Dense SwiGLU feed-forward: down( silu(gate h) * (up h) ), no bias
(native/src/v2_runtime.cpp:28797-28805; silu with a sign-split sigmoid,
native/include/flyweight_v2_qwen_kernels.hpp:1217-1222)."""
from __future__ import annotations

import torch

from ..kernels import ops, tensorcore
from ..weights.loader import TensorDecl
from .base import FeedForward, Precision, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: hidden_size, ffn_dim.  tensors: gate [F][H], up [F][H], down [H][F]."""
    graph_safe = True
    takes_deferred_norm = True
    adds_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.ffn_dim = int(self.params["ffn_dim"])
        self.w_gate_up = self.w_down = None

    def declare(self):
        n, H, F = self.names, self.hidden, self.ffn_dim
        return {n["gate"]: TensorDecl((F, H)), n["up"]: TensorDecl((F, H)),
                n["down"]: TensorDecl((H, F))}

    def bind(self, get, precision: Precision, device):
        n = self.names
        gate, up = get(n["gate"]), get(n["up"])
        if gate.dtype != up.dtype:
            gate, up = gate.to(torch.float32), up.to(torch.float32)
        # gate and up as one projection: gate rows first, then up rows
        self.w_gate_up = precision.matrix(torch.cat([gate, up], dim=0), device)
        self.w_down = precision.matrix(get(n["down"]), device)

    def weight_bytes(self):
        return (self.w_gate_up.numel() * self.w_gate_up.element_size()
                + self.w_down.numel() * self.w_down.element_size())

    def flops_per_token(self):
        return 2.0 * (self.w_gate_up.numel() + self.w_down.numel())

    def forward(self, ctx, h, residual=None):
        act = ctx.precision.act_dtype
        if not isinstance(h, torch.Tensor):                   # a norm not yet applied
            if h.kind == "rmsnorm" and tensorcore.normed_accepts(h.n_rows, self.hidden, self.w_gate_up, 2,
                                                                  self.ffn_dim):
                # the norm, both products and silu(g)*u in one kernel
                a = tensorcore.swiglu_gate_up_normed(h.x, h.weight, h.eps, self.w_gate_up)
                return ops.linear_into_residual(a, self.w_down, residual)
            h = h.materialize(act)
        if tensorcore.swiglu_accepts(h, self.w_gate_up):
            # gate and up accumulate side by side in tensor memory; silu(g)*u is the epilogue
            a = tensorcore.swiglu_gate_up(h, self.w_gate_up)
        else:
            gate_up = ops.linear(h, self.w_gate_up, act)
            a = ops.silu_mul(gate_up, act)
        return ops.linear_into_residual(a, self.w_down, residual)

    def plan(self, builder, norm):
        """Norm, gate|up with silu(g)*u, down with the residual sum, for the native step plan."""
        from ..engine.plan import EPI_SWIGLU
        a = builder.tokens(self.ffn_dim, builder.act_dtype)
        builder.norm_linear(norm, self.w_gate_up, EPI_SWIGLU, a, "gate|up")
        builder.linear_residual(a, self.w_down, "down")
        builder.free(a)
