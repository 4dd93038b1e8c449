"""RMSNorm with a plain (not 1+w) weight, computed in fp32.

``(x * rsqrt(mean(x^2) + eps)) * w`` -- native/include/flyweight_v2_qwen_kernels.hpp:424-447,
called with one_centered=0 (native/src/v2_runtime.cpp:27741).  The residual sum that
precedes a norm in a block is folded into the same kernel.
"""
from __future__ import annotations

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import DeferredNorm, Norm, Precision, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: size, eps.  tensors: weight [size]."""
    graph_safe = True


    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])
        self.eps = float(self.params["eps"])
        self.weight = None

    def declare(self):
        return {self.names["weight"]: TensorDecl((self.size,), "norm")}

    def bind(self, get, precision: Precision, device):
        self.weight = precision.vector(get(self.names["weight"]), device)

    def weight_bytes(self):
        return self.size * 4

    def forward(self, ctx, x, delta=None, rows=None):
        return ops.rmsnorm(x, self.weight, self.eps, ctx.precision.act_dtype, delta=delta, rows=rows)

    def defer(self, ctx, x, rows=None):
        return DeferredNorm(x, self.weight, self.eps, rows)

    def plan_params(self):
        """(weight, eps): what the native step plan needs to run this norm in front of a product."""
        return self.weight, self.eps
