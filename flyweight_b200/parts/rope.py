"""Rotary position encoding as a (cos, sin) table, with either pairing of channels.

Pair i of a head's first ``rotary_dim`` channels turns by ``pos * theta^(-2i/rot)``
(native/include/flyweight_v2_native_kernels.hpp:993-1008 for the angle, :1034-1047
for the rotation; rot = min(rotary_dimension or hd, hd), native/src/v2_runtime.cpp:4232-4234).
LFM2 pairs channel i with channel i + rot/2 ("half-split", NEOX); the other common
convention pairs 2i with 2i+1 ("interleaved").  Which one is a parameter of the part and of
the kernel, not a property of the attention mixer.
flyweight evaluates powf/cosf/sinf in fp32 on a float position; here the angles are
computed once in float64 on the host and rounded to fp32, so that the rotation at
position 100 000 is as exact as at position 10 and every kernel reads the same values.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position


@register_position("rope")
class Rope(PositionEncoding):
    """params: theta, rotary_dim (even, <= head size), pairing ("half_split" | "interleaved")."""

    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(self.params["theta"])
        self.rotary_dim = int(self.params["rotary_dim"])
        self.pairing = str(self.params.get("pairing", self.pairing))
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        if self.pairing not in ("half_split", "interleaved"):
            raise ValueError(f"unknown rotary pairing {self.pairing!r}")

    def table(self, n_positions: int, device):
        """[n_positions][rotary_dim/2][2] fp32: (cos, sin) of every angle."""
        half = self.rotary_dim // 2
        exponent = torch.arange(half, dtype=torch.float64) * (-2.0 / max(self.rotary_dim, 1))
        inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), exponent)
        angle = torch.arange(n_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        table = torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).to(torch.float32)
        return table.contiguous().to(device)


@register_position("rope_half_split")
class RopeHalfSplit(Rope):
    """params: theta, rotary_dim.  The pairing LFM2 uses."""
    pairing = "half_split"


@register_position("no_position")
class NoPosition(PositionEncoding):
    """Nothing turns: queries and keys go to the attention as the head norm left them."""
