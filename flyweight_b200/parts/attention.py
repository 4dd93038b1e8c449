"""Grouped-query attention mixer with per-head q/k RMSNorm and rotary positions.

Order of operations (native/src/v2_runtime.cpp:28429-28478): q, k, v projections
without bias; RMSNorm over each head of q and of k with a [head_dim] weight shared by
all heads; rotary encoding of q and k; k and v appended to the cache; scores of query
head j against KV head j // (heads / kv_heads), scaled by head_dim^-1/2, causal,
softmax in fp32; output projection without gate.
"""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Mixer, PagedKV, Precision, build_position, register_mixer


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (None: no
    q/k norm), position (PartSpec of a position encoding), window (0: all keys),
    shares_cache (True: reads the cache of another execution and projects q only).
    tensors: q, k, v, o, q_norm, k_norm."""
    graph_safe = True
    takes_deferred_norm = True
    adds_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.eps = p.get("qk_norm_eps")
        self.window = int(p.get("window", 0) or 0)
        self.shares_cache = bool(p.get("shares_cache", False))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.position = build_position(p["position"])
        if self.n_heads % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.head_dim % 16:
            raise ValueError(f"head size {self.head_dim}: the attention kernels take head sizes "
                             "in steps of 16")
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    @property
    def _kv_in(self) -> int:
        return 0 if self.shares_cache else self.n_kv

    def declare(self):
        n, hd, H = self.names, self.head_dim, self.hidden
        out = {n["q"]: TensorDecl((self.n_heads * hd, H)),
               n["o"]: TensorDecl((H, self.n_heads * hd))}
        if not self.shares_cache:
            out[n["k"]] = TensorDecl((self.n_kv * hd, H))
            out[n["v"]] = TensorDecl((self.n_kv * hd, H))
        if self.eps is not None:
            out[n["q_norm"]] = TensorDecl((hd,), "norm")
            if not self.shares_cache:
                out[n["k_norm"]] = TensorDecl((hd,), "norm")
        return out

    def bind(self, get, precision: Precision, device):
        n = self.names
        mats = [get(n["q"])]
        if not self.shares_cache:
            mats += [get(n["k"]), get(n["v"])]
        dtypes = {m.dtype for m in mats}
        if len(dtypes) > 1:
            mats = [m.to(torch.float32) for m in mats]
        # one projection for q|k|v: the rows of the three matrices, one after the other
        self.w_qkv = precision.matrix(torch.cat(mats, dim=0), device)
        self.w_o = precision.matrix(get(n["o"]), device)
        if self.eps is not None:
            self.q_norm = precision.vector(get(n["q_norm"]), device)
            if not self.shares_cache:
                self.k_norm = precision.vector(get(n["k_norm"]), device)

    def weight_bytes(self):
        return (self.w_qkv.numel() * self.w_qkv.element_size()
                + self.w_o.numel() * self.w_o.element_size())

    def flops_per_token(self):
        return 2.0 * (self.w_qkv.numel() + self.w_o.numel())

    def context_flops(self, n_tokens):
        # QK^T and PV: 4 operations per (query, visible key, channel); half the pairs are masked
        return 2.0 * n_tokens * n_tokens * self.n_heads * self.head_dim

    def state_spec(self):
        return None if self.shares_cache else PagedKV(self.n_kv, self.head_dim, self.window)

    def prepare(self, max_positions, device):
        self.position.prepare(max_positions, device)

    def forward(self, ctx, h, cache, residual=None):
        act = ctx.precision.act_dtype
        # q|k|v in the activation dtype; the head norm and the rotation widen it to fp32
        qkv = ops.linear(h, self.w_qkv, act)
        block_table = ctx.batch.block_tables[cache.group]
        from ..kernels import attention as attention_kernels
        rotation = self.position.rotation()
        if rotation is not None and attention_kernels.decode_fusable(ctx, qkv, cache, block_table, self.n_heads, rotation[1], self.window):
            # a step of single tokens whose position part is a plain rotation: the decode attention
            # kernel norms, turns and stores its own token's heads (one kernel and one pass less)
            table, rotary_dim, pairing = rotation
            out = attention_kernels.fused_decode_attention(
                ctx, qkv, cache, block_table, self.n_heads, self._kv_in, self.window, self.scale,
                self.q_norm, self.k_norm, self.eps, table, rotary_dim, pairing)
            return ops.linear_into_residual(out, self.w_o, residual)
        # positions are the position part's business: it norms, encodes and writes the pages
        q = self.position.encode(ctx, qkv, n_heads=self.n_heads, n_kv_in=self._kv_in,
                                 head_dim=self.head_dim, q_norm=self.q_norm, k_norm=self.k_norm,
                                 eps=self.eps, cache=cache, block_table=block_table)
        out = attention_kernels.paged_attention(ctx, q, cache, block_table, self.n_heads,
                                                self.window, self.scale, act)
        return ops.linear_into_residual(out, self.w_o, residual)

    def plan(self, builder, norm, cache):
        """The same operations for the native step plan (``engine/plan.py``)."""
        from ..engine.plan import EPI_ACT, NotPlannable
        act = builder.act_dtype
        plan_position = getattr(self.position, "plan", None)
        if plan_position is None:
            raise NotPlannable(f"position encoding {self.position.kind!r} has no native form")
        width = self.n_heads * self.head_dim
        qkv = builder.tokens(width + 2 * self._kv_in * self.head_dim, act)
        builder.norm_linear(norm, self.w_qkv, EPI_ACT, qkv, "q|k|v")
        q = builder.tokens(width, act)
        plan_position(builder, qkv, q, n_heads=self.n_heads, n_kv_in=self._kv_in, head_dim=self.head_dim,
                      q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, cache=cache)
        builder.free(qkv)
        out = builder.tokens(width, act)
        builder.attention(q, cache, out, self.n_heads, self.window, self.scale)
        builder.free(q)
        builder.linear_residual(out, self.w_o, "attention out_proj")
        builder.free(out)
