"""Dispatch between the attention kernels for one step's batch."""
from __future__ import annotations

from . import ops


def paged_attention(ctx, q, cache, block_table, n_heads, window, scale, out_dtype):
    """Causal GQA of every token of the step over its request's pages."""
    batch = ctx.batch
    return ops.attention_simt(q, cache.k_pool, cache.v_pool, batch.positions, batch.tok_seg,
                              block_table, n_heads, window, scale, out_dtype)
