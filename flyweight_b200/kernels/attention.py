"""Dispatch between the attention kernels for one step's batch.

bfloat16 cache and a shape the tensor-core kernels take: a step of single decode tokens runs
the split-context decode kernel; prompt portions that fill 128-row tiles run the tcgen05 kernel
(head sizes 64 and 128); anything else the tiled mma.sync kernel.  Everything else
(the 32-bit path, head sizes above 128, more than 16 query heads per KV head) runs the SIMT
kernel.
"""
from __future__ import annotations

import torch

from . import lib, ops

SM_COUNT = 148
CLUSTER_MERGE_CTAS = 1024
_use_mma = True


def set_mma_enabled(flag: bool) -> None:
    """Tests switch the tensor-core kernels off to compare them with the SIMT kernel."""
    global _use_mma
    _use_mma = bool(flag)
    lib.set_option("attention_mma", _use_mma)


_force_tiled = False
_use_tcgen05 = True


def set_tcgen05_enabled(flag: bool) -> None:
    """Prompt portions through the mma.sync kernel instead of the tcgen05 one (for comparisons)."""
    global _use_tcgen05
    _use_tcgen05 = bool(flag)
    lib.set_option("attention_tcgen05", _use_tcgen05)



_split_mixed = True


def set_mixed_split(flag: bool) -> None:
    """Decoding requests at the head of a mixed step through the decode kernel (on by default)."""
    global _split_mixed
    _split_mixed = bool(flag)
    lib.set_option("mixed_split", _split_mixed)


def tiled_forced() -> bool:
    """Whether single decode tokens go through the tiled kernel too (``force_tiled``)."""
    return _force_tiled


def heads_the_decode_kernel() -> bool:
    """Whether the decoding requests at the head of a mixed step go to the decode kernel (the tile
    lists of the prompt kernels then start behind them)."""
    return _split_mixed and not _force_tiled


def force_tiled(flag: bool) -> None:
    """Send single decode tokens through the tiled kernel too.  A row of that kernel is summed
    in one order whatever else is in the step, so tests can compare cuts bit by bit."""
    global _force_tiled
    _force_tiled = bool(flag)
    lib.set_option("force_tiled", _force_tiled)


def decode_splits(n_tokens: int, n_kv: int, max_tiles: int, head_dim: int = 64):
    """How many slices of the context run as separate CTAs: (slices, tiles per slice, merged inside the
    kernel by a cluster).  Depends only on static sizes of the step (tokens, KV heads, block-table
    width), so a captured graph stays valid."""
    # Measured on B200 (hd 64, 8 KV heads, batch 1 to 256, 512 to 127k keys), tiles by TMA: the kernel
    # is fastest when all its CTAs are resident at once -- five an SM -- and there are as many of
    # them as that allows: 8 x 4,096 keys in 8 slices (512 CTAs) 15.5 us, 16 x 4,096 in 4 slices 25.4 us
    # (in 8: 32.7), 32 x 4,096 in 2 slices 45.9 us (in 8: 52.9), 64 x 4,096 in one piece 83.7 us (in 8:
    # 91.8).  A slice has at least 8 tiles, and at most 128: the grid is laid out for the longest request
    # of the step, and one long request among short ones must not walk its context alone.  Where the
    # CTAs cannot all be resident, the fewest slices that fill the last round of the SMs to 85 % (128 x
    # 4,096 in one piece is 1.4 rounds: 182 us; in two slices 163 us).  Up to 8 slices merge inside the
    # kernel as a cluster while the launch is small; more, or many CTAs, go through a merge kernel.
    pairs = max(1, n_tokens * n_kv)
    resident = SM_COUNT * (5 if head_dim <= 64 else 3)
    least = 1
    while least * 128 < max_tiles and least < 64:
        least *= 2
    choice = 0
    splits = least
    while splits <= 64 and pairs * splits <= resident and (splits == least or splits * 8 <= max_tiles):
        choice = splits
        splits *= 2
    if not choice:
        splits = least
        while splits <= 64:
            ctas = pairs * splits
            if ctas >= 0.85 * (-(-ctas // resident) * resident):
                choice = splits
                break
            splits *= 2
    if not choice:
        choice = least
    tiles_per_split = -(-max_tiles // choice)
    splits = -(-max_tiles // tiles_per_split)
    in_cluster = 1 < splits <= 8 and pairs * splits <= CLUSTER_MERGE_CTAS
    return splits, tiles_per_split, in_cluster


_fuse_rope = True


def set_rope_fusion(flag: bool) -> None:
    """Whether a step of single tokens does its q/k norm, rotation and page write inside the decode
    attention kernel (the default) or in the kernel of its own that every other step uses."""
    global _fuse_rope
    _fuse_rope = bool(flag)


FUSE_ROPE_CLUSTER_CTAS = 256


def decode_fusable(ctx, qkv, cache, block_table, n_heads: int, rotary_dim: int, window: int = 0) -> bool:
    """Whether ``fused_decode_attention`` takes this step: single tokens only, everything bfloat16, a
    shape the tensor-core decode kernel has, a rotary width the 16-byte lanes can pair up -- and a
    launch that gains by it.  Measured in the decode step of LFM2-1.2B: batch 1 (64 CTAs in clusters)
    0.783 -> 0.775 ms, batch 64 (512 CTAs, no clusters) 1.56 -> 1.53 ms, but batch 8 (512 CTAs in clusters
    of 8) 0.867 -> 0.881 ms: the kernel of its own was the window in which that many clusters found
    their SMs and fetched their first tiles, so such launches keep it."""
    k_pool = cache.k_pool
    if window:
        return False                 # (layers with a sliding window keep the two kernels: not measured, not tested)
    if not (_fuse_rope and _use_mma and not _force_tiled and ctx.batch.max_segment == 1
            and qkv.dtype == torch.bfloat16 and k_pool is not None and k_pool.dtype == torch.bfloat16
            and ctx.precision.act_dtype == torch.bfloat16 and rotary_dim % 16 == 0
            and ops.attention_mma_shape_ok(n_heads, k_pool.shape[1], k_pool.shape[3], k_pool.shape[2])):
        return False
    n_kv, head_dim = k_pool.shape[1], k_pool.shape[3]
    splits, _, in_cluster = decode_splits(ctx.batch.n_tokens, n_kv, block_table.shape[1], head_dim)
    return not (in_cluster and ctx.batch.n_tokens * n_kv * splits >= FUSE_ROPE_CLUSTER_CTAS)


def fused_decode_attention(ctx, qkv, cache, block_table, n_heads, n_kv_in, window, scale, q_norm, k_norm, eps,
                           table, rotary_dim, pairing):
    """A step of single tokens: head norms, rotation, page write and attention in one kernel."""
    batch = ctx.batch
    _, n_kv, _, head_dim = cache.k_pool.shape
    splits, tiles_per_split, in_cluster = decode_splits(batch.n_tokens, n_kv, block_table.shape[1], head_dim)
    return ops.attention_decode_fused(qkv, q_norm, k_norm, table, rotary_dim, float(eps or 0.0), pairing, n_kv_in,
                                      cache.k_pool, cache.v_pool, batch.positions, batch.tok_seg, block_table,
                                      n_heads, window, scale, splits, tiles_per_split, in_cluster)


def paged_attention(ctx, q, cache, block_table, n_heads, window, scale, out_dtype):
    """Causal GQA of every token of the step over its request's pages."""
    batch = ctx.batch
    k_pool, v_pool = cache.k_pool, cache.v_pool
    _, n_kv, page_size, head_dim = k_pool.shape
    if (_use_mma and q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16
            and out_dtype == torch.bfloat16
            and ops.attention_mma_shape_ok(n_heads, n_kv, head_dim, page_size)):
        if batch.max_segment == 1 and not _force_tiled:
            splits, tiles_per_split, in_cluster = decode_splits(batch.n_tokens, n_kv, block_table.shape[1], head_dim)
            return ops.attention_decode_mma(q, k_pool, v_pool, batch.positions, batch.tok_seg,
                                            block_table, n_heads, window, scale, splits,
                                            tiles_per_split, in_cluster)
        group = n_heads // n_kv
        out = None
        first = 0
        if batch.leading_singles and not _force_tiled and _split_mixed:
            # a mixed step: the decoding requests at its head run the split-context kernel (a tile
            # of the prompt kernels would hold one token and walk the whole context alone), the
            # portions of prompts behind them the tiled kernels; both write their rows of `out`
            first = batch.leading_singles
            out = torch.empty_like(q)
            splits, tiles_per_split, in_cluster = decode_splits(first, n_kv, block_table.shape[1], head_dim)
            ops.attention_decode_mma(q, k_pool, v_pool, batch.positions, batch.tok_seg, block_table,
                                     n_heads, window, scale, splits, tiles_per_split, in_cluster,
                                     out=out, n_tokens=first)
        if (_use_tcgen05 and not _force_tiled and ops.attention_tcgen05_shape_ok(n_heads, n_kv, head_dim, page_size)
                and 2 * batch.max_segment * group >= 128):
            # prompt portions that fill at least half of a 128-row tile: S and PV in tensor memory
            tokens_per_tile = max(1, 128 // group)
            tile_seg, tile_tok0, n_tiles = batch.attention_tiles(tokens_per_tile, first)
            return ops.attention_prefill_tcgen05(q, k_pool, v_pool, batch.positions, batch.seg_start,
                                                 tile_seg, tile_tok0, n_tiles, tokens_per_tile,
                                                 block_table, n_heads, window, scale, out=out)
        tokens_per_tile = max(1, 64 // group)
        tile_seg, tile_tok0, n_tiles = batch.attention_tiles(tokens_per_tile, first)
        return ops.attention_prefill_mma(q, k_pool, v_pool, batch.positions, batch.seg_start,
                                         tile_seg, tile_tok0, n_tiles, tokens_per_tile, block_table,
                                         n_heads, window, scale, out=out)
    return ops.attention_simt(q, k_pool, v_pool, batch.positions, batch.tok_seg, block_table,
                              n_heads, window, scale, out_dtype)
