"""Python faces of the CUDA kernels: argument checks, output allocation, launch.

Each function is one kernel (or one dispatch between kernels of the same operation).
Shapes are checked here on the host before anything is launched.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import lib
from .lib import KernelError, c_float, c_longlong, check_tensor, is_bf16, ptr, stream


def _i32(name: str, tensor: torch.Tensor, count: Optional[int] = None) -> None:
    check_tensor(name, tensor, torch.int32)
    if count is not None and tensor.numel() < count:
        raise KernelError(f"{name} holds {tensor.numel()} entries, {count} are needed")


# ------------------------------------------------------------------ embedding
def embed(table: torch.Tensor, ids: torch.Tensor, bad_flag: Optional[torch.Tensor] = None,
          scale: float = 1.0) -> torch.Tensor:
    """Rows ``ids`` of ``table`` ([V][H], fp32 or bf16) widened to fp32 and multiplied by
    ``scale``: [T][H]."""
    check_tensor("embedding table", table)
    _i32("token ids", ids)
    T, (V, H) = ids.numel(), table.shape
    out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    lib.call("fwb_embed", ptr(table), is_bf16(table), ptr(ids), ptr(out), T, H, V, ptr(bad_flag),
             c_float(scale), stream())
    return out


def patch_tokens_(token_ids: torch.Tensor, dst: torch.Tensor, source: torch.Tensor, src: torch.Tensor) -> None:
    """``token_ids[dst[i]] = source[src[i]]`` on the device (all int32): ids that the step before
    sampled and the host has not read yet go straight into this step's batch."""
    for name, tensor in (("token ids", token_ids), ("patch places", dst), ("patch source", source),
                         ("patch rows", src)):
        _i32(name, tensor)
    if dst.numel() != src.numel():
        raise KernelError("one source row per patched place is needed")
    lib.call("fwb_patch_tokens", ptr(token_ids), ptr(dst), ptr(source), ptr(src), dst.numel(), stream())


# ------------------------------------------------------------------ norms
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None
            ) -> torch.Tensor:
    """``(x * rsqrt(mean(x^2) + eps)) * weight`` per row of the fp32 residual ``x``.

    With ``delta`` the residual sum ``x += delta`` happens first, in place and in fp32.
    With ``rows`` (int32 indices) only those rows are normalised, into a compact output.
    """
    check_tensor("residual", x, torch.float32)
    H = x.shape[-1]
    check_tensor("norm weight", weight, torch.float32, (H,))
    if delta is not None:
        check_tensor("delta", delta, torch.float32, x.shape)
    if rows is not None:
        _i32("row indices", rows)
        R = rows.numel()
    else:
        R = x.numel() // H
    out = torch.empty((R, H), dtype=out_dtype, device=x.device)
    lib.call("fwb_rmsnorm", ptr(x), ptr(delta), ptr(weight), ptr(out), is_bf16(out), ptr(rows), R, H,
             c_float(eps), stream())
    return out


def add_(x: torch.Tensor, delta: torch.Tensor) -> None:
    check_tensor("residual", x, torch.float32)
    check_tensor("delta", delta, torch.float32, x.shape)
    lib.call("fwb_add", ptr(x), ptr(delta), c_longlong(x.numel()), stream())


def softcap_(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """``cap * tanh(logits / cap)`` in place on fp32."""
    check_tensor("logits", logits, torch.float32)
    if not cap > 0:
        raise KernelError("a soft-cap must be positive")
    lib.call("fwb_softcap", ptr(logits), c_longlong(logits.numel()), c_float(cap), stream())
    return logits


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    check_tensor("cast input", x)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    lib.call("fwb_cast", ptr(x), is_bf16(x), ptr(out), is_bf16(out), c_longlong(x.numel()), stream())
    return out


# ------------------------------------------------------------------ matrix products
def gemm_simt(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype,
              addend: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None
              ) -> torch.Tensor:
    """``x @ w.T`` with fp32 FMA accumulation (no tensor cores).  x: [M][K], w: [N][K]."""
    check_tensor("gemm input", x)
    check_tensor("gemm weight", w)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: input has {K} columns, weight has {K2}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        check_tensor("gemm output", out, out_dtype, (M, N))
    if addend is not None:
        check_tensor("gemm addend", addend, torch.float32, (M, N))
    lib.call("fwb_gemm_simt", ptr(x), is_bf16(x), ptr(w), is_bf16(w), ptr(out), is_bf16(out),
             ptr(addend), M, N, K, K, N, stream())
    return out


def linear(x, w: torch.Tensor, out_dtype: torch.dtype,
           addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The matrix product the model uses: picks the kernel for the dtypes and sizes.

    float32 weights always take the SIMT kernel (true 32-bit).  bfloat16 weights take
    the tensor-core kernel when it accepts the shape, else the SIMT kernel.  ``x`` may be a
    norm not yet applied (``parts.base.DeferredNorm``): an RMS norm in front of a decode-sized
    bfloat16 product runs inside that product's kernel, otherwise its own kernel runs first.
    """
    from . import tensorcore
    if not isinstance(x, torch.Tensor):                       # a DeferredNorm
        if (addend is None and x.kind == "rmsnorm"
                and tensorcore.normed_accepts(x.n_rows, x.x.shape[-1], w, 1, w.shape[0])):
            return tensorcore.gemm_normed(x.x, x.weight, x.eps, w, out_dtype, rows=x.rows, n_rows=x.n_rows)
        x = x.materialize(torch.float32 if w.dtype == torch.float32 else torch.bfloat16)
    if w.dtype == torch.float32:
        if x.dtype != torch.float32:
            x = cast(x, torch.float32)
        return gemm_simt(x, w, out_dtype, addend)
    if x.dtype != torch.bfloat16:
        x = cast(x, torch.bfloat16)
    if tensorcore.accepts(x, w, out_dtype, addend):
        return tensorcore.gemm(x, w, out_dtype, addend)
    return gemm_simt(x, w, out_dtype, addend)


def linear_into_residual(x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor]):
    """``residual += x @ w.T`` in the product's epilogue when the tensor-core kernel has that
    form for the shape (returns None); otherwise the fp32 product, for the caller to hand on."""
    from . import tensorcore
    if (residual is not None and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
            and tensorcore.adds_in_place(x, w, residual)):
        tensorcore.gemm(x, w, torch.float32, addend=residual, out=residual)
        return None
    return linear(x, w, torch.float32)


def silu_mul(gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up`` = [T][gate(F) | up(F)]."""
    check_tensor("gate|up", gate_up)
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError("gate|up needs an even number of columns")
    out = torch.empty((T, F2 // 2), dtype=out_dtype, device=gate_up.device)
    lib.call("fwb_silu_mul", ptr(gate_up), is_bf16(gate_up), ptr(out), is_bf16(out), T, F2 // 2,
             stream())
    return out


# ------------------------------------------------------------------ gated short convolution
def shortconv(p: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor],
              state: torch.Tensor, seg_start: torch.Tensor, seg_slot: torch.Tensor,
              tok_seg: torch.Tensor, n_segments: int, out_dtype: torch.dtype) -> torch.Tensor:
    """p: [T][B|C|x]; taps: [H][L] fp32; state: [slots][H][L-1] fp32 (read and advanced)."""
    check_tensor("conv input", p)
    T, H3 = p.shape
    H = H3 // 3
    if H * 3 != H3:
        raise KernelError("conv input needs 3*H columns")
    L = taps.shape[1]
    check_tensor("conv taps", taps, torch.float32, (H, L))
    if bias is not None:
        check_tensor("conv bias", bias, torch.float32, (H,))
    if not state.is_cuda or state.dtype != torch.float32 or tuple(state.shape[1:]) != (H, L - 1):
        raise KernelError(f"conv state must be CUDA fp32 [slots][{H}][{L - 1}], got {tuple(state.shape)}")
    if state.stride(2) != 1 or state.stride(1) != L - 1 or (state.shape[0] > 1 and state.stride(0) < H * (L - 1)):
        raise KernelError("a slot of the conv state must be contiguous")
    slot_stride = state.stride(0) if state.shape[0] > 1 else H * (L - 1)
    _i32("seg_start", seg_start, n_segments + 1)
    _i32("seg_slot", seg_slot, n_segments)
    _i32("tok_seg", tok_seg, T)
    out = torch.empty((T, H), dtype=out_dtype, device=p.device)
    lib.call("fwb_shortconv", ptr(p), is_bf16(p), ptr(taps), ptr(bias), ptr(state), ptr(seg_start),
             ptr(seg_slot), ptr(tok_seg), ptr(out), is_bf16(out), T, n_segments, H, L,
             c_longlong(slot_stride), stream())
    return out


# ------------------------------------------------------------------ attention
ROPE_PAIRINGS = {"half_split": 0, "interleaved": 1}


def qk_norm_rope(qkv: torch.Tensor, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                 table: torch.Tensor, positions: torch.Tensor, tok_seg: torch.Tensor,
                 block_table: Optional[torch.Tensor], k_pool: Optional[torch.Tensor],
                 v_pool: Optional[torch.Tensor], n_heads: int, n_kv_in: int, head_dim: int,
                 rotary_dim: int, eps: float, q_dtype: torch.dtype, pairing: str = "half_split"
                 ) -> torch.Tensor:
    """Per-head RMSNorm + RoPE of q and k, k/v written to their pages; returns q [T][nh*hd].

    ``n_kv_in`` is the number of KV heads present in ``qkv`` (0: queries only).
    ``table`` is [max_pos][rotary_dim/2][2] fp32 (cos, sin); pair i turns by entry i.
    ``pairing``: which two channels pair i is made of -- "half_split" (i, i + rotary_dim/2) or
    "interleaved" (2i, 2i + 1)."""
    try:
        pairing_code = ROPE_PAIRINGS[pairing]
    except KeyError:
        raise KernelError(f"unknown rotary pairing {pairing!r}; known: " + ", ".join(ROPE_PAIRINGS)) from None
    check_tensor("qkv", qkv)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_in) * head_dim:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected "
                          f"{(n_heads + 2 * n_kv_in) * head_dim}")
    check_tensor("rope table", table, torch.float32)
    if table.dim() != 3 or table.shape[1] != max(1, rotary_dim // 2) or table.shape[2] != 2:
        raise KernelError("rope table must be [positions][rotary_dim/2][2]")
    use_norm = 1 if q_norm is not None else 0
    if use_norm:
        check_tensor("q norm weight", q_norm, torch.float32, (head_dim,))
        if n_kv_in:
            check_tensor("k norm weight", k_norm, torch.float32, (head_dim,))
    _i32("positions", positions, T)
    _i32("tok_seg", tok_seg, T)
    max_pages = page_size = 0
    cache_bf16 = is_bf16(qkv) if n_kv_in == 0 else 0
    if n_kv_in:
        _i32("block table", block_table)
        check_tensor("k pool", k_pool)
        check_tensor("v pool", v_pool, k_pool.dtype, k_pool.shape)
        if k_pool.dim() != 4 or k_pool.shape[1] != n_kv_in or k_pool.shape[3] != head_dim:
            raise KernelError("cache pools must be [pages][kv_heads][page_size][head_dim]")
        max_pages, page_size = block_table.shape[1], k_pool.shape[2]
        cache_bf16 = is_bf16(k_pool)
    q_out = torch.empty((T, n_heads * head_dim), dtype=q_dtype, device=qkv.device)
    if n_kv_in == 0:
        cache_bf16 = is_bf16(q_out)
    lib.call("fwb_qk_norm_rope", ptr(qkv), is_bf16(qkv), ptr(q_norm), ptr(k_norm), ptr(table),
             ptr(positions), ptr(tok_seg), ptr(block_table), max_pages, page_size, ptr(q_out),
             is_bf16(q_out), ptr(k_pool), ptr(v_pool), cache_bf16, T, n_heads, n_kv_in, head_dim,
             rotary_dim, c_float(eps), use_norm, pairing_code, stream())
    return q_out


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   positions: torch.Tensor, tok_seg: torch.Tensor, block_table: torch.Tensor,
                   n_heads: int, window: int, scale: float, out_dtype: torch.dtype) -> torch.Tensor:
    """Causal GQA over the paged cache, SIMT fp32 arithmetic.  q: [T][nh*hd]."""
    check_tensor("q", q)
    check_tensor("k pool", k_pool)
    check_tensor("v pool", v_pool, k_pool.dtype, k_pool.shape)
    T = q.shape[0]
    _, n_kv, page_size, head_dim = k_pool.shape
    if q.shape[1] != n_heads * head_dim:
        raise KernelError(f"q has {q.shape[1]} columns, expected {n_heads * head_dim}")
    _i32("positions", positions, T)
    _i32("tok_seg", tok_seg, T)
    _i32("block table", block_table)
    out = torch.empty((T, n_heads * head_dim), dtype=out_dtype, device=q.device)
    lib.call("fwb_attention_simt", ptr(q), is_bf16(q), ptr(k_pool), ptr(v_pool), is_bf16(k_pool),
             ptr(positions), ptr(tok_seg), ptr(block_table), block_table.shape[1], page_size,
             ptr(out), is_bf16(out), T, n_heads, n_kv, head_dim, window, c_float(scale), stream())
    return out


def attention_mma_shape_ok(n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """Shapes the tensor-core attention kernels take (the SIMT kernel takes the rest)."""
    return (n_heads % n_kv == 0 and n_heads // n_kv <= 16 and 16 <= head_dim <= 128
            and head_dim % 16 == 0 and page_size == 64)


def attention_prefill_mma(q, k_pool, v_pool, positions, seg_start, tile_seg, tile_tok0, n_tiles,
                          tokens_per_tile, block_table, n_heads, window, scale, out=None) -> torch.Tensor:
    """Causal GQA of prompt portions (any mix of segments) on tensor cores; all bf16.  Only the
    rows of the given tiles are written (``out``: a tensor like q that other rows already live in)."""
    check_tensor("q", q, torch.bfloat16)
    check_tensor("k pool", k_pool, torch.bfloat16)
    check_tensor("v pool", v_pool, torch.bfloat16, k_pool.shape)
    T = q.shape[0]
    _, n_kv, page_size, head_dim = k_pool.shape
    if q.shape[1] != n_heads * head_dim:
        raise KernelError(f"q has {q.shape[1]} columns, expected {n_heads * head_dim}")
    _i32("positions", positions, T)
    _i32("seg_start", seg_start)
    _i32("tile_seg", tile_seg, n_tiles)
    _i32("tile_tok0", tile_tok0, n_tiles)
    _i32("block table", block_table)
    if out is None:
        out = torch.empty_like(q)
    else:
        check_tensor("attention output", out, torch.bfloat16, q.shape)
    lib.call("fwb_attention_prefill_mma", ptr(q), ptr(k_pool), ptr(v_pool), ptr(positions),
             ptr(seg_start), ptr(tile_seg), ptr(tile_tok0), ptr(block_table), block_table.shape[1],
             page_size, ptr(out), n_tiles, n_heads, n_kv, head_dim, tokens_per_tile, window,
             c_float(scale), stream())
    return out


def attention_tcgen05_shape_ok(n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """Shapes the tcgen05 prompt kernel takes: head sizes 64 and 128, up to 128 rows per KV head."""
    return (head_dim in (64, 128) and page_size == 64 and n_kv > 0 and n_heads % n_kv == 0
            and n_heads // n_kv <= 128)


def attention_prefill_tcgen05(q, k_pool, v_pool, positions, seg_start, tile_seg, tile_tok0, n_tiles,
                              tokens_per_tile, block_table, n_heads, window, scale, out=None) -> torch.Tensor:
    """The same operation on tcgen05 tensor cores: 128 query rows per CTA, S and PV in tensor
    memory (head sizes 64 and 128); all bf16."""
    check_tensor("q", q, torch.bfloat16)
    check_tensor("k pool", k_pool, torch.bfloat16)
    check_tensor("v pool", v_pool, torch.bfloat16, k_pool.shape)
    T = q.shape[0]
    num_pages, n_kv, page_size, head_dim = k_pool.shape
    if q.shape[1] != n_heads * head_dim:
        raise KernelError(f"q has {q.shape[1]} columns, expected {n_heads * head_dim}")
    _i32("positions", positions, T)
    _i32("seg_start", seg_start)
    _i32("tile_seg", tile_seg, n_tiles)
    _i32("tile_tok0", tile_tok0, n_tiles)
    _i32("block table", block_table)
    if out is None:
        out = torch.empty_like(q)
    else:
        check_tensor("attention output", out, torch.bfloat16, q.shape)
    lib.call("fwb_attention_prefill_tcgen05", ptr(q), ptr(k_pool), ptr(v_pool), ptr(positions),
             ptr(seg_start), ptr(tile_seg), ptr(tile_tok0), ptr(block_table), block_table.shape[1],
             page_size, num_pages, ptr(out), n_tiles, n_heads, n_kv, head_dim, tokens_per_tile, window,
             c_float(scale), stream())
    return out


def attention_decode_fused(qkv, q_norm, k_norm, table, rotary_dim: int, eps: float, pairing: str, n_kv_in: int,
                           k_pool, v_pool, positions, tok_seg, block_table, n_heads: int, window: int,
                           scale: float, splits: int, tiles_per_split: int, merge_in_cluster: bool = False
                           ) -> torch.Tensor:
    """``qk_norm_rope`` and ``attention_decode_mma`` of a step of single tokens in one kernel: every
    CTA of the attention norms and turns the queries of its KV head's group itself, and the slice that
    holds a token's own position its key (and copies its value) into the pages.  ``qkv`` is the fused
    projection [T][(n_heads + 2 n_kv_in) head_dim] in bfloat16; the other arguments are those of the two
    functions.  The same bits as the two kernels (one device function does the arithmetic of both)."""
    pairing_code = ROPE_PAIRINGS[pairing]
    check_tensor("qkv", qkv, torch.bfloat16)
    check_tensor("k pool", k_pool, torch.bfloat16)
    check_tensor("v pool", v_pool, torch.bfloat16, k_pool.shape)
    check_tensor("rope table", table, torch.float32)
    T = qkv.shape[0]
    num_pages, n_kv, page_size, head_dim = k_pool.shape
    if qkv.shape[1] != (n_heads + 2 * n_kv_in) * head_dim:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected {(n_heads + 2 * n_kv_in) * head_dim}")
    if table.dim() != 3 or table.shape[1] != max(1, rotary_dim // 2) or table.shape[2] != 2:
        raise KernelError("rope table must be [positions][rotary_dim/2][2]")
    use_norm = 1 if q_norm is not None else 0
    if use_norm:
        check_tensor("q norm weight", q_norm, torch.float32, (head_dim,))
        if n_kv_in:
            check_tensor("k norm weight", k_norm, torch.float32, (head_dim,))
    _i32("positions", positions, T)
    _i32("tok_seg", tok_seg, T)
    _i32("block table", block_table)
    out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    part_o = part_ml = None
    in_cluster = merge_in_cluster and 1 < splits <= 8
    if splits > 1 and not in_cluster:
        group = n_heads // n_kv
        part_o = torch.empty((T, n_kv, splits, group, head_dim), dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty((T, n_kv, splits, group, 2), dtype=torch.float32, device=qkv.device)
    lib.call("fwb_attention_decode_fused", ptr(qkv), n_kv_in, ptr(q_norm), ptr(k_norm), ptr(table), rotary_dim,
             c_float(eps), use_norm, pairing_code, ptr(k_pool), ptr(v_pool), ptr(positions), ptr(tok_seg),
             ptr(block_table), block_table.shape[1], page_size, num_pages, ptr(out), ptr(part_o), ptr(part_ml),
             T, n_heads, n_kv, head_dim, splits, tiles_per_split, window, c_float(scale),
             1 if in_cluster else 0, stream(), launches=2 if (splits > 1 and not in_cluster) else 1)
    return out


def set_decode_attention_tma(on: bool, stages: int = 0) -> None:
    """Test switch: whether the decode attention kernel takes its key and value tiles by TMA at head
    sizes 64 and 128 (the default) or by cp.async, as at the other head sizes; and the depth of the TMA
    way's ring (2 to 8; 0: the launcher's choice).  The same bits."""
    lib.call("fwb_attention_decode_set_tma", 1 if on else 0, int(stages))


def attention_decode_mma(q, k_pool, v_pool, positions, tok_seg, block_table, n_heads, window, scale,
                         splits: int, tiles_per_split: int, merge_in_cluster: bool = False,
                         out=None, n_tokens=None) -> torch.Tensor:
    """Causal GQA of single decode tokens on tensor cores, the context cut into ``splits``
    slices of ``tiles_per_split`` 64-key tiles that run as separate CTAs and are merged: inside
    the kernel (``merge_in_cluster``, up to 8 slices as a thread-block cluster) or through scratch
    and a second kernel.  ``n_tokens``: only the first that many rows of q are decode tokens (the
    head of a mixed step); the other rows of ``out`` are left alone."""
    check_tensor("q", q, torch.bfloat16)
    check_tensor("k pool", k_pool, torch.bfloat16)
    check_tensor("v pool", v_pool, torch.bfloat16, k_pool.shape)
    T = q.shape[0] if n_tokens is None else int(n_tokens)
    if not 0 < T <= q.shape[0]:
        raise KernelError(f"{T} decode tokens of {q.shape[0]} rows")
    _, n_kv, page_size, head_dim = k_pool.shape
    if q.shape[1] != n_heads * head_dim:
        raise KernelError(f"q has {q.shape[1]} columns, expected {n_heads * head_dim}")
    _i32("positions", positions, T)
    _i32("tok_seg", tok_seg, T)
    _i32("block table", block_table)
    if out is None:
        out = torch.empty_like(q)
    else:
        check_tensor("attention output", out, torch.bfloat16, q.shape)
    part_o = part_ml = None
    in_cluster = merge_in_cluster and 1 < splits <= 8
    if splits > 1 and not in_cluster:
        group = n_heads // n_kv
        part_o = torch.empty((T, n_kv, splits, group, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((T, n_kv, splits, group, 2), dtype=torch.float32, device=q.device)
    lib.call("fwb_attention_decode_mma", ptr(q), ptr(k_pool), ptr(v_pool), ptr(positions),
             ptr(tok_seg), ptr(block_table), block_table.shape[1], page_size, k_pool.shape[0], ptr(out), ptr(part_o),
             ptr(part_ml), T, n_heads, n_kv, head_dim, splits, tiles_per_split, window,
             c_float(scale), 1 if in_cluster else 0, stream(),
             launches=2 if (splits > 1 and not in_cluster) else 1)
    return out
