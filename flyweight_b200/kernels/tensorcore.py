"""Tensor-core (tcgen05) matrix products of the bfloat16 path.

``accepts`` says whether the kernel takes a product; the dispatcher in ``ops.linear`` falls
back to the SIMT kernel otherwise, so every shape the configuration allows still runs.
"""
from __future__ import annotations

import torch

from . import lib
from .lib import KernelError, check_tensor, ptr, stream

EPI_F32, EPI_BF16, EPI_ADD_F32, EPI_SWIGLU_BF16 = 0, 1, 2, 3
SM_COUNT = 148
_enabled = True


def set_enabled(flag: bool) -> None:
    """Tests switch the tensor-core path off to compare it with the SIMT path."""
    global _enabled
    _enabled = bool(flag)


def _aligned(t: torch.Tensor) -> bool:
    return t.data_ptr() % 16 == 0


def accepts(x, w, out_dtype, addend=None) -> bool:
    if not _enabled:
        return False
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if out_dtype not in (torch.float32, torch.bfloat16):
        return False
    if addend is not None and out_dtype != torch.float32:
        return False
    K = x.shape[1]
    return K % 8 == 0 and K >= 8 and _aligned(x) and _aligned(w) and x.shape[0] <= 65535 * 16


_forced_splits = None
# Per-shape overrides found by measurement: (features, K, accumulators) -> (splits, stages);
# 0 keeps the rule's choice.  Only decode-sized token counts (<= 64) consult it.
TUNED = {}


def force_splits(splits) -> None:
    """Pin the split-K factor (None: chosen per shape).  With one fixed factor every output
    element is summed in the same order whatever the number of tokens in the step, which
    lets tests compare ways of cutting the work bit by bit."""
    global _forced_splits
    _forced_splits = splits


def pick_splits(M: int, N: int, K: int) -> int:
    """CTAs that share one output tile's K range (a cluster, <= 8): as many as it takes to
    put work on every SM when the token tile is small (decode), 1 otherwise."""
    if _forced_splits is not None:
        return _forced_splits if M <= 64 else 1
    if M > 64:
        return 1
    return _splits_for(M, N, K, 1)


def _ring_depth(bn: int, accumulators: int) -> int:
    """Stages of the shared-memory ring for decode-sized steps: shallow enough that several
    CTAs (and the next kernel's, prefetching weights) fit an SM."""
    if accumulators == 2:
        return 3 if bn <= 32 else 4
    return 4


def _splits_for(M: int, N: int, K: int, accumulators: int) -> int:
    """The largest power of two (<= 8) that still lets every CTA be resident at once; measured
    on B200 inside the decode step of LFM2-1.2B at batch 1, 8 and 64: a second wave costs more
    than the extra slices win."""
    bn = 16 if M <= 16 else (32 if M <= 32 else 64)
    if accumulators == 2 and bn == 64:
        return 1
    stage = accumulators * 16384 + bn * 128
    per_sm = max(1, (227 * 1024) // (_ring_depth(bn, accumulators) * stage + 2048))
    tiles = -(-N // 128)
    k_blocks = -(-K // 64)
    splits = 1
    while splits < 8 and tiles * splits * 2 <= 0.9 * SM_COUNT * per_sm and k_blocks >= splits * 8:
        splits *= 2
    return splits


def gemm(x, w, out_dtype, addend=None, splits=None, stages=0, tile_tokens=0, wide=-1) -> torch.Tensor:
    """``x @ w.T``: x [M][K] bf16, w [N][K] bf16 -> [M][N] fp32 or bf16 (+ fp32 addend)."""
    check_tensor("gemm input", x, torch.bfloat16)
    check_tensor("gemm weight", w, torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: input has {K} columns, weight has {w.shape[1]}")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if addend is not None:
        check_tensor("gemm addend", addend, torch.float32, (M, N))
        epilogue = EPI_ADD_F32
    else:
        epilogue = EPI_F32 if out_dtype == torch.float32 else EPI_BF16
    if M <= 64 and (N, K, 1) in TUNED and _forced_splits is None:
        tuned = TUNED[(N, K, 1)]
        splits = splits or tuned[0] or None
        stages = stages or tuned[1]
    if splits is None:
        splits = pick_splits(M, N, K)
    if not stages and M <= 64:
        stages = _ring_depth(16 if M <= 16 else (32 if M <= 32 else 64), 1)
    lib.call("fwb_gemm_tcgen05", ptr(x), ptr(w), ptr(out), ptr(addend), M, N, K, N, N, epilogue, 0,
             splits, stages, tile_tokens, wide, stream())
    return out


def swiglu_accepts(x, w_gate_up) -> bool:
    return accepts(x, w_gate_up, torch.bfloat16)


def swiglu_gate_up(x, w_gate_up, splits=None, stages=0, tile_tokens=0) -> torch.Tensor:
    """``silu(x @ gate.T) * (x @ up.T)`` as bf16, for ``w_gate_up`` = [gate rows | up rows]:
    both products accumulate side by side in tensor memory and never reach global memory."""
    check_tensor("swiglu input", x, torch.bfloat16)
    check_tensor("swiglu weight", w_gate_up, torch.bfloat16)
    M, K = x.shape
    F2 = w_gate_up.shape[0]
    F = F2 // 2
    if w_gate_up.shape[1] != K or F * 2 != F2:
        raise KernelError("swiglu: weight must be [2F][K]")
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    if M <= 64 and (F, K, 2) in TUNED and _forced_splits is None:
        tuned = TUNED[(F, K, 2)]
        splits = splits or tuned[0] or None
        stages = stages or tuned[1]
    if splits is None:
        splits = (_forced_splits if _forced_splits is not None else _splits_for(M, F, K, 2)) if M <= 64 else 1
    if not stages and M <= 64:
        stages = _ring_depth(16 if M <= 16 else (32 if M <= 32 else 64), 2)
    lib.call("fwb_gemm_tcgen05", ptr(x), ptr(w_gate_up), ptr(out), ptr(None), M, F, K, F2, F,
             EPI_SWIGLU_BF16, F, splits, stages, tile_tokens, -1, stream())
    return out


def status() -> int:
    """0, or the code a wait that gave up inside the kernel left (reads and clears it;
    synchronises the device)."""
    return int(lib.library().fwb_gemm_tcgen05_status())
