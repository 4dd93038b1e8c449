"""Turning rows of logits into token ids on the device.

One launch for a batch of greedy rows (argmax, ties to the lowest id -- the order
flyweight's fused argmax gives, native/include/flyweight_v2_qwen_kernels.hpp:2392-2398);
one launch for rows that sample (top-k, penalties, temperature, top-p, min-p, draw: the
order of native/src/v2_runtime.cpp:29331-29744); rows that keep more than 1024 candidates
(the whole vocabulary among them) need a scratch word per logit and are not sorted at all,
and take their penalties on the whole row before the cut (src/flyweight/v2.py:1497-1518).
"""
from __future__ import annotations

import struct
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import lib
from ..kernels.lib import KernelError, check_tensor, ptr, stream
from .config import SamplingConfig

SMALL_K = 1024


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """int32 [R]: index of the largest logit of each row, the lowest id among equals."""
    check_tensor("logits", logits, torch.float32)
    R, V = logits.shape
    out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    # few rows: a row is cut into slices that run as separate blocks (8 rows x 65,536: 6 us against 9);
    # from 64 rows on the rows fill the GPU by themselves and one block a row is faster (512 rows:
    # 28 us, three quarters of the copy bandwidth, against 82 us in 32 slices)
    chunks = max(1, min(64, V // 2048)) if R < 64 else 1
    partial, counters = _argmax_scratch(logits.device, R * chunks, R)
    lib.call("fwb_argmax", ptr(logits), R, V, ptr(out), ptr(partial), ptr(counters), chunks, stream())
    return out


_scratch = {}
_staging = {}


def _stage(values: "np.ndarray", device) -> torch.Tensor:
    """Bytes to the device through a kept ring of pinned buffers (no pageable copy, which would
    make the host wait for the stream)."""
    key = str(device)
    ring = _staging.setdefault(key, {"buffers": [None] * 4, "events": [None] * 4, "turn": 0})
    turn = ring["turn"]
    ring["turn"] = (turn + 1) % 4
    if ring["events"][turn] is not None:
        ring["events"][turn].synchronize()
    buffer = ring["buffers"][turn]
    if buffer is None or buffer.numel() < values.size:
        buffer = ring["buffers"][turn] = torch.empty(max(4096, 2 * values.size), dtype=torch.uint8).pin_memory()
    host = buffer[:values.size]
    host.numpy()[:] = values
    dev = host.to(device, non_blocking=True)
    if ring["events"][turn] is None:
        ring["events"][turn] = torch.cuda.Event()
    ring["events"][turn].record()
    return dev


def _argmax_scratch(device, n_partial: int, n_rows: int):
    """Scratch of the split argmax: slice maxima and per-row arrival counters (kept zero by the
    kernel itself).  One buffer per device, grown when a larger batch comes."""
    key = str(device)
    held = _scratch.get(key)
    if held is None or held[0].numel() < n_partial or held[1].numel() < n_rows:
        held = (torch.empty(max(n_partial, 4096), dtype=torch.int64, device=device),
                torch.zeros(max(n_rows, 256), dtype=torch.int32, device=device))
        _scratch[key] = held
    return held


def set_ctas_per_row(ctas: int) -> None:
    """CTAs that share a row in the sampling kernel: 8, 4, 2 or 1; 0 (the default) lets the number of
    rows decide -- eight for a few rows, fewer as rows fill the GPU by themselves.  Every choice
    draws the same tokens (the masses are summed as integers)."""
    lib.call("fwb_sample_set_cluster", int(ctas))


def sample(logits: torch.Tensor, configs: Sequence[SamplingConfig], uniforms: Sequence[float],
           recents: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
    """int32 [R]: one token per row.  ``uniforms[r]`` is the number in [0, 1) row r draws
    with; ``recents[r]`` the request's recent generated tokens (for the penalties)."""
    check_tensor("logits", logits, torch.float32)
    R, V = logits.shape
    if len(configs) != R or len(uniforms) != R:
        raise KernelError("one sampling config and one uniform number per row are needed")
    stride = 0
    rows: List[List[int]] = []
    for r, cfg in enumerate(configs):
        recent = list(recents[r])[-cfg.penalty_window:] if (recents and cfg.penalizes) else []
        rows.append(recent)
        stride = max(stride, len(recent))
    need_large = penalize_rows = False
    blob = bytearray()
    for cfg, recent in zip(configs, rows):
        k = min(cfg.top_k, V) if cfg.top_k > 0 else V
        sampled = (cfg.temperature > 0.0 or bool(recent)) and k > 1
        if sampled and k > SMALL_K:
            need_large = True
            penalize_rows = penalize_rows or bool(recent)
        blob += struct.pack("<fifffffi", cfg.temperature, cfg.top_k, cfg.top_p, cfg.min_p,
                            cfg.repetition_penalty, cfg.presence_penalty, cfg.frequency_penalty,
                            len(recent))
    device = logits.device
    # one upload for the three small arrays: records (32 bytes a row), uniform numbers, recent tokens
    blob += np.asarray(uniforms, dtype=np.float64).tobytes()
    if stride:
        padded = np.full((R, stride), -1, dtype=np.int32)
        for r, row in enumerate(rows):
            padded[r, :len(row)] = row
        blob += padded.tobytes()
    staged = _stage(np.frombuffer(blob, dtype=np.uint8), device)
    params = staged[:32 * R]
    uni = staged[32 * R:40 * R].view(torch.float64)
    recent_dev = staged[40 * R:].view(torch.int32) if stride else None
    out = torch.empty((R,), dtype=torch.int32, device=device)
    keys = probs = None
    vpad = 0
    if need_large:
        vpad = 1
        while vpad < V:
            vpad <<= 1
        keys = torch.empty((R, vpad), dtype=torch.int64, device=device)     # fixed-point masses
    if penalize_rows:
        # rows that are never sorted take their penalties on the logits themselves, over the whole
        # vocabulary and before any cut (src/flyweight/v2.py:1497-1518); on a copy, the caller's
        # logits stay as they are
        logits = logits.clone()
        lib.call("fwb_penalize_rows", ptr(logits), R, V, ptr(params), ptr(recent_dev), stride, stream())
    lib.call("fwb_sample", ptr(logits), R, V, ptr(params), ptr(uni), ptr(recent_dev), stride,
             ptr(out), ptr(keys), ptr(probs), vpad, 1 if need_large else 0, stream())
    return out
