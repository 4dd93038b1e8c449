"""The batch of one step: portions of prompts beside single decoded tokens, flattened.

A *segment* is a run of consecutive tokens of one request that this step processes,
starting at position ``pos0`` (the number of that request's tokens already in the
cache).  All segments of a step are laid end to end into one token axis; kernels find
their way with a handful of int32 arrays that are uploaded in a single copy:

    token_ids[T]  positions[T]  tok_seg[T]      per token
    seg_start[S+1]  seg_slot[S]  seg_pos0[S]    per segment
    logit_rows[R]                               token indices whose logits are wanted
    block_tables[g][S][W]                       page ids per page group, -1 = unmapped
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class Segment:
    request: Hashable
    slot: int
    pos0: int
    tokens: List[int]
    want: List[int] = field(default_factory=list)     # indices into ``tokens``


class _PinnedStaging:
    """A small ring of pinned host buffers for the step's int32 arrays.  Page-locking memory is a
    system call that costs more than the whole upload, so the buffers are kept and grown; an
    event per buffer says when the copy that last read it has finished."""

    def __init__(self, slots: int = 4):
        self._buffers = [None] * slots
        self._events = [None] * slots
        self._turn = 0

    def upload(self, values: np.ndarray, device) -> torch.Tensor:
        turn = self._turn
        self._turn = (turn + 1) % len(self._buffers)
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        buffer = self._buffers[turn]
        if buffer is None or buffer.numel() < values.size:
            buffer = self._buffers[turn] = torch.empty(max(4096, 2 * values.size), dtype=torch.int32).pin_memory()
        host = buffer[:values.size]
        host.numpy()[:] = values
        dev = host.to(device, non_blocking=True)
        if self._events[turn] is None:
            self._events[turn] = torch.cuda.Event()
        self._events[turn].record()
        return dev


_staging = {}


def _to_device(values: np.ndarray, device, pinned: bool) -> torch.Tensor:
    if device is None or torch.device(device).type != "cuda":
        return torch.from_numpy(values.copy())
    if not pinned:
        return torch.from_numpy(values.copy()).to(device)
    key = str(device)
    if key not in _staging:
        _staging[key] = _PinnedStaging()
    return _staging[key].upload(values, device)


def patch_from_device(token_ids: torch.Tensor, places: Sequence[int], source: torch.Tensor,
                      rows: Sequence[int], device) -> None:
    """Put ``source[rows[i]]`` into ``token_ids[places[i]]`` on the device; the two small index
    arrays go up through the pinned staging ring, so the host does not wait."""
    from ..kernels import ops
    n = len(places)
    if n == 0:
        return
    both = _to_device(np.asarray(list(places) + list(rows), dtype=np.int32), device, True)
    ops.patch_tokens_(token_ids, both[:n], source, both[n:])


class StepBatch:
    def __init__(self, segments: Sequence[Segment], block_tables_host: Sequence[List[List[int]]],
                 device, pinned: bool = True):
        self.segments = list(segments)
        self.n_segments = S = len(self.segments)
        lengths = [len(seg.tokens) for seg in self.segments]
        self.n_tokens = T = sum(lengths)
        wanted = sum(len(seg.want) for seg in self.segments)
        self.n_logit_rows = R = wanted
        offsets = {}
        cursor = 0
        for name, count in (("token_ids", T), ("positions", T), ("tok_seg", T),
                            ("seg_start", S + 1), ("seg_slot", S), ("seg_pos0", S),
                            ("logit_rows", R)):
            offsets[name] = (cursor, count)
            cursor += count
        table_slices = []
        for rows in block_tables_host:
            width = len(rows[0]) if len(rows) else 1
            table_slices.append((cursor, S, width))
            cursor += S * width
        flat = np.empty(cursor, dtype=np.int32)
        ids, positions, tok_seg = (flat[offsets[name][0]:offsets[name][0] + T]
                                   for name in ("token_ids", "positions", "tok_seg"))
        seg_start = flat[offsets["seg_start"][0]:offsets["seg_start"][0] + S + 1]
        logit_rows = flat[offsets["logit_rows"][0]:offsets["logit_rows"][0] + R]
        seg_start[0] = 0
        base = row = 0
        for index, (seg, n) in enumerate(zip(self.segments, lengths)):
            if n == 1:
                ids[base] = seg.tokens[0]
                positions[base] = seg.pos0
                tok_seg[base] = index
            else:
                ids[base:base + n] = seg.tokens
                positions[base:base + n] = np.arange(seg.pos0, seg.pos0 + n, dtype=np.int32)
                tok_seg[base:base + n] = index
            for w in seg.want:
                logit_rows[row] = base + w
                row += 1
            base += n
            seg_start[index + 1] = base
        start = offsets["seg_slot"][0]
        flat[start:start + S] = [seg.slot for seg in self.segments]
        start = offsets["seg_pos0"][0]
        flat[start:start + S] = [seg.pos0 for seg in self.segments]
        for (start, s, w), rows in zip(table_slices, block_tables_host):
            if s:
                flat[start:start + s * w] = np.asarray(rows, dtype=np.int32).reshape(-1)
        self.seg_start_host = seg_start.copy()
        self.h2d_bytes = flat.size * 4
        dev = _to_device(flat, device, pinned)
        self._dev = dev
        for name, (start, count) in offsets.items():
            setattr(self, name, dev[start:start + count])
        self.block_tables = [dev[start:start + s * w].view(s, w) for start, s, w in table_slices]
        self.max_context = max((seg.pos0 + n for seg, n in zip(self.segments, lengths)), default=0)
        self.max_segment = max(lengths, default=0)
        # segments of one token at the head of the batch (the scheduler puts decoding requests first)
        self.leading_singles = next((i for i, n in enumerate(lengths) if n != 1), S)
        self._device = device
        self._pinned = pinned
        self._tiles = {}

    def attention_tiles(self, tokens_per_tile: int, first_segment: int = 0):
        """Row tiles for the tiled attention kernels: every segment from ``first_segment`` on cut
        into runs of at most ``tokens_per_tile`` tokens.  Returns (tile_seg, tile_tok0, n_tiles),
        int32 on the device; made once per step, tile size and first segment."""
        cached = self._tiles.get((tokens_per_tile, first_segment))
        if cached is None:
            seg_of, tok0 = [], []
            base = 0
            for index, seg in enumerate(self.segments):
                n = len(seg.tokens)
                if index >= first_segment:
                    starts = np.arange(base, base + n, tokens_per_tile, dtype=np.int32)
                    seg_of.append(np.full(starts.size, index, dtype=np.int32))
                    tok0.append(starts)
                base += n
            seg_of = np.concatenate(seg_of) if seg_of else np.empty(0, dtype=np.int32)
            n = seg_of.size
            host = np.concatenate([seg_of] + tok0) if n else np.empty(0, dtype=np.int32)
            self.h2d_bytes += host.size * 4
            dev = _to_device(host, self._device, self._pinned)
            cached = self._tiles[(tokens_per_tile, first_segment)] = (dev[:n], dev[n:], n)
        return cached


@dataclass
class StepContext:
    """What the parts see of the running step."""
    batch: StepBatch
    precision: object
    device: object
    bad_token_flag: Optional[torch.Tensor] = None
