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

import torch


@dataclass
class Segment:
    request: Hashable
    slot: int
    pos0: int
    tokens: List[int]
    want: List[int] = field(default_factory=list)     # indices into ``tokens``


class StepBatch:
    def __init__(self, segments: Sequence[Segment], block_tables_host: Sequence[List[List[int]]],
                 device, pinned: bool = True):
        self.segments = list(segments)
        self.n_segments = S = len(self.segments)
        token_ids: List[int] = []
        positions: List[int] = []
        tok_seg: List[int] = []
        seg_start = [0]
        logit_rows: List[int] = []
        for index, seg in enumerate(self.segments):
            base = len(token_ids)
            token_ids.extend(seg.tokens)
            positions.extend(range(seg.pos0, seg.pos0 + len(seg.tokens)))
            tok_seg.extend([index] * len(seg.tokens))
            seg_start.append(base + len(seg.tokens))
            logit_rows.extend(base + w for w in seg.want)
        self.n_tokens = T = len(token_ids)
        self.n_logit_rows = R = len(logit_rows)
        seg_slot = [seg.slot for seg in self.segments]
        seg_pos0 = [seg.pos0 for seg in self.segments]
        flat = token_ids + positions + tok_seg + seg_start + seg_slot + seg_pos0 + logit_rows
        offsets = {}
        cursor = 0
        for name, count in (("token_ids", T), ("positions", T), ("tok_seg", T),
                            ("seg_start", S + 1), ("seg_slot", S), ("seg_pos0", S),
                            ("logit_rows", R)):
            offsets[name] = (cursor, count)
            cursor += count
        table_slices = []
        for rows in block_tables_host:
            width = len(rows[0]) if rows else 1
            table_slices.append((cursor, S, width))
            for row in rows:
                flat.extend(row)
            cursor += S * width
        host = torch.tensor(flat, dtype=torch.int32)
        self.h2d_bytes = host.numel() * 4
        if device is not None and torch.device(device).type == "cuda":
            if pinned:
                host = host.pin_memory()
            dev = host.to(device, non_blocking=True)
        else:
            dev = host
        self._host = host
        self._dev = dev
        for name, (start, count) in offsets.items():
            setattr(self, name, dev[start:start + count])
        self.block_tables = [dev[start:start + s * w].view(s, w) for start, s, w in table_slices]
        self.max_context = max((seg.pos0 + len(seg.tokens) for seg in self.segments), default=0)
        self.max_segment = max((len(seg.tokens) for seg in self.segments), default=0)
        self._device = device
        self._tiles = {}

    def attention_tiles(self, tokens_per_tile: int):
        """Row tiles for the tiled attention kernel: every segment cut into runs of at most
        ``tokens_per_tile`` tokens.  Returns (tile_seg, tile_tok0, n_tiles), int32 on the
        device; made once per step and tile size."""
        cached = self._tiles.get(tokens_per_tile)
        if cached is None:
            seg_of, tok0 = [], []
            base = 0
            for index, seg in enumerate(self.segments):
                for start in range(0, len(seg.tokens), tokens_per_tile):
                    seg_of.append(index)
                    tok0.append(base + start)
                base += len(seg.tokens)
            host = torch.tensor(seg_of + tok0, dtype=torch.int32)
            self.h2d_bytes += host.numel() * 4
            if self._device is not None and torch.device(self._device).type == "cuda":
                dev = host.pin_memory().to(self._device, non_blocking=True)
            else:
                dev = host
            n = len(seg_of)
            cached = self._tiles[tokens_per_tile] = (dev[:n], dev[n:], n)
        return cached


@dataclass
class StepContext:
    """What the parts see of the running step."""
    batch: StepBatch
    precision: object
    device: object
    bad_token_flag: Optional[torch.Tensor] = None
