"""CUDA graphs for decode steps.

A decode step (every request brings exactly one token and wants its logits) is the same
sequence of ~100 small kernel launches every time; only the contents of the batch
arrays change.  For each (batch size, block-table width) the runner captures that
sequence once into a CUDA graph over *static* device buffers, and afterwards a step is
one upload of the batch arrays and one graph launch.  (flyweight captures only the dense
feed-forward, seven launches per layer: native/src/v2_runtime.cpp:28797-28830.)

The batch arrays live in one int32 buffer with the same fields as ``StepBatch``.  The
upload goes through a small ring of pinned host buffers guarded by events, because the
host may run several steps ahead of the device.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels.lib import add_launches, launch_count
from .batch import Segment, StepContext

RING = 4


class DecodeBatch:
    """The fields of ``StepBatch`` for B one-token segments, over static buffers."""

    def __init__(self, batch_size: int, n_groups: int, width: int, device):
        B = self.n_segments = self.n_tokens = self.n_logit_rows = batch_size
        self.width = width
        self.n_groups = n_groups
        fields = (("token_ids", B), ("positions", B), ("tok_seg", B), ("seg_start", B + 1),
                  ("seg_slot", B), ("seg_pos0", B), ("logit_rows", B))
        self._offsets = {}
        cursor = 0
        for name, count in fields:
            self._offsets[name] = (cursor, count)
            cursor += count
        self._table_offsets = []
        for _ in range(n_groups):
            self._table_offsets.append(cursor)
            cursor += B * width
        self.size = cursor
        self._dev = torch.zeros(cursor, dtype=torch.int32, device=device)
        self._hosts = [torch.zeros(cursor, dtype=torch.int32).pin_memory() for _ in range(RING)]
        self._events = [None] * RING
        self._turn = 0
        for name, (start, count) in self._offsets.items():
            setattr(self, name, self._dev[start:start + count])
        self.block_tables = [self._dev[start:start + B * width].view(B, width)
                             for start in self._table_offsets]
        self.segments: List[Segment] = []
        self.max_segment = 1
        self.leading_singles = batch_size
        self.max_context = 0
        self.h2d_bytes = cursor * 4
        # host mirror of the arrays; the parts that never change are written once
        import numpy as np
        self._current = np.zeros(cursor, dtype=np.int32)
        for name, count in (("tok_seg", B), ("seg_start", B + 1), ("logit_rows", B)):
            start = self._offsets[name][0]
            self._current[start:start + count] = np.arange(count, dtype=np.int32)
        self._views = tuple(self._current[self._offsets[name][0]:self._offsets[name][0] + B]
                            for name in ("token_ids", "seg_slot", "seg_pos0"))
        self._table_rows = [self._current[start:start + B * width].reshape(B, width)
                            for start in self._table_offsets]
        for rows in self._table_rows:
            rows[:] = -1
        self._stamps = [[None] * B for _ in range(n_groups)]
        self._host_arrays = [host.numpy() for host in self._hosts]

    def upload(self, segments: Sequence[Segment], cache) -> None:
        """Refresh the batch arrays for these one-token segments and send them to the device.
        Block-table rows are rewritten only for requests whose table changed since the last
        step of this batch size (a row grows by one page every 64 tokens)."""
        B = self.n_segments
        values = self._current
        tokens, slots, pos0 = self._views
        for index, seg in enumerate(segments):
            tokens[index] = seg.tokens[0]
            slots[index] = seg.slot
            pos0[index] = seg.pos0
        start = self._offsets["positions"][0]
        values[start:start + B] = pos0
        self.segments = segments
        self.refresh_rows(cache, range(len(segments)))
        turn = self._turn
        self._turn = (turn + 1) % RING
        if self._events[turn] is not None:
            self._events[turn].synchronize()      # the copy that last used this buffer is done
        host = self._hosts[turn]
        self._host_arrays[turn][:] = values
        self._dev.copy_(host, non_blocking=True)
        event = self._events[turn]
        if event is None:
            event = self._events[turn] = torch.cuda.Event()
        event.record()
        self.segments = segments
        self.max_context = int(pos0.max()) + 1


    def refresh_rows(self, cache, indices) -> None:
        """Bring the host copy of the block-table rows of these segments up to date (a row is
        rewritten only if the request's table changed since it was last written here); the next
        upload sends them."""
        for g in range(len(self._table_offsets)):
            group = cache.groups[g]
            rows = self._table_rows[g]
            stamps = self._stamps[g]
            for index in indices:
                request = self.segments[index].request
                table = group.tables[request]
                stamp = (cache.serial(request), len(table),
                         group.window and sum(1 for p in table if p < 0))
                if stamps[index] != stamp:
                    stamps[index] = stamp
                    row = rows[index]
                    row[:len(table)] = table
                    row[len(table):] = -1

    def upload_next(self, tokens: Optional[Sequence[int]]) -> None:
        """The same requests one position further (no page changes): only the token ids and the
        positions move.  ``tokens`` None: the ids are put into ``token_ids`` on the device by the
        caller, after this upload."""
        B = self.n_segments
        values = self._current
        ids, _, pos0 = self._views
        if tokens is not None:
            ids[:] = tokens
        pos0 += 1
        start = self._offsets["positions"][0]
        values[start:start + B] = pos0
        for seg in self.segments:
            seg.pos0 += 1
        turn = self._turn
        self._turn = (turn + 1) % RING
        if self._events[turn] is not None:
            self._events[turn].synchronize()
        self._host_arrays[turn][:] = values
        self._dev.copy_(self._hosts[turn], non_blocking=True)
        event = self._events[turn]
        if event is None:
            event = self._events[turn] = torch.cuda.Event()
        event.record()
        self.max_context += 1


class DecodeGraph:
    def __init__(self, model, caches, precision, device, bad_token_flag, batch_size: int,
                 n_groups: int, width: int):
        self.model = model
        self.caches = caches
        self.batch = DecodeBatch(batch_size, n_groups, width, device)
        self.ctx = StepContext(self.batch, precision, device, bad_token_flag)
        self.graph = None
        self.logits = None
        self.kernels = 0

    def run(self, segments, cache, patch_source=None, patch=None) -> torch.Tensor:
        """The step for these segments.  The first call runs the kernels directly and then
        records the graph; later calls replay it.  The returned logits are a static buffer:
        they are overwritten by the next step of the same batch size.  ``patch``: (segment index,
        row of ``patch_source``) pairs whose token ids are still on the device."""
        self.batch.upload(segments, cache)
        if patch:
            from .batch import patch_from_device
            patch_from_device(self.batch.token_ids, [index for index, _ in patch], patch_source,
                              [row for _, row in patch], self.batch._dev.device)
        if self.graph is None:
            logits = self.model.forward(self.ctx, self.caches)
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            before = launch_count()
            with torch.cuda.graph(graph):
                self.logits = self.model.forward(self.ctx, self.caches)
            self.kernels = launch_count() - before     # recorded, not run
            add_launches(-self.kernels)
            self.graph = graph
            return logits
        self.graph.replay()
        add_launches(self.kernels)
        return self.logits

    def run_next(self, tokens: Optional[Sequence[int]] = None,
                 device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Replay for the same requests, each one token further; the tokens come from the host
        or, as int32 on the device, straight from the sampler of the step before."""
        self.batch.upload_next(tokens)
        if device_tokens is not None:
            self.batch.token_ids.copy_(device_tokens)
        self.graph.replay()
        add_launches(self.kernels)
        return self.logits
