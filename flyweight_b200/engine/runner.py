"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step`` takes entries ``(request, tokens, want)``: a request's next tokens
(a portion of its prompt, cut anywhere, or one decoded token) and the places among them
whose logits are wanted.  It runs only those tokens, as one batch, from the cache that
earlier steps left, writes their keys, values and state into the cache, and returns the
logits at the wanted places, ``[wanted][vocab]`` fp32, in the order of the entries.

flyweight has two forwards instead, one token of one sequence
(native/src/v2_runtime.cpp:27525) or a chunk of one sequence
(native/src/v2_mtp_verifier.inc:296), and interleaves requests between forwards
(native/src/v2_runtime.cpp:33695-33972); here requests share every kernel launch.
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import lib as kernel_lib

from ..cache.manager import PAGE_SIZE, CacheManager, OutOfPages, OutOfSlots
from ..kernels.lib import require_cuda
from .batch import Segment, StepBatch, StepContext, patch_from_device
from .graphs import DecodeGraph
from .plan import build_plan

Entry = Tuple[Hashable, Sequence[int], Sequence[int]]


class StepError(ValueError):
    """An entry the step function refuses (bad token id, empty portion, over-long request).
    ``request`` names the entry at fault when there is one (None: the step as a whole)."""

    def __init__(self, message: str, request: Hashable = None):
        super().__init__(message)
        self.request = request


def _token_array(request, tokens):
    """The entry's token ids as one int64 array (a prompt portion is thousands of them: no
    Python loop over tokens anywhere on the way to the device); a single decoded token stays
    a list of one int, which costs less than an array."""
    if len(tokens) == 1 and not isinstance(tokens, np.ndarray):
        try:
            return [int(tokens[0])]
        except (TypeError, ValueError) as error:
            raise StepError(f"request {request!r}: token ids must be integers ({error})", request) from None
    try:
        array = np.asarray(tokens, dtype=np.int64)
    except (OverflowError, TypeError, ValueError) as error:
        raise StepError(f"request {request!r}: token ids must be integers ({error})", request) from None
    if array.ndim != 1:
        raise StepError(f"request {request!r}: tokens must be a flat list of ids", request)
    return array


class StepPlanner:
    """The host side of a step: checks, admission to the cache, page mapping.  It needs
    no device, so schedulers and cache logic can be tested against it on the CPU."""

    def __init__(self, cache: CacheManager, vocab_size: int, max_model_len: int,
                 max_batched_tokens: int):
        self.cache = cache
        self.vocab_size = int(vocab_size)
        self.max_model_len = int(max_model_len)
        self.max_batched_tokens = int(max_batched_tokens)

    # ------------------------------------------------------------------ checks
    def _check_entries(self, entries: Sequence[Entry]) -> None:
        vocab = self.vocab_size
        seen = set()
        total = 0
        for request, tokens, want in entries:
            if request in seen:
                raise StepError(f"request {request!r} appears twice in one step", request)
            seen.add(request)
            if len(tokens) == 0:
                raise StepError(f"request {request!r} brings no tokens", request)
            if len(tokens) == 1:
                low = high = int(tokens[0])
            else:
                low, high = int(tokens.min()), int(tokens.max())
            if low < 0 or high >= vocab:                                 # native/src/v2_runtime.cpp:27530
                token = next(int(t) for t in tokens if not 0 <= int(t) < vocab)
                raise StepError(f"token id {token} of request {request!r} is outside "
                                f"[0, {vocab})", request)
            for place in want:
                if not 0 <= int(place) < len(tokens):
                    raise StepError(f"request {request!r} wants logits at place {place} of "
                                    f"{len(tokens)} tokens", request)
            have = self.cache.length(request) if self.cache.has(request) else 0
            if have + len(tokens) > self.max_model_len:
                raise StepError(f"request {request!r} would reach {have + len(tokens)} tokens, "
                                f"beyond max_model_len {self.max_model_len}", request)
            total += len(tokens)
        if total > self.max_batched_tokens:
            raise StepError(f"step of {total} tokens exceeds max_batched_tokens "
                            f"{self.max_batched_tokens}")

    def pages_short(self, entries: Sequence[Entry]) -> int:
        """Pages lacking for this step over all groups (0: it fits).  Pages that a window
        has passed are given back first."""
        cache = self.cache
        needs = [0] * len(cache.groups)
        for request, tokens, _ in entries:
            try:
                if len(tokens) == 1 and cache.has(request) and cache.fits_last_page(request):
                    continue                        # a decoding request inside its last page
                have = 0
                if cache.has(request):
                    cache.release_passed(request)
                    have = cache.length(request)
                for g, need in enumerate(cache.pages_needed(request, have + len(tokens))):
                    needs[g] += need
            except Exception as error:
                if getattr(error, "request", None) is None:
                    error.request = request         # whose bookkeeping failed: it alone is given up
                raise
        return sum(max(0, need - group.pool.n_free) for need, group in zip(needs, cache.groups))

    # ------------------------------------------------------------------ planning
    def plan(self, entries: Sequence[Entry], pages_checked: bool = False,
             own_entries: bool = False) -> List[Segment]:
        """Check the entries, admit new requests, map their pages; all or nothing: if a
        slot or a page is lacking, nothing has changed when the error is raised.
        ``pages_checked``: the caller (the scheduler) has just asked ``pages_short`` for exactly
        these entries and got 0.  ``own_entries``: the entries were built by the engine's own
        scheduler from token ids that were checked when the request was submitted or that its
        sampler drew (each request once, ids inside the vocabulary, lengths inside the limits), so
        the checks of what a caller from outside may hand in are not repeated on every step."""
        cache = self.cache
        if own_entries:
            vocab = self.vocab_size
            checked, total = [], 0
            for request, tokens, want in entries:
                if len(tokens) == 1:
                    low = high = tokens[0]
                else:
                    tokens = _token_array(request, tokens)
                    low, high = int(tokens.min()), int(tokens.max())
                if low < 0 or high >= vocab:        # a text damaged after it was submitted: that request alone
                    raise StepError(f"a token id of request {request!r} is outside [0, {vocab})", request)
                total += len(tokens)
                checked.append((request, tokens, want))
            entries = checked
            if total > self.max_batched_tokens:
                raise StepError(f"step of {total} tokens exceeds max_batched_tokens {self.max_batched_tokens}")
        else:
            entries = [(r, _token_array(r, toks), [int(w) for w in want]) for r, toks, want in entries]
            self._check_entries(entries)
        new = 0
        for entry in entries:
            if not cache.has(entry[0]):
                new += 1
        if new > cache.free_slots:
            raise OutOfSlots(f"{new} new requests but {cache.free_slots} free state slots")
        short = 0 if pages_checked else self.pages_short(entries)
        if short:
            raise OutOfPages(f"this step needs {short} more cache pages than are free")
        segments: List[Segment] = []
        for request, tokens, want in entries:
            if new and not cache.has(request):
                cache.admit(request)
            slot, pos0 = cache.grow(request, len(tokens))
            segments.append(Segment(request, slot, pos0, tokens, want))
        return segments

    def finish(self, request: Hashable) -> None:
        """The request is over: its pages and its state slot go back to the pools."""
        if self.cache.has(request):
            self.cache.release(request)


class ModelRunner(StepPlanner):
    def __init__(self, model, num_pages: int, num_slots: int, max_model_len: int,
                 max_batched_tokens: int = 8192, use_graphs: bool = True, use_plan: bool = True,
                 graph_after: int = 0):
        require_cuda()
        self.model = model
        self.precision = model.precision
        self.device = model.device
        if torch.device(self.device).type == "cuda":
            kernel_lib.use_device(self.device)
        if int(max_model_len) > model.spec.max_positions:
            raise StepError(f"max_model_len {max_model_len} exceeds the model's "
                            f"{model.spec.max_positions} positions")
        model.prepare(int(max_model_len))
        cache = CacheManager(model.state_specs(), num_pages, num_slots,
                             cache_dtype=self.precision.cache_dtype, device=self.device)
        super().__init__(cache, model.spec.vocab_size, max_model_len, max_batched_tokens)
        self.bad_token_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        # the forward pass of a step as one native call, when every part of the model has that form
        self.use_plan = bool(use_plan)
        self.step_plan = build_plan(model, cache.layer_caches, self.max_batched_tokens, self.max_batched_tokens,
                               num_slots, len(cache.groups), self.bad_token_flag) if use_plan else None
        # decode steps replay a CUDA graph per (batch size, block-table width)
        self.use_graphs = bool(use_graphs) and model.graph_safe
        self.max_graph_batch = 256
        # A graph for a (batch size, table width) is recorded only once that many decode steps in a
        # row have had this shape: recording costs 8 to 30 ms, ten to thirty steps, and pays only
        # while the same requests go on decoding together.  0: at the first step of a shape.
        self.graph_after = int(graph_after)
        self._shape_run = (None, 0)         # the shape of the last decode steps and how many in a row
        self.max_graphs = 32                # graphs kept; the one unused for longest goes first
        self._graphs = {}
        self.last_decode_graph = None      # the graph the last step replayed (None: it ran eagerly)
        self.graph_replays = 0
        self.graphs_recorded = 0
        self.steps = 0
        self.tokens_run = 0
        self.h2d_bytes = 0

    def step(self, entries: Sequence[Entry], pages_checked: bool = False,
             patch_source: Optional[torch.Tensor] = None, patch: Optional[Sequence] = None,
             own_entries: bool = False) -> torch.Tensor:
        """``pages_checked``, ``own_entries``: see ``plan``.  ``patch``: (entry index, row of ``patch_source``) pairs.  The last token of those entries
        was sampled by the step before and has not been read by the host (the entry carries a
        placeholder id); its value is taken from ``patch_source`` (int32, on the device) there."""
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        segments = self.plan(entries, pages_checked, own_entries)
        requests = [seg.request for seg in segments]
        width = self.cache.max_table_len(requests)
        n_groups = len(self.cache.groups)
        if (self.use_graphs and len(segments) <= self.max_graph_batch
                and all(len(seg.tokens) == 1 and seg.want == [0] for seg in segments)):
            bucket = 16 * (-(-width // 16))         # a new graph every 1,024 tokens of context
            key = (len(segments), bucket)
            seen = self._shape_run[1] + 1 if self._shape_run[0] == key else 1
            self._shape_run = (key, seen)
            graph = self._graphs.pop(key, None)
            if graph is None and seen <= self.graph_after:
                return self._step_without_graph(segments, requests, width, n_groups, patch_source, patch)
            if graph is not None:
                self._graphs[key] = graph              # most recently used: last in the dict
            if graph is None:
                # every graph keeps activations and a [batch][vocab] logits buffer of its own: a
                # runtime whose batch sizes and contexts wander would otherwise grow without bound
                while len(self._graphs) >= self.max_graphs:
                    oldest = next(iter(self._graphs))
                    if self._graphs[oldest] is self.last_decode_graph:
                        self.last_decode_graph = None
                    del self._graphs[oldest]
                graph = self._graphs[key] = DecodeGraph(
                    self.model, self.cache.layer_caches, self.precision, self.device,
                    self.bad_token_flag, len(segments), n_groups, bucket)
                self.graphs_recorded += 1
            else:
                self.graph_replays += 1
            logits = graph.run(segments, self.cache, patch_source, patch)
            self.last_decode_graph = graph
            self.steps += 1
            self.tokens_run += len(segments)
            self.h2d_bytes += graph.batch.h2d_bytes
            return logits
        self._shape_run = (None, 0)
        return self._step_without_graph(segments, requests, width, n_groups, patch_source, patch)

    def _step_without_graph(self, segments, requests, width, n_groups, patch_source, patch) -> torch.Tensor:
        self.last_decode_graph = None
        tables = [self.cache.block_table_array(g, requests, width) for g in range(n_groups)]
        if self.step_plan is not None and self.use_plan:
            logits = self.step_plan.run(segments, tables, patch_source, patch)
            self.steps += 1
            self.tokens_run += self.step_plan._step.T
            self.h2d_bytes += self.step_plan.h2d_bytes
            return logits
        batch = StepBatch(segments, tables, self.device)
        if patch:
            patch_from_device(batch.token_ids, [int(batch.seg_start_host[index + 1]) - 1 for index, _ in patch],
                              patch_source, [row for _, row in patch], self.device)
        ctx = StepContext(batch, self.precision, self.device, self.bad_token_flag)
        logits = self.model.forward(ctx, self.cache.layer_caches)
        self.steps += 1
        self.tokens_run += batch.n_tokens
        self.h2d_bytes += batch.h2d_bytes
        return logits

    def check_health(self) -> None:
        """Raise if a kernel recorded a failure since the last check: a bounded wait inside a
        tensor-core kernel that gave up (the results of its step are not to be trusted), or a
        token id outside the vocabulary that reached the embedding.  Reads two words from the
        device, so it waits for the work queued so far."""
        from ..kernels import KernelError, tensorcore
        code = tensorcore.status()
        if code:
            raise KernelError(f"a tensor-core kernel gave up waiting on a barrier (code {code}); "
                              "the logits of that step are not valid")
        if int(self.bad_token_flag.item()):
            self.bad_token_flag.zero_()
            raise KernelError("a token id outside the vocabulary reached the embedding kernel")

    def step_same_requests(self, tokens: Optional[Sequence[int]] = None,
                           device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The decode step that follows the last one for exactly the same requests: lengths grow by
        one (a request at a page's edge gets its next page, pages that a window has passed go back:
        the caller has asked ``cache.room_for_one_more``), the captured graph is replayed.  The tokens are given by the
        host, or on the device (int32, one per request, in the batch's order)."""
        graph = self.last_decode_graph
        cache = self.cache
        advance = cache.advance_one
        changed = [index for index, seg in enumerate(graph.batch.segments) if advance(seg.request)]
        if changed:
            graph.batch.refresh_rows(cache, changed)
        logits = graph.run_next(tokens, device_tokens)
        self.graph_replays += 1
        self.steps += 1
        self.tokens_run += graph.batch.n_segments
        self.h2d_bytes += graph.batch.h2d_bytes
        return logits
