"""The native step plan: the forward pass of a step as one call into the compiled library.

``build_plan`` asks every part of the model, in schedule order, to add its operations to a
``PlanBuilder`` (``part.plan(builder, ...)``, the symbolic twin of its ``forward``).  The
builder hands out buffers from one arena (sized for the engine's token budget, reused as soon
as a buffer's last reader has been added) and records the operations; ``finish`` allocates the
arena and passes operations and device pointers to the library once.  ``StepPlan.run`` then
packs a step's int32 arrays into one block of host memory and makes one native call, which
uploads the block and launches every kernel of the step (``csrc/plan.cu``).

A model is plannable when all its parts are (a part defined outside the package has no
``plan`` and leaves its model on the Python path, launch by launch) and all its matrices have
the precision's own dtype.  Kernel choices that depend on the size of the step are made inside
the library, per step, by the same rules as the Python dispatch; ``tests/test_plan_gpu.py``
compares the two paths bit for bit.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import attention as attention_kernels
from ..kernels import lib as kernel_lib
from ..kernels.lib import KernelError
from ..kernels.ops import ROPE_PAIRINGS
from .batch import Segment

EPI_F32, EPI_ACT, EPI_SWIGLU = 0, 1, 3
MAX_GROUPS = 8
META_NAMES = ("token_ids", "positions", "tok_seg", "seg_start", "seg_slot", "seg_pos0", "logit_rows",
              "tile_seg_a", "tile_tok0_a", "tile_seg_b", "tile_tok0_b", "patch_dst", "patch_src")
META_COUNT = len(META_NAMES) + MAX_GROUPS


class NotPlannable(Exception):
    """A part (or a combination of dtypes or shapes) the native plan has no operation for; the
    model then runs through the parts' ``forward``, launch by launch."""


class FwbStep(ctypes.Structure):
    """``struct FwbStep`` of csrc/plan.cu."""
    _fields_ = [("meta_host", ctypes.c_void_p), ("meta_dev", ctypes.c_void_p),
                ("meta_words", ctypes.c_int), ("upload", ctypes.c_int),
                ("offsets", ctypes.c_int * META_COUNT),
                ("T", ctypes.c_int), ("S", ctypes.c_int), ("R", ctypes.c_int),
                ("width", ctypes.c_int * MAX_GROUPS),
                ("max_segment", ctypes.c_int), ("leading_singles", ctypes.c_int),
                ("tokens_per_tile", ctypes.c_int * 2), ("n_tiles", ctypes.c_int * 2),
                ("logits", ctypes.c_void_p), ("patch_source", ctypes.c_void_p), ("n_patch", ctypes.c_int)]


class Buf:
    """A buffer of the arena: ``rows`` x ``width`` elements of ``dtype`` at ``offset`` bytes."""
    __slots__ = ("offset", "nbytes", "width", "dtype")

    def __init__(self, offset, nbytes, width, dtype):
        self.offset, self.nbytes, self.width, self.dtype = offset, nbytes, width, dtype


class _Arena:
    """First-fit allocation of byte ranges with reuse; only the high-water mark is allocated."""
    ALIGN = 256

    def __init__(self):
        self.free: List[List[int]] = []          # [offset, size], sorted by offset
        self.top = 0

    def take(self, nbytes: int) -> int:
        nbytes = -(-max(nbytes, 1) // self.ALIGN) * self.ALIGN
        for block in self.free:
            if block[1] >= nbytes:
                offset = block[0]
                block[0] += nbytes
                block[1] -= nbytes
                if block[1] == 0:
                    self.free.remove(block)
                return offset
        if self.free and self.free[-1][0] + self.free[-1][1] == self.top:      # grow the last block
            offset = self.free[-1][0]
            self.top = offset + nbytes
            self.free.pop()
            return offset
        offset = self.top
        self.top += nbytes
        return offset

    def give(self, offset: int, nbytes: int) -> None:
        nbytes = -(-max(nbytes, 1) // self.ALIGN) * self.ALIGN
        self.free.append([offset, nbytes])
        self.free.sort()
        merged: List[List[int]] = []
        for block in self.free:
            if merged and merged[-1][0] + merged[-1][1] == block[0]:
                merged[-1][1] += block[1]
            else:
                merged.append(block)
        self.free = merged


class PlanBuilder:
    """What the parts see while a plan is built.  ``x`` is the fp32 residual stream [tokens][H];
    every other buffer is taken with ``tokens``/``rows`` and given back with ``free`` when the last
    operation that reads it has been added."""

    def __init__(self, precision, device, hidden: int, max_tokens: int, max_rows: int, num_slots: int,
                 bad_flag: torch.Tensor):
        self.precision = precision
        self.device = torch.device(device)
        self.act_dtype = precision.act_dtype
        self.act_bf16 = 1 if self.act_dtype == torch.bfloat16 else 0
        self.hidden = int(hidden)
        self.max_tokens, self.max_rows, self.num_slots = int(max_tokens), int(max_rows), int(num_slots)
        self.bad_flag = bad_flag
        self._arena = _Arena()
        self._ops = []                      # (launcher name, argument tuple with Buf placeholders)
        self._keep = []                     # tensors the plan's pointers refer to
        self.group_sizes = set()            # query heads per KV head of the attention operations
        self.x = self.tokens(hidden, torch.float32)
        self.delta = self.tokens(hidden, torch.float32)

    # ------------------------------------------------------------------ buffers
    def _take(self, rows: int, width: int, dtype) -> Buf:
        nbytes = rows * width * torch.empty((), dtype=dtype).element_size()
        return Buf(self._arena.take(nbytes), nbytes, width, dtype)

    def tokens(self, width: int, dtype) -> Buf:
        return self._take(self.max_tokens, width, dtype)

    def rows(self, width: int, dtype) -> Buf:
        return self._take(self.max_rows, width, dtype)

    def sized(self, nbytes: int) -> Buf:
        return Buf(self._arena.take(nbytes), nbytes, nbytes, torch.uint8)

    def free(self, buf: Optional[Buf]) -> None:
        if buf is not None:
            self._arena.give(buf.offset, buf.nbytes)

    def matrix(self, w: torch.Tensor, what: str) -> int:
        """1 if ``w`` is bfloat16, 0 if fp32; the plan takes matrices in the precision's own dtype."""
        if w.dtype != (torch.bfloat16 if self.act_bf16 else torch.float32):
            raise NotPlannable(f"{what} is stored as {w.dtype} in a {self.precision.name} model")
        if not w.is_contiguous() or not w.is_cuda:
            raise NotPlannable(f"{what} is not a contiguous tensor on {self.device}")
        self._keep.append(w)
        return 1 if w.dtype == torch.bfloat16 else 0

    def _vector(self, v: Optional[torch.Tensor]):
        if v is None:
            return None
        if v.dtype != torch.float32 or not v.is_contiguous():
            raise NotPlannable("a vector that is not contiguous fp32")
        self._keep.append(v)
        return v

    # ------------------------------------------------------------------ operations
    def embed(self, table: torch.Tensor, vocab: int, scale: float) -> None:
        if not table.is_contiguous():
            raise NotPlannable("the embedding table is not contiguous")
        self._keep.append(table)
        self._ops.append(("fwb_plan_embed", (table, kernel_lib.is_bf16(table), self.x, self.hidden, int(vocab),
                                             ctypes.c_float(scale), self.bad_flag)))

    def norm_linear(self, norm, w: torch.Tensor, epilogue: int, out: Optional[Buf], what: str,
                    on_logit_rows: bool = False) -> None:
        """``out = epilogue(norm(x [+ the pending delta]) @ w.T)``.  ``norm`` is the norm part in
        front of the product (an RMSNorm).  ``epilogue``: EPI_F32, EPI_ACT (the activation dtype) or
        EPI_SWIGLU (w = [gate | up], out [.][F]).  ``out`` None with ``on_logit_rows``: the step's
        logits."""
        params = getattr(norm, "plan_params", lambda: None)()
        if params is None:
            raise NotPlannable(f"norm {norm.kind!r} has no native form")
        weight, eps = params
        w_bf16 = self.matrix(w, what)
        K = w.shape[1]
        N = w.shape[0] // 2 if epilogue == EPI_SWIGLU else w.shape[0]
        if weight.numel() != K:
            raise NotPlannable(f"{what}: the norm has {weight.numel()} weights for {K} columns")
        taker = self.rows if on_logit_rows else self.tokens
        scratch = taker(K, w.dtype)
        scratch2 = taker(2 * N, self.act_dtype) if epilogue == EPI_SWIGLU else None
        native_epilogue = epilogue
        if epilogue == EPI_ACT and not self.act_bf16:
            native_epilogue = EPI_F32
        self._ops.append(("fwb_plan_norm_linear",
                          (self.x, self.delta, self._vector(weight), ctypes.c_float(eps), w, w_bf16, N, K,
                           native_epilogue, 1 if on_logit_rows else 0, out, scratch, scratch2)))
        self.free(scratch)
        self.free(scratch2)

    def linear_residual(self, inp: Buf, w: torch.Tensor, what: str) -> None:
        """``x += inp @ w.T`` (in the epilogue, or through the pending delta)."""
        w_bf16 = self.matrix(w, what)
        if w.shape[0] != self.hidden or w.shape[1] != inp.width:
            raise NotPlannable(f"{what}: shape {tuple(w.shape)} does not map {inp.width} to {self.hidden}")
        self._ops.append(("fwb_plan_linear_residual", (inp, w, w_bf16, w.shape[0], w.shape[1], self.x, self.delta)))

    def shortconv(self, p: Buf, taps, bias, state: torch.Tensor, z: Buf) -> None:
        H, L = taps.shape
        if state.dtype != torch.float32 or tuple(state.shape[1:]) != (H, L - 1) or state.stride(2) != 1 \
                or state.stride(1) != L - 1:
            raise NotPlannable("the conv state is not fp32 [slots][H][L-1] with contiguous slots")
        self._keep.append(state)
        stride = state.stride(0) if state.shape[0] > 1 else H * (L - 1)
        self._ops.append(("fwb_plan_shortconv", (p, self._vector(taps), self._vector(bias), state,
                                                 ctypes.c_longlong(stride), z, H, L)))

    def qk_rope(self, qkv: Buf, q_norm, k_norm, table: torch.Tensor, q_out: Buf, cache, n_heads: int,
                n_kv_in: int, head_dim: int, rotary_dim: int, pairing: str, eps: float) -> None:
        self._keep.append(table)
        k_pool = cache.k_pool if n_kv_in else None
        v_pool = cache.v_pool if n_kv_in else None
        if n_kv_in and k_pool.dtype != self.act_dtype:
            raise NotPlannable("the cache is not in the activation dtype")
        page_size = k_pool.shape[2] if n_kv_in else 0
        self._ops.append(("fwb_plan_qk_rope",
                          (qkv, self._vector(q_norm), self._vector(k_norm), table, q_out, k_pool, v_pool,
                           self._group(cache), page_size, n_heads, n_kv_in, head_dim, rotary_dim,
                           ROPE_PAIRINGS[pairing], ctypes.c_float(eps or 0.0), 1 if q_norm is not None else 0)))

    def attention(self, q: Buf, cache, out: Buf, n_heads: int, window: int, scale: float) -> None:
        k_pool, v_pool = cache.k_pool, cache.v_pool
        num_pages, n_kv, page_size, head_dim = k_pool.shape
        if k_pool.dtype != self.act_dtype:
            raise NotPlannable("the cache is not in the activation dtype")
        self.group_sizes.add(n_heads // n_kv)
        # scratch of the split decode kernel when its slices are merged by a second kernel: only
        # single tokens go there, one per live request at most, in at most 16 slices
        part_o = self.sized(self.num_slots * n_kv * 16 * (n_heads // n_kv) * head_dim * 4)
        part_ml = self.sized(self.num_slots * n_kv * 16 * (n_heads // n_kv) * 2 * 4)
        self._ops.append(("fwb_plan_attention",
                          (q, k_pool, v_pool, out, self._group(cache), page_size, num_pages, n_heads, n_kv,
                           head_dim, int(window), ctypes.c_float(scale), part_o, part_ml)))
        self.free(part_o)
        self.free(part_ml)

    def softcap(self, cap: float, vocab: int) -> None:
        self._ops.append(("fwb_plan_softcap", (ctypes.c_float(cap), int(vocab))))

    @staticmethod
    def _group(cache) -> int:
        if cache.group is None or not 0 <= cache.group < MAX_GROUPS:
            raise NotPlannable(f"page group {cache.group} is beyond the plan's {MAX_GROUPS}")
        return cache.group

    # ------------------------------------------------------------------ the finished plan
    def finish(self, n_groups: int, vocab: int) -> "StepPlan":
        if len(self.group_sizes) > 1:
            raise NotPlannable("attention layers with different numbers of query heads per KV head")
        arena = torch.empty(max(self._arena.top, 256), dtype=torch.uint8, device=self.device)
        base = arena.data_ptr()
        library = kernel_lib.library()
        library.fwb_plan_create.restype = ctypes.c_void_p
        library.fwb_plan_create.argtypes = [ctypes.c_int]
        handle = ctypes.c_void_p(library.fwb_plan_create(self.act_bf16))

        def pointer(value):
            if isinstance(value, Buf):
                return base + value.offset
            if isinstance(value, torch.Tensor):
                return value.data_ptr()
            return value

        for name, args in self._ops:
            function = getattr(library, name)
            status = function(handle, *(pointer(a) for a in args))
            if status != 0:
                library.fwb_plan_destroy(handle)
                raise KernelError(f"{name} refused its arguments while the plan was built (status {status})")
        group = next(iter(self.group_sizes), 1)
        return StepPlan(handle, arena, self._keep, self.device, n_groups, vocab, group, self.max_tokens,
                        self.max_rows, len(self._ops))


class StepPlan:
    """A built plan.  ``run`` executes one step: segments in, fp32 logits [wanted][vocab] out."""

    def __init__(self, handle, arena, keep, device, n_groups, vocab, group, max_tokens, max_rows, n_ops):
        self._handle = handle
        self._arena = arena
        self._keep = keep
        self.device = device
        self.n_groups = n_groups
        self.vocab = vocab
        self.tokens_per_tile = (max(1, 128 // group), max(1, 64 // group))
        self.max_tokens, self.max_rows = max_tokens, max_rows
        self.n_ops = n_ops
        self._library = kernel_lib.library()
        self._run = self._library.fwb_plan_run
        self._step = FwbStep()
        self._step.tokens_per_tile[0], self._step.tokens_per_tile[1] = self.tokens_per_tile
        self._launches = ctypes.c_int(0)
        self._meta_dev = torch.empty(1 << 16, dtype=torch.int32, device=device)
        self._host = np.empty(1 << 16, dtype=np.int32)
        self.h2d_bytes = 0

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                self._library.fwb_plan_destroy(handle)
            except Exception:
                pass

    @property
    def arena_bytes(self) -> int:
        return self._arena.numel()

    def pack(self, segments: Sequence[Segment], tables_host: Sequence[np.ndarray],
             patch: Optional[Sequence] = None) -> FwbStep:
        """The step's int32 arrays, one after the other in one block of host memory, and the
        counts the library needs; returns the filled ``FwbStep`` (reused from step to step)."""
        step = self._step
        S = len(segments)
        lengths = [len(seg.tokens) for seg in segments]
        T = sum(lengths)
        R = sum(len(seg.want) for seg in segments)
        leading = next((i for i, n in enumerate(lengths) if n != 1), S)
        max_segment = max(lengths)
        # tiles of the two prompt attention kernels: every segment from `first` on cut into runs
        first = leading if (max_segment > 1 and attention_kernels.heads_the_decode_kernel()) else 0
        tiles = []
        if max_segment > 1 or attention_kernels.tiled_forced():
            for per_tile in self.tokens_per_tile:
                seg_of, tok0 = [], []
                base = 0
                for index, n in enumerate(lengths):
                    if index >= first:
                        starts = np.arange(base, base + n, per_tile, dtype=np.int32)
                        seg_of.append(np.full(starts.size, index, dtype=np.int32))
                        tok0.append(starts)
                    base += n
                tiles.append((np.concatenate(seg_of), np.concatenate(tok0)))
        else:
            empty = np.empty(0, dtype=np.int32)
            tiles = [(empty, empty), (empty, empty)]
        n_patch = len(patch) if patch else 0
        counts = [T, T, T, S + 1, S, S, R, tiles[0][0].size, tiles[0][0].size, tiles[1][0].size, tiles[1][0].size,
                  n_patch, n_patch]
        widths = [int(rows.shape[1]) if rows.ndim == 2 and rows.shape[0] else 1 for rows in tables_host]
        counts += [S * w for w in widths]
        words = sum(counts)
        if words > self._host.size:
            self._host = np.empty(2 * words, dtype=np.int32)
        if words > self._meta_dev.numel():
            self._meta_dev = torch.empty(2 * words, dtype=torch.int32, device=self.device)
        flat = self._host
        cursor = 0
        for index, count in enumerate(counts):
            step.offsets[index] = cursor
            cursor += count
        o = step.offsets
        ids, positions, tok_seg = (flat[o[i]:o[i] + T] for i in range(3))
        seg_start = flat[o[3]:o[3] + S + 1]
        logit_rows = flat[o[6]:o[6] + R]
        seg_start[0] = 0
        first_tokens = [seg.pos0 for seg in segments]
        base = row = 0
        if leading:
            # the decoding requests at the head of the step (hundreds, in a large batch): whole
            # columns at once instead of element by element
            heads = segments[:leading]
            ids[:leading] = [seg.tokens[0] for seg in heads]
            positions[:leading] = first_tokens[:leading]
            counting = np.arange(leading + 1, dtype=np.int32)
            tok_seg[:leading] = counting[:leading]
            seg_start[1:leading + 1] = counting[1:]
            wanted = [index for index, seg in enumerate(heads) if seg.want]    # of one token: [] or [0]
            row = len(wanted)
            logit_rows[:row] = wanted
            base = leading
        for index in range(leading, S):
            seg, n = segments[index], lengths[index]
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
        flat[o[4]:o[4] + S] = [seg.slot for seg in segments]
        flat[o[5]:o[5] + S] = first_tokens
        for k, (seg_of, tok0) in enumerate(tiles):
            n = seg_of.size
            flat[o[7 + 2 * k]:o[7 + 2 * k] + n] = seg_of
            flat[o[8 + 2 * k]:o[8 + 2 * k] + n] = tok0
            step.n_tiles[k] = n
        if n_patch:
            # (segment index, row of the source): the segment's last token is the one in flight
            flat[o[11]:o[11] + n_patch] = [int(seg_start[index + 1]) - 1 for index, _ in patch]
            flat[o[12]:o[12] + n_patch] = [row for _, row in patch]
        step.n_patch = n_patch
        for g, rows in enumerate(tables_host):
            start = o[len(META_NAMES) + g]
            if S and widths[g]:
                flat[start:start + S * widths[g]] = np.asarray(rows, dtype=np.int32).reshape(-1)
            step.width[g] = widths[g]
        step.meta_host = flat.ctypes.data
        step.meta_dev = self._meta_dev.data_ptr()
        step.meta_words = words
        step.upload = 1
        step.T, step.S, step.R = T, S, R
        step.max_segment, step.leading_singles = max_segment, leading
        return step

    def run(self, segments: Sequence[Segment], tables_host: Sequence[np.ndarray],
            patch_source: Optional[torch.Tensor] = None, patch: Optional[Sequence] = None) -> torch.Tensor:
        """``patch``: (segment index, row of ``patch_source``) pairs: the last token of those
        segments is still on the device, in ``patch_source`` (int32), and is put into the step's
        token ids there."""
        if len(tables_host) > MAX_GROUPS:
            raise KernelError(f"a plan serves at most {MAX_GROUPS} page groups")
        step = self.pack(segments, tables_host, patch)
        step.patch_source = patch_source.data_ptr() if (patch and patch_source is not None) else None
        if step.T > self.max_tokens or step.R > self.max_rows:
            raise KernelError(f"a step of {step.T} tokens and {step.R} wanted rows exceeds the plan's "
                              f"{self.max_tokens} and {self.max_rows}")
        logits = torch.empty((step.R, self.vocab), dtype=torch.float32, device=self.device)
        step.logits = logits.data_ptr() if step.R else None
        status = self._run(self._handle, ctypes.byref(step), ctypes.byref(self._launches), kernel_lib.stream())
        kernel_lib.add_launches(self._launches.value)
        self.h2d_bytes = 4 * step.meta_words
        if status != 0:
            failed = self._library.fwb_plan_failed_op(self._handle)
            raise KernelError(f"the step plan failed at operation {failed} of {self.n_ops} with status {status}")
        return logits


def build_plan(model, caches, max_tokens: int, max_rows: int, num_slots: int, n_groups: int,
               bad_flag: torch.Tensor) -> Optional[StepPlan]:
    """The plan of ``model`` over the given layer caches, or None if some part has no native form."""
    spec = model.spec
    builder = PlanBuilder(model.precision, model.device, spec.hidden_size, max_tokens, max_rows, num_slots,
                          bad_flag)
    try:
        builder.embed(model.embedding, spec.vocab_size, spec.embedding_scale)
        for position, entry in enumerate(spec.schedule):
            source = position if entry.cache_of is None else entry.cache_of
            layer = model.layers[entry.layer]
            plan = getattr(layer, "plan", None)
            if plan is None:
                raise NotPlannable(f"arrangement {layer.layer.arrangement!r} has no native form")
            plan(builder, caches[source])
        builder.norm_linear(model.final_norm, model.head, EPI_F32, None, "the head", on_logit_rows=True)
        if spec.logit_softcap > 0:
            builder.softcap(spec.logit_softcap, spec.vocab_size)
        return builder.finish(n_groups, spec.vocab_size)
    except NotPlannable as reason:
        model.not_plannable = str(reason)
        return None
