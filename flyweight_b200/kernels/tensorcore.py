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
    lib.set_option("tensorcore", _enabled)


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
_use_pairs = True


def set_pairs_enabled(flag: bool) -> None:
    """Prompt-sized products on CTA pairs (on by default); off: the single-CTA kernel."""
    global _use_pairs
    _use_pairs = bool(flag)
    lib.set_option("pairs", _use_pairs)

# Per-shape overrides found by measurement: (features, K, accumulators) -> (splits, stages);
# 0 keeps the rule's choice.  Only decode-sized token counts (<= 64) consult it.
TUNED = {}


def force_splits(splits) -> None:
    """Pin the split-K factor (None: chosen per shape).  With one fixed factor every output
    element is summed in the same order whatever the number of tokens in the step, which
    lets tests compare ways of cutting the work bit by bit."""
    global _forced_splits
    _forced_splits = splits
    lib.set_option("forced_splits", splits or 0)


def pick_splits(M: int, N: int, K: int) -> int:
    """CTAs that share one output tile's K range (a cluster, <= 8): as many as it takes to
    put work on every SM when the token tile is small (decode), 1 otherwise."""
    if _forced_splits is not None:
        return _forced_splits if M <= 64 else 1
    if M > 64:
        return 1
    return _splits_for(M, N, K, 1)


def _decode_tile(M: int, N: int) -> int:
    """Token tile of a decode-sized step.  33..64 tokens are cut into two tiles of 32 when the
    product has too few feature tiles to occupy the GPU (measured at batch 64: 6 % off the
    step); a product with many tiles keeps one token tile, so no weight is fetched twice."""
    if M <= 16:
        return 16
    if M <= 32 or -(-N // 128) < SM_COUNT:
        return 32
    return 64


_stage_cap = 8


def _ring_depth(M: int, N: int, splits: int, accumulators: int) -> int:
    """Stages of the shared-memory ring for decode-sized steps: at most four, and few enough
    that every CTA of the product is resident at once (measured: a product that needs a second
    wave of CTAs loses far more than a shallower ring does)."""
    bn = _decode_tile(M, N)
    stage = accumulators * 16384 + bn * 128
    ctas = -(-N // 128) * -(-M // bn) * splits
    per_sm = max(1, -(-ctas // SM_COUNT))
    fit = ((227 * 1024) // per_sm - 2048) // stage
    return max(2, min(3 if (accumulators == 2 and bn <= 16) else 4, fit, _stage_cap))


def _splits_for(M: int, N: int, K: int, accumulators: int) -> int:
    """Slices of K per output tile (a cluster, a power of two <= 8).  Measured inside the decode
    step of LFM2-1.2B on B200 at batch 1, 8 and 64: the step is fastest with about 400 CTAs per
    product (256 with two accumulators), as long as a slice keeps at least four 64-wide blocks."""
    bn = _decode_tile(M, N)
    tiles = -(-N // 128) * -(-M // bn)
    k_blocks = -(-K // 64)
    budget = 256 if accumulators == 2 else 400
    limit = 4 if accumulators == 2 else 8
    if accumulators == 2 and M > 32:
        return 1                    # two accumulators of two token tiles: the reduction costs more
    splits = 1
    while splits < limit and tiles * splits * 2 <= budget and k_blocks >= splits * 8:
        splits *= 2
    return splits


# ---- 65 to 512 tokens: which tile, how many slices of K, or CTA pairs ----------------------
# Between decode-sized steps (a weight streamer on every SM) and prompt-sized ones (256-token
# tiles that fill the GPU) a product has few output tiles, and a CTA's walk over K is bound by
# latency, not by bandwidth: about 0.38 us per 64-wide block whatever the tile (0.6 us with two
# accumulators, 0.84 us for two accumulators of 256 tokens), 3 us of fixed cost, and a cluster
# reduction that costs 2.6 to 3.9 us depending on the tile and the number of slices.  The choice
# below evaluates that cost model (hundredths of a microsecond, fitted to products of LFM2-1.2B
# and LFM2-350M at 65 to 1,024 tokens on B200) for every tile and split the kernels have and takes
# the cheapest; a split is only considered when all its CTAs run at once (clusters in a second
# wave were measured far slower than the model).  The native dispatch (csrc/plan.cu) has the same
# table and the same loop.
MID_FROM, MID_TO = 65, 512
_MID_FIXED = 310
_MID_BLOCK = {1: {64: 38, 128: 38, 256: 42}, 2: {64: 63, 128: 58, 256: 84}}
_MID_PAIR_BLOCK = 36
_MID_REDUCE = {(128, 2): 360, (128, 4): 260, (64, 2): 390, (64, 4): 310}
_mid_size_split = True


def set_mid_size_split(flag: bool) -> None:
    """The cost-model choice for products of 65 to 512 tokens (on by default); off: CTA pairs
    above 128 tokens and one CTA per 128-token tile below, without a split."""
    global _mid_size_split
    _mid_size_split = bool(flag)
    lib.set_option("mid_size_split", _mid_size_split)


def mid_size_choice(M: int, N: int, K: int, accumulators: int, pair_ok: bool):
    """For ``MID_FROM <= M <= MID_TO``: ("pair", 0, 1) or ("single", token tile, slices of K)."""
    k_blocks = -(-K // 64)
    feature_tiles = -(-N // 128)
    best = None
    for tile in (64, 128, 256):
        if tile == 256 and M <= 128:
            continue
        for splits in (1, 2, 4):
            if splits > 1 and (tile > 128 or accumulators == 2 or _forced_splits is not None
                               or k_blocks < 4 * splits):
                continue
            ctas = feature_tiles * -(-M // tile) * splits
            waves = -(-ctas // SM_COUNT)
            if splits > 1 and waves > 1:
                continue
            cost = _MID_FIXED + _MID_BLOCK[accumulators][tile] * -(-k_blocks // splits) * waves
            if splits > 1:
                cost += _MID_REDUCE[(tile, splits)]
            if best is None or cost < best[0]:
                best = (cost, "single", tile, splits)
    if pair_ok:
        pairs = -(-N // 256) * -(-M // 256)
        cost = _MID_FIXED + _MID_PAIR_BLOCK * k_blocks * -(-pairs // (SM_COUNT // 2))
        if cost < best[0]:
            best = (cost, "pair", 0, 1)
    return best[1:]


def adds_in_place(x, w, residual) -> bool:
    """Whether ``gemm(x, w, fp32, addend=residual, out=residual)`` is available: the single-CTA
    kernel has the epilogue (every element is read and written by the same thread), the
    CTA-pair kernel of prompt-sized steps has not."""
    return (_add_in_place and (x.shape[0] >= FUSE_FROM_TOKENS or _fuse_always)
            and accepts(x, w, torch.float32, residual) and x.shape[0] <= 128
            and residual.dtype == torch.float32 and residual.is_contiguous()
            and tuple(residual.shape) == (x.shape[0], w.shape[0]))


def gemm(x, w, out_dtype, addend=None, splits=None, stages=0, tile_tokens=0, wide=-1, out=None) -> torch.Tensor:
    """``x @ w.T``: x [M][K] bf16, w [N][K] bf16 -> [M][N] fp32 or bf16 (+ fp32 addend).
    ``out`` may be the addend itself (the sum in place)."""
    check_tensor("gemm input", x, torch.bfloat16)
    check_tensor("gemm weight", w, torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: input has {K} columns, weight has {w.shape[1]}")
    free_choice = splits is None and not stages and not tile_tokens and wide == -1
    pair_ok = _use_pairs and M > 128 and addend is None and out is None and N >= 256
    if free_choice and _mid_size_split and MID_FROM <= M <= MID_TO:
        kind, tile_tokens, splits = mid_size_choice(M, N, K, 1, pair_ok)
        if kind == "pair":
            return gemm_pair(x, w, out_dtype, wide=False)
    elif pair_ok and free_choice:
        # prompt-sized: CTA pairs (cta_group::2); two feature blocks per pair when single blocks
        # would make more CTAs than the GPU holds at once (measured at 2,048 tokens on B200)
        pairs = -(-N // 256) * -(-M // 256)
        return gemm_pair(x, w, out_dtype, wide=pairs > SM_COUNT // 2)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    else:
        check_tensor("gemm output", out, out_dtype, (M, N))
    if addend is not None:
        check_tensor("gemm addend", addend, torch.float32, (M, N))
        epilogue = EPI_ADD_F32
    else:
        epilogue = EPI_F32 if out_dtype == torch.float32 else EPI_BF16
    if M <= 64 and (N, K, 1) in TUNED and _forced_splits is None:
        tuned = TUNED[(N, K, 1)]
        splits = splits or tuned[0] or None
        stages = stages or tuned[1]
        if len(tuned) > 2:
            tile_tokens = tile_tokens or tuned[2]
    if splits is None:
        splits = pick_splits(M, N, K)
    if M <= 64:
        stages = stages or _ring_depth(M, N, splits, 1)
        tile_tokens = tile_tokens or _decode_tile(M, N)
    lib.call("fwb_gemm_tcgen05", ptr(x), ptr(w), ptr(out), ptr(addend), M, N, K, N, N, epilogue, 0,
             splits, stages, tile_tokens, wide, stream(), tag=f"{N}x{K} splits {splits}")
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
        if len(tuned) > 2:
            tile_tokens = tile_tokens or tuned[2]
    free_choice = splits is None and not stages and not tile_tokens
    if splits is None:
        splits = (_forced_splits if _forced_splits is not None else _splits_for(M, F, K, 2)) if M <= 64 else 1
    if M <= 64:
        stages = stages or _ring_depth(M, F, splits, 2)
        tile_tokens = tile_tokens or _decode_tile(M, F)
    mid = free_choice and _mid_size_split and MID_FROM <= M <= MID_TO
    if mid:
        _, tile_tokens, splits = mid_size_choice(M, F, K, 2, False)
    cut = _wave_cut(M, F) if (M > 128 and splits == 1 and not stages and not tile_tokens and not mid) else 0
    if cut:
        # Prompt-sized: 256-token tiles make a number of CTAs that ends in a part-filled wave.  The
        # feature tiles of the whole waves run as they are; the rest runs with 128-token tiles, twice
        # as many CTAs of half the length, which fit one wave and start as the first launch drains.
        first = cut * 128
        lib.call("fwb_gemm_tcgen05", ptr(x), ptr(w_gate_up), ptr(out), ptr(None), M, first, K, F2, F,
                 EPI_SWIGLU_BF16, F, 1, 0, 256, -1, stream(), tag=f"swiglu {F}x{K} first")
        lib.call("fwb_gemm_tcgen05", ptr(x), _offset(w_gate_up, first * K), _offset(out, first), ptr(None), M,
                 F - first, K, F2 - first, F, EPI_SWIGLU_BF16, F, 1, 0, 128, -1, stream(), tag=f"swiglu {F}x{K} rest")
        return out
    lib.call("fwb_gemm_tcgen05", ptr(x), ptr(w_gate_up), ptr(out), ptr(None), M, F, K, F2, F,
             EPI_SWIGLU_BF16, F, splits, stages, tile_tokens, -1, stream(), tag=f"swiglu {F}x{K} splits {splits}")
    return out


def _offset(tensor, elements: int):
    """The address ``elements`` into a contiguous tensor (a slice without making a view)."""
    return tensor.data_ptr() + elements * tensor.element_size()


def _wave_cut(M: int, F: int) -> int:
    """How many 128-feature tiles the first of two launches takes (0: one launch).  With one CTA
    per SM, ``tiles`` CTAs take ceil(tiles / 148) rounds; when the last round would be less than
    three quarters full and what is left fits one round of half-length CTAs, cutting there saves
    most of a round (measured at 2,048 tokens, 8,192 features: 115.6 -> 110.6 us)."""
    token_tiles = -(-M // 256)
    feature_tiles = -(-F // 128)
    ctas = token_tiles * feature_tiles
    whole = ctas // SM_COUNT
    left = ctas - whole * SM_COUNT
    if whole == 0 or left == 0 or left > 0.75 * SM_COUNT:
        return 0
    cut = (whole * SM_COUNT) // token_tiles
    rest = feature_tiles - cut
    if cut <= 0 or rest <= 0 or rest * -(-M // 128) > SM_COUNT:
        return 0
    return cut


_fuse_norm = True
_add_in_place = True
_fuse_always = False
# Measured inside the decode step of LFM2-1.2B on B200: folding the norms into the products
# (and the residual sums into the epilogues) takes 2-3 % off the step from 16 tokens on; below
# that the separate norm kernel is faster, because the next product's first weight tiles are
# fetched while it runs.
FUSE_FROM_TOKENS = 16


def fuse_always(flag: bool) -> None:
    """Fold norms and residual sums at every decode-sized token count (tests of that path)."""
    global _fuse_always
    _fuse_always = bool(flag)
    lib.set_option("fuse_always", _fuse_always)



def set_norm_fusion(flag: bool) -> None:
    """Norms folded into the product that follows them (on by default).  Off: the norm kernel
    writes bf16 rows first, as prompt-sized steps always do; tests that compare cuts bit by bit
    switch it off so that every cut runs the same arithmetic."""
    global _fuse_norm, _add_in_place
    _fuse_norm = _add_in_place = bool(flag)
    lib.set_option("fuse_norm", _fuse_norm)
    lib.set_option("add_in_place", _add_in_place)


def normed_accepts(M: int, K: int, w, accumulators: int, N: int) -> bool:
    """Decode-sized token counts whose K slice per CTA is short enough that building the
    activation tiles inside the kernel stays off the critical path."""
    if not (_enabled and _fuse_norm) or w.dtype != torch.bfloat16 or M > 64 or K % 8 or not _aligned(w):
        return False
    if M < FUSE_FROM_TOKENS and not _fuse_always:
        return False
    splits = _forced_splits if _forced_splits is not None else _splits_for(M, N, K, accumulators)
    return -(-K // 64) <= 8 * splits


def gemm_normed(x_res, norm_weight, eps, w, out_dtype, rows=None, n_rows=None, splits=None, stages=0,
                tile_tokens=0) -> torch.Tensor:
    """``rmsnorm(x_res[rows]) @ w.T`` in one kernel: fp32 residual rows in, [M][N] fp32 or bf16 out."""
    check_tensor("residual", x_res, torch.float32)
    check_tensor("norm weight", norm_weight, torch.float32)
    check_tensor("gemm weight", w, torch.bfloat16)
    K = x_res.shape[-1]
    M = x_res.numel() // K if rows is None else (rows.numel() if n_rows is None else n_rows)
    N = w.shape[0]
    if w.shape[1] != K or norm_weight.numel() != K:
        raise KernelError(f"gemm: residual has {K} columns, weight has {w.shape[1]}, norm {norm_weight.numel()}")
    out = torch.empty((M, N), dtype=out_dtype, device=x_res.device)
    if splits is None:
        splits = pick_splits(M, N, K)
    stages = stages or _ring_depth(M, N, splits, 1)
    tile_tokens = tile_tokens or _decode_tile(M, N)
    lib.call("fwb_gemm_tcgen05_normed", ptr(x_res), ptr(norm_weight), ptr(rows), lib.c_float(eps), ptr(w),
             ptr(out), M, N, K, N, N, EPI_F32 if out_dtype == torch.float32 else EPI_BF16, 0, splits,
             stages, tile_tokens, stream(), tag=f"normed {N}x{K} splits {splits}")
    return out


def swiglu_gate_up_normed(x_res, norm_weight, eps, w_gate_up, splits=None, stages=0, tile_tokens=0) -> torch.Tensor:
    """``silu(n @ gate.T) * (n @ up.T)`` with n = rmsnorm(x_res), in one kernel."""
    check_tensor("residual", x_res, torch.float32)
    check_tensor("norm weight", norm_weight, torch.float32)
    check_tensor("swiglu weight", w_gate_up, torch.bfloat16)
    K = x_res.shape[-1]
    M = x_res.numel() // K
    F2 = w_gate_up.shape[0]
    F = F2 // 2
    if w_gate_up.shape[1] != K or F * 2 != F2 or norm_weight.numel() != K:
        raise KernelError("swiglu: weight must be [2F][K] and the norm weight [K]")
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x_res.device)
    if splits is None:
        splits = _forced_splits if _forced_splits is not None else _splits_for(M, F, K, 2)
    stages = stages or _ring_depth(M, F, splits, 2)
    tile_tokens = tile_tokens or _decode_tile(M, F)
    lib.call("fwb_gemm_tcgen05_normed", ptr(x_res), ptr(norm_weight), ptr(None), lib.c_float(eps),
             ptr(w_gate_up), ptr(out), M, F, K, F2, F, EPI_SWIGLU_BF16, F, splits, stages, tile_tokens,
             stream(), tag=f"normed swiglu {F}x{K} splits {splits}")
    return out


def status() -> int:
    """0, or the code a wait that gave up inside the kernel left (reads and clears it;
    synchronises the device)."""
    return int(lib.library().fwb_gemm_tcgen05_status())


def gemm_pair(x, w, out_dtype, wide=False) -> torch.Tensor:
    """``x @ w.T`` on CTA pairs (tcgen05 cta_group::2): 256 features x 256 tokens per pair and
    accumulator.  For prompt-sized steps; bf16 in, fp32 or bf16 out."""
    check_tensor("gemm input", x, torch.bfloat16)
    check_tensor("gemm weight", w, torch.bfloat16)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: input has {K} columns, weight has {w.shape[1]}")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    epilogue = EPI_F32 if out_dtype == torch.float32 else EPI_BF16
    cut = _pair_wave_cut(M, N) if wide else 0
    if cut:
        # the wide blocks of the whole rounds, then the rest as narrow pairs that fit one round
        first = cut * 512
        lib.call("fwb_gemm_tcgen05_pair", ptr(x), ptr(w), ptr(out), M, first, K, N, N, epilogue, 0, 1, stream())
        lib.call("fwb_gemm_tcgen05_pair", ptr(x), _offset(w, first * K), _offset(out, first), M, N - first, K,
                 N - first, N, epilogue, 0, 0, stream())
        return out
    lib.call("fwb_gemm_tcgen05_pair", ptr(x), ptr(w), ptr(out), M, N, K, N, N, epilogue, 0,
             1 if wide else 0, stream(), tag=f"{N}x{K}")
    return out


def _pair_wave_cut(M: int, N: int) -> int:
    """For the wide CTA-pair form (512 features a pair): how many 512-feature blocks the first of
    two launches takes (0: one launch).  74 pairs run at a time; when the last round would be less
    than three quarters full and what is left fits one round of one-block pairs (half the length),
    cutting there saves most of half a round (in_proj at 2,048 tokens: 96 pairs = 1.3 rounds)."""
    slots = SM_COUNT // 2
    token_tiles = -(-M // 256)
    pairs = -(-N // 512) * token_tiles
    whole = pairs // slots
    left = pairs - whole * slots
    if whole == 0 or left == 0 or left > 0.75 * slots:
        return 0
    cut = (whole * slots) // token_tiles
    rest = N - cut * 512
    if cut <= 0 or rest <= 0 or -(-rest // 256) * token_tiles > slots:
        return 0
    return cut


def swiglu_gate_up_pair(x, w_gate_up) -> torch.Tensor:
    """The fused gate/up product with the SwiGLU epilogue on CTA pairs."""
    check_tensor("swiglu input", x, torch.bfloat16)
    check_tensor("swiglu weight", w_gate_up, torch.bfloat16)
    M, K = x.shape
    F = w_gate_up.shape[0] // 2
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    lib.call("fwb_gemm_tcgen05_pair", ptr(x), ptr(w_gate_up), ptr(out), M, F, K, 2 * F, F,
             EPI_SWIGLU_BF16, F, 0, stream())
    return out
