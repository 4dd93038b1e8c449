"""Run one kernel of the library alone on synthetic inputs, timed with CUDA events.

    python -m flyweight_b200.kernels.microbench gemm --tokens 8 --features 6144 --k 2048
    python -m flyweight_b200.kernels.microbench gemm --tokens 2048 --features 8192 --k 2048 --swiglu
    python -m flyweight_b200.kernels.microbench attention-decode --batch 8 --context 4096
    python -m flyweight_b200.kernels.microbench attention-prefill --tokens 2048
    python -m flyweight_b200.kernels.microbench shortconv --tokens 2048
    python -m flyweight_b200.kernels.microbench qk-norm-rope --tokens 2048
    python -m flyweight_b200.kernels.microbench sample --rows 8 --top-k 40

It is what the ncu summaries under ``profiles/`` were captured from (small cases of the same
kernels the engine runs), and a quick way to see what a shape costs.  Weight matrices are
rotated through enough copies to exceed the L2 cache, so the timed reads come from HBM.
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def _time(fn, repeat: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeat):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / repeat          # microseconds


def _time_graph(fn, repeat: int) -> float:
    """The same for kernels shorter than a Python call: ``repeat`` launches captured into one
    CUDA graph, the replay timed."""
    fn()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(repeat):
                fn()
    return _time(graph.replay, 5) / repeat


def run_gemm(args) -> dict:
    from . import tensorcore
    M, N, K = args.tokens, args.features, args.k
    rows = 2 * N if args.swiglu else N
    copies = max(2, min(16, int(160e6 // (rows * K * 2)) + 1))
    weights = [(torch.randn(rows, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16)
               for _ in range(copies)]
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    turn = [0]

    def step():
        turn[0] = (turn[0] + 1) % copies
        w = weights[turn[0]]
        if args.swiglu:
            return tensorcore.swiglu_gate_up(x, w, args.splits or None, args.stages, args.tile_tokens)
        return tensorcore.gemm(x, w, torch.float32 if args.fp32_out else torch.bfloat16, None,
                               args.splits or None, args.stages, args.tile_tokens, args.wide)

    # a decode-sized product is shorter than a Python call: time it from a CUDA graph
    us = _time_graph(step, args.repeat) if M <= 128 else _time(step, args.repeat)
    flops = 2.0 * M * rows * K
    return {"kernel": "gemm_tcgen05", "tokens": M, "features": N, "k": K, "swiglu": args.swiglu,
            "us": us, "tflops": flops / us / 1e6, "weight_gb_s": rows * K * 2 / us / 1e3,
            "status": tensorcore.status()}


def _paged_inputs(batch, context, new, n_heads, n_kv, head_dim):
    pages_per = -(-context // 64)
    width = 16 * (-(-pages_per // 16))
    k_pool = torch.randn(batch * pages_per, n_kv, 64, head_dim, device="cuda").to(torch.bfloat16)
    v_pool = torch.randn(batch * pages_per, n_kv, 64, head_dim, device="cuda").to(torch.bfloat16)
    table = torch.full((batch, width), -1, dtype=torch.int32)
    for b in range(batch):
        table[b, :pages_per] = torch.arange(b * pages_per, (b + 1) * pages_per)
    q = torch.randn(batch * new, n_heads * head_dim, device="cuda").to(torch.bfloat16)
    return q, k_pool, v_pool, table.cuda(), width


def run_attention_decode(args) -> dict:
    from . import attention, ops
    B, ctx = args.batch, args.context
    q, k_pool, v_pool, table, width = _paged_inputs(B, ctx, 1, args.heads, args.kv_heads, args.head_dim)
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    tok_seg = torch.arange(B, dtype=torch.int32, device="cuda")
    splits, per, in_cluster = attention.decode_splits(B, args.kv_heads, width, args.head_dim)
    if args.splits:
        splits, per, in_cluster = args.splits, -(-width // args.splits), args.cluster_merge
    scale = 1.0 / math.sqrt(args.head_dim)
    ops.set_decode_attention_tma(not args.cp_async, args.stages)
    us = _time(lambda: ops.attention_decode_mma(q, k_pool, v_pool, positions, tok_seg, table,
                                                args.heads, 0, scale, splits, per, in_cluster), args.repeat)
    ops.set_decode_attention_tma(True)
    kv_bytes = B * ctx * args.kv_heads * args.head_dim * 2 * 2
    from . import tensorcore
    return {"kernel": "attention_decode_mma", "batch": B, "context": ctx, "splits": splits,
            "tiles_by": "cp.async" if args.cp_async or args.head_dim not in (64, 128) else "tma",
            "us": us, "kv_gb_s": kv_bytes / us / 1e3, "status": tensorcore.status()}


def run_attention_prefill(args) -> dict:
    from . import ops
    T = args.tokens
    group = args.heads // args.kv_heads
    q, k_pool, v_pool, table, _ = _paged_inputs(1, T, T, args.heads, args.kv_heads, args.head_dim)
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    seg_start = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    per_tile = max(1, (64 if args.mma_sync else 128) // group)
    n_tiles = -(-T // per_tile)
    tile_seg = torch.zeros(n_tiles, dtype=torch.int32, device="cuda")
    tile_tok0 = (torch.arange(n_tiles, dtype=torch.int32) * per_tile).cuda()
    scale = 1.0 / math.sqrt(args.head_dim)
    kernel = ops.attention_prefill_mma if args.mma_sync else ops.attention_prefill_tcgen05
    us = _time(lambda: kernel(q, k_pool, v_pool, positions, seg_start, tile_seg, tile_tok0, n_tiles,
                              per_tile, table, args.heads, 0, scale), args.repeat)
    flops = 2.0 * T * T * args.heads * args.head_dim        # causal: half of 4*T*T*h*d
    from . import tensorcore
    return {"kernel": "attention_prefill_mma" if args.mma_sync else "attention_prefill_tcgen05",
            "tokens": T, "us": us, "tflops": flops / us / 1e6, "status": tensorcore.status()}


def run_shortconv(args) -> dict:
    from . import ops
    T, H, L = args.tokens, args.hidden, args.taps
    p = torch.randn(T, 3 * H, device="cuda").to(torch.bfloat16)
    taps = torch.randn(H, L, device="cuda")
    state = torch.zeros(1, H, L - 1, device="cuda")
    seg_start = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    seg_slot = torch.zeros(1, dtype=torch.int32, device="cuda")
    tok_seg = torch.zeros(T, dtype=torch.int32, device="cuda")
    us = _time_graph(lambda: ops.shortconv(p, taps, None, state, seg_start, seg_slot, tok_seg, 1,
                                           torch.bfloat16), args.repeat)
    return {"kernel": "shortconv", "tokens": T, "hidden": H, "taps": L, "us": us,
            "gb_s": T * H * 2 * 4 / us / 1e3}


def run_qk_norm_rope(args) -> dict:
    from . import ops
    T, nh, nkv, hd = args.tokens, args.heads, args.kv_heads, args.head_dim
    pages = -(-T // 64)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda").to(torch.bfloat16)
    w = torch.ones(hd, device="cuda")
    angles = torch.arange(T, dtype=torch.float64)[:, None] * (1e6 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))
    table = torch.stack([angles.cos(), angles.sin()], -1).float().cuda()
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    tok_seg = torch.zeros(T, dtype=torch.int32, device="cuda")
    block_table = torch.arange(pages, dtype=torch.int32, device="cuda")[None]
    k_pool = torch.zeros(pages, nkv, 64, hd, device="cuda", dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    us = _time_graph(lambda: ops.qk_norm_rope(qkv, w, w, table, positions, tok_seg, block_table,
                                              k_pool, v_pool, nh, nkv, hd, hd, 1e-5, torch.bfloat16),
                     args.repeat)
    return {"kernel": "qk_norm_rope", "tokens": T, "us": us,
            "gb_s": T * (nh + 2 * nkv) * hd * 2 * 2 / us / 1e3}


def run_sample(args) -> dict:
    from ..sampling import sampler
    from ..sampling.config import SamplingConfig
    rows, vocab = args.rows, args.vocab
    # enough copies of the logits that the timed reads come from HBM
    copies = max(2, min(16, int(160e6 // (rows * vocab * 4)) + 1))
    # Gaussian logits of the given spread: at temperature 0.8 and top-p 0.95 a spread of 3 keeps about
    # 1,200 candidates of 65,536 (a flat row), a spread of 4 about 200 (a peaked one, like a model's)
    logits = [torch.randn(rows, vocab, device="cuda") * args.logit_scale for _ in range(copies)]
    config = SamplingConfig(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=0.0, seed=1)
    uniforms = [((i * 37) % 97) / 97.0 for i in range(rows)]
    turn = [0]

    def step():
        turn[0] = (turn[0] + 1) % copies
        if args.temperature <= 0.0:
            return sampler.argmax(logits[turn[0]])
        return sampler.sample(logits[turn[0]], [config] * rows, uniforms)

    if args.kernel_only and args.temperature > 0.0:
        # the launches alone: the rows' settings are staged once, not by every call's Python
        import struct
        from . import lib
        from .lib import ptr, stream
        k = min(args.top_k, vocab) if args.top_k > 0 else vocab
        large = k > sampler.SMALL_K
        record = struct.pack("<fifffffi", args.temperature, args.top_k, args.top_p, 0.0, 1.0, 0.0, 0.0, 0)
        params = torch.frombuffer(bytearray(record * rows), dtype=torch.uint8).cuda()
        uni = torch.tensor(uniforms, dtype=torch.float64, device="cuda")
        out = torch.empty(rows, dtype=torch.int32, device="cuda")
        vpad = 1
        while vpad < vocab:
            vpad <<= 1
        keys = torch.empty((rows, vpad), dtype=torch.int64, device="cuda") if large else None

        def step():
            turn[0] = (turn[0] + 1) % copies
            lib.call("fwb_sample", ptr(logits[turn[0]]), rows, vocab, ptr(params), ptr(uni), None, 0, ptr(out),
                     ptr(keys), None, vpad if large else 0, 1 if large else 0, stream())

    us = _time(step, args.repeat)
    return {"kernel": "argmax" if args.temperature <= 0.0 else "sample_kernel", "rows": rows, "vocab": vocab,
            "top_k": args.top_k, "top_p": args.top_p, "logit_scale": args.logit_scale,
            "kernel_only": bool(args.kernel_only), "us": us, "gb_s": rows * vocab * 4 / us / 1e3}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m flyweight_b200.kernels.microbench",
                                     description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="kernel", required=True)
    gemm = sub.add_parser("gemm")
    gemm.add_argument("--tokens", type=int, default=8)
    gemm.add_argument("--features", type=int, default=2048)
    gemm.add_argument("--k", type=int, default=2048)
    gemm.add_argument("--swiglu", action="store_true", help="features = F; the weight is [2F][K]")
    gemm.add_argument("--fp32-out", action="store_true")
    gemm.add_argument("--splits", type=int, default=0)
    gemm.add_argument("--stages", type=int, default=0)
    gemm.add_argument("--tile-tokens", type=int, default=0, help="128 or 256 (0: by token count)")
    gemm.add_argument("--wide", type=int, default=-1, help="two feature tiles per CTA: 1/0 (-1: auto)")
    for name in ("attention-decode", "attention-prefill"):
        p = sub.add_parser(name)
        p.add_argument("--batch", type=int, default=8)
        p.add_argument("--context", type=int, default=4096)
        p.add_argument("--tokens", type=int, default=2048)
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=64)
        p.add_argument("--splits", type=int, default=0)
        p.add_argument("--mma-sync", action="store_true", help="the mma.sync prompt kernel")
        p.add_argument("--cluster-merge", action="store_true", help="with --splits <= 8: merge inside the kernel")
        p.add_argument("--cp-async", action="store_true", help="decode: key and value tiles by cp.async, not TMA")
        p.add_argument("--stages", type=int, default=0, help="decode by TMA: ring depth, 2 to 8 (0: the launcher's choice)")
    conv = sub.add_parser("shortconv")
    conv.add_argument("--tokens", type=int, default=2048)
    conv.add_argument("--hidden", type=int, default=2048)
    conv.add_argument("--taps", type=int, default=3)
    rope = sub.add_parser("qk-norm-rope")
    rope.add_argument("--tokens", type=int, default=2048)
    rope.add_argument("--heads", type=int, default=32)
    rope.add_argument("--kv-heads", type=int, default=8)
    rope.add_argument("--head-dim", type=int, default=64)
    smp = sub.add_parser("sample")
    smp.add_argument("--rows", type=int, default=8)
    smp.add_argument("--vocab", type=int, default=65536)
    smp.add_argument("--temperature", type=float, default=0.8, help="0: arg-max")
    smp.add_argument("--top-k", type=int, default=40, help="0: the whole vocabulary")
    smp.add_argument("--top-p", type=float, default=0.95)
    smp.add_argument("--logit-scale", type=float, default=3.0, help="spread of the Gaussian logits")
    smp.add_argument("--kernel-only", action="store_true", help="time the launches without the Python call around them")
    for p in sub.choices.values():
        p.add_argument("--repeat", type=int, default=20)
    args = parser.parse_args(argv)
    runner = {"gemm": run_gemm, "attention-decode": run_attention_decode,
              "attention-prefill": run_attention_prefill, "shortconv": run_shortconv,
              "qk-norm-rope": run_qk_norm_rope, "sample": run_sample}[args.kernel]
    print(json.dumps(runner(args)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
