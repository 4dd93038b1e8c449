#!/usr/bin/env python3
"""Headline benchmark: LFM2-1.2B with random bfloat16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests at a 4,096-token context.  The
one JSON line it prints carries the decode rate timed on the device (``value``), the same
through the Python entry point with host tokens in and out (``e2e``), a 2,048-token
prefill (``prefill``), the decode step against the HBM roofline (``roofline``) and
decode at batch 1 and 64 (``points``).  Inputs are synthetic: uniform-random token ids
and seeded random weights (there are no published LFM2 numbers to compare with, so
``vs_baseline`` is null).  For N > 1 it prints one line that says so and exits with 2:
the engine is single-GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The layer sizes of LFM2-1.2B (the benchmark configuration).
LFM2_1P2B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "num_hidden_layers": 16, "full_attn_idxs": [2, 5, 8, 10, 12, 14],
    "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "intermediate_size": 12288, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "conv_L_cache": 3, "conv_bias": False, "vocab_size": 65536, "rope_theta": 1000000.0,
    "norm_eps": 1e-5, "max_position_embeddings": 128000, "tie_embedding": True,
}
# The other two sizes the baseline names (same family; --sizes measures decode steps on them).
LFM2_350M = dict(LFM2_1P2B, hidden_size=1024, num_attention_heads=16, intermediate_size=6656)
LFM2_2P6B = dict(LFM2_1P2B, num_hidden_layers=30, full_attn_idxs=[2, 6, 10, 14, 18, 21, 24, 27],
                 intermediate_size=10752)
MODELS = {"lfm2-350m": LFM2_350M, "lfm2-1.2b": LFM2_1P2B, "lfm2-2.6b": LFM2_2P6B}
CONTEXT = 4096
BATCH = 8
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def read_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            raw = json.load(handle)
        peaks = {"hbm_gbs": float(raw["hbm_gbs"]),
                 "bf16_tflops": float(raw.get("bf16_tflops_sustained") or raw["bf16_tflops"]),
                 "bf16_tflops_burst": float(raw["bf16_tflops"]), "source": "measured"}
        return peaks
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while a region is timed."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


def model_flops_per_token(model) -> float:
    """2 x (weights of every matrix product a token passes through), head excluded: every part
    states its own."""
    return model.flops_per_token()


def attention_flops(model, n_tokens: int) -> float:
    """Causal attention of one n-token prompt: QK^T and PV, 2 * n^2 * heads * head_dim a layer
    (4 flops per query-key pair and channel, half of the pairs masked), as the mixers state it."""
    return model.context_flops(n_tokens)


def kv_bytes_per_token(model) -> int:
    total = 0
    for entry in model.spec.schedule:
        spec = model.layers[entry.layer].state_spec() if entry.cache_of is None else None
        if spec is not None and hasattr(spec, "n_kv_heads"):
            total += 2 * spec.n_kv_heads * spec.head_dim * model.precision.cache_dtype.itemsize
    return total


def fill_context(runner, requests, context, vocab, rng, chunk=2048):
    """Put ``context`` random tokens of every request into the cache (untimed set-up)."""
    import torch
    prompts = {r: torch.randint(0, vocab, (context,), generator=rng).tolist() for r in requests}
    for rid in requests:
        for start in range(0, context, chunk):
            runner.step([(rid, prompts[rid][start:start + chunk], [])])
    return prompts


SETTLE_STEPS = 32      # untimed steps before the warm-up steps of a decode timing


def time_decode(model, batch, context, steps, warmup, vocab, seed=0, per_step=False):
    """K decode steps of ``batch`` requests at ``context`` cached tokens each, timed with CUDA
    events on the launching stream: model step + greedy sampling, tokens given by the host.
    Before the W warm-up steps come ``SETTLE_STEPS`` untimed ones: the first twenty or so replays of a
    graph that has just been recorded run several per cent slower (with 5 warm-up steps and 20 timed
    ones the figure came out 8 % under the one of 200 timed steps)."""
    import torch
    from flyweight_b200.engine import ModelRunner
    from flyweight_b200.kernels import launch_count
    from flyweight_b200.sampling import sampler
    warmup = SETTLE_STEPS + warmup
    total = context + warmup + steps + 2
    pages = batch * (-(-total // 64))
    runner = ModelRunner(model, num_pages=pages, num_slots=batch, max_model_len=total,
                         max_batched_tokens=max(2048, batch))
    rng = torch.Generator().manual_seed(seed)
    requests = [f"b{i}" for i in range(batch)]
    fill_context(runner, requests, context, vocab, rng)
    tokens = torch.randint(0, vocab, (warmup + steps, batch), generator=rng).tolist()
    for i in range(warmup):
        sampler.argmax(runner.step([(r, [tokens[i][j]], [0]) for j, r in enumerate(requests)]))
    torch.cuda.synchronize()
    launches = launch_count()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)] if per_step else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, warmup + steps):
        if per_step:
            marks[i - warmup].record()
        sampler.argmax(runner.step([(r, [tokens[i][j]], [0]) for j, r in enumerate(requests)]))
    stop.record()
    if per_step:
        marks[steps].record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    launches = launch_count() - launches
    for r in requests:
        runner.finish(r)
    del runner
    torch.cuda.empty_cache()
    out = {"ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1e3), "launches": launches}
    if per_step:
        out["step_ms"] = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    return out


def _percentile(values, q):
    ordered = sorted(values)
    return ordered[min(len(ordered) - 1, int(round(q * (len(ordered) - 1))))]


def decode_spread(model, batch, context, vocab, regions=5, steps=200, warmup=5):
    """``regions`` timed regions of ``steps`` decode steps each (a fresh runner and a fresh context
    per region), every step between its own pair of events: median, p90 and p99 of the per-step
    time, the regions' means, and the SM clock sampled meanwhile."""
    clock = ClockSampler(0)
    clock.start()
    per_step, means = [], []
    for region in range(regions):
        timed = time_decode(model, batch, context, steps, warmup, vocab, seed=10 + region, per_step=True)
        per_step += timed["step_ms"]
        means.append(round(timed["ms_per_step"], 4))
    clocks = clock.stop()
    median = statistics.median(per_step)
    return {"regions": regions, "steps_per_region": steps, "ms_median": round(median, 4),
            "ms_p90": round(_percentile(per_step, 0.90), 4), "ms_p99": round(_percentile(per_step, 0.99), 4),
            "region_means_ms": means, "tokens_per_s_median": round(batch / (median / 1e3), 1),
            "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}


SAMPLING_PRESETS = {
    "greedy": dict(temperature=0.0),
    "topk": dict(temperature=0.8, top_k=20, top_p=0.95),                 # the shape of flyweight's served default
    "topp": dict(temperature=0.8, top_k=0, top_p=0.95),                  # the whole vocabulary, cut by mass only
    "penalty": dict(temperature=0.8, top_k=20, top_p=0.95, repetition_penalty=1.2),
}


def time_e2e(model, batch, context, steps, warmup, vocab, seed=1, sampling="greedy"):
    """The same through the public entry point: tasks queued on a Runtime, ``engine_step``
    pumped; every step uploads its batch from pinned host memory and reads its tokens back."""
    import torch
    from flyweight_b200.engine.runtime import Model
    rng = torch.Generator().manual_seed(seed)
    # requests admitted first decode while the later ones still read their prompts, so every
    # request gets room for those extra tokens and none finishes inside the timed region
    slack = 2 * batch * (-(-context // 2048)) + 8 + 24 + SETTLE_STEPS
    total = context + warmup + steps + slack
    runtime = Model(_model=model).native_runtime(context_limit=total, parallel_sequences=batch,
                                                max_batched_tokens=2048)
    for index in range(batch):
        prompt = torch.randint(0, vocab, (context,), generator=rng).tolist()
        runtime.task_submit(prompt, warmup + steps + slack - 2, seed=index + 1, **SAMPLING_PRESETS[sampling])
    while runtime.scheduler.waiting or any(t.pending > 1 for t in runtime.scheduler.running):
        runtime.engine_step()                     # prompts in (untimed)
    # untimed: the steps after which the runtime records a CUDA graph for a batch that stays the same
    # (EngineConfig.graph_after), and the asked-for warm-up steps behind them
    for _ in range(runtime.config.graph_after + 4 + SETTLE_STEPS + warmup):
        runtime.engine_step()
    torch.cuda.synchronize()
    h2d0, d2h0 = runtime.runner.h2d_bytes, runtime.info["d2h_bytes"]
    begin = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += sum(1 for _, _, kind in runtime.engine_step() if kind == 0)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    h2d = (runtime.runner.h2d_bytes - h2d0) / steps
    d2h = (runtime.info["d2h_bytes"] - d2h0) / steps
    runtime.close()
    torch.cuda.empty_cache()
    return {"value": produced / seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": seconds * 1e3 / steps}


def time_prefill(model, n_tokens, vocab, repeats=5, warmup=3, seed=2):
    import torch
    from flyweight_b200.engine import ModelRunner
    runner = ModelRunner(model, num_pages=-(-n_tokens // 64) + 1, num_slots=1,
                         max_model_len=n_tokens + 64, max_batched_tokens=n_tokens)
    rng = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, vocab, (n_tokens,), generator=rng).tolist()
    times = []
    for i in range(warmup + repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([("p", prompt, [n_tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        runner.finish("p")
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    del runner
    torch.cuda.empty_cache()
    return statistics.median(times)


def run_ours(args) -> int:
    import torch
    from flyweight_b200.engine.runtime import Model
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: flyweight_b200 has no CPU path"}))
        return 1
    peaks = read_peaks()
    config = dict(LFM2_1P2B)
    full_layers = config["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        config["num_hidden_layers"] = args.layers
        config["full_attn_idxs"] = [i for i in config["full_attn_idxs"] if i < args.layers]
    model = Model.random(config, seed=0, dtype="bfloat16", device="cuda:0").module
    vocab = config["vocab_size"]
    params = model.parameter_count()

    sampler_clock = ClockSampler(0)
    sampler_clock.start()
    main = time_decode(model, BATCH, CONTEXT, args.steps, args.warmup, vocab)
    clocks = sampler_clock.stop()
    e2e = time_e2e(model, BATCH, CONTEXT, args.steps, args.warmup, vocab)
    points = {}
    for batch in (1, 64):
        points[f"decode_b{batch}"] = time_decode(model, batch, CONTEXT, args.steps, args.warmup,
                                                 vocab)["tokens_per_s"]
    spread = {f"decode_b{batch}": decode_spread(model, batch, CONTEXT, vocab) for batch in (1, 8, 64)}
    prefill_ms = time_prefill(model, PREFILL_TOKENS, vocab)
    flops = (model_flops_per_token(model) * PREFILL_TOKENS + attention_flops(model, PREFILL_TOKENS)
             + 2.0 * model.head.numel())
    prefill_tflops = flops / (prefill_ms / 1e3) / 1e12
    step_bytes = model.weight_bytes(with_embedding_rows=BATCH) + BATCH * CONTEXT * kv_bytes_per_token(model)
    achieved = step_bytes / (main["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tokens/s, LFM2-1.2B bf16, batch 8, context 4096",
        "value": main["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: uniform-random token ids, seeded random weights N(0, 0.02)",
        "impl": "ours",
        "config": {
            "model": "LFM2-1.2B", "layers": config["num_hidden_layers"], "layers_full": full_layers,
            "attention_layers": len(config["full_attn_idxs"]), "hidden": config["hidden_size"],
            "heads": config["num_attention_heads"], "kv_heads": config["num_key_value_heads"],
            "head_dim": model.config.head_dim, "ffn_dim": model.config.ffn_dim,
            "conv_L_cache": config["conv_L_cache"], "vocab": vocab, "parameters": params,
            "global_batch": BATCH, "seq_len": CONTEXT, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single GPU", "page_size": 64,
            "l2": "inputs larger than L2 (2.3 GB of weights read per step), no flush",
            "settle_steps": SETTLE_STEPS,
            "peaks": peaks["source"],
        },
        "e2e": e2e,
        "gpu_launches": main["launches"],
        "clocks": clocks,
        # the prefill step is a few milliseconds between two synchronisations: a burst, so `frac`
        # is against the burst peak; the fraction of the sustained (power-capped) peak is beside it
        "prefill": {"value": PREFILL_TOKENS / (prefill_ms / 1e3), "tokens": PREFILL_TOKENS,
                    "ms": prefill_ms, "frac": prefill_tflops / peaks.get("bf16_tflops_burst", peaks["bf16_tflops"]),
                    "frac_of_burst_peak": prefill_tflops / peaks.get("bf16_tflops_burst", peaks["bf16_tflops"]),
                    "frac_of_sustained_peak": prefill_tflops / peaks["bf16_tflops"],
                    "flops": flops, "burst_peak_tflops": peaks.get("bf16_tflops_burst", peaks["bf16_tflops"]),
                    "sustained_peak_tflops": peaks["bf16_tflops"]},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "bytes_per_step": step_bytes,
                     "of": peaks["source"]},
        "points": points,
        "spread": spread,
    }
    print(json.dumps(line))
    return 0


def run_sizes(args) -> int:
    """Decode steps at other sizes: ``--sizes lfm2-2.6b:8x32768,64x32768`` prints one JSON line
    per BATCHxCONTEXT point (the same timer as the default run; not the contract's line)."""
    import torch
    from flyweight_b200.engine.runtime import Model
    name, _, points = args.sizes.partition(":")
    if name not in MODELS or not points:
        print(json.dumps({"error": f"--sizes wants MODEL:BATCHxCONTEXT[,...] with MODEL in {sorted(MODELS)}"}))
        return 1
    peaks = read_peaks()
    config = dict(MODELS[name])
    model = Model.random(config, seed=0, dtype="bfloat16", device="cuda:0").module
    for point in points.split(","):
        batch, context = (int(v) for v in point.lower().split("x"))
        timed = time_decode(model, batch, context, args.steps, args.warmup, config["vocab_size"])
        step_bytes = model.weight_bytes(with_embedding_rows=batch) + batch * context * kv_bytes_per_token(model)
        achieved = step_bytes / (timed["ms_per_step"] / 1e3) / 1e9
        # the same point through the public runtime, host tokens in and out every step
        e2e = time_e2e(model, batch, context, args.steps, args.warmup, config["vocab_size"], sampling=args.sampling)
        print(json.dumps({"sizes": True, "model": name, "parameters": model.parameter_count(),
                          "batch": batch, "context": context, "ms_per_step": timed["ms_per_step"],
                          "tokens_per_s": timed["tokens_per_s"], "bytes_per_step": step_bytes,
                          "hbm_gbs": achieved, "frac": achieved / peaks["hbm_gbs"], "of": peaks["source"],
                          "e2e_tokens_per_s": e2e["value"], "e2e_ms_per_step": e2e["ms_per_step"],
                          "e2e_sampling": args.sampling}),
              flush=True)
    return 0


def run_prefill_lengths(args) -> int:
    """One prompt of each given length through one step (``--prefill-lengths 128,512,8192``): a
    JSON line per length, the timer and the flop count of the default run's prefill figure."""
    import torch
    from flyweight_b200.engine.runtime import Model
    peaks = read_peaks()
    model = Model.random(dict(LFM2_1P2B), seed=0, dtype="bfloat16", device="cuda:0").module
    for n_tokens in (int(v) for v in args.prefill_lengths.split(",")):
        ms = time_prefill(model, n_tokens, LFM2_1P2B["vocab_size"])
        flops = (model_flops_per_token(model) * n_tokens + attention_flops(model, n_tokens)
                 + 2.0 * model.head.numel())
        print(json.dumps({"prefill_lengths": True, "model": "lfm2-1.2b", "tokens": n_tokens, "ms": ms,
                          "tokens_per_s": n_tokens / (ms / 1e3), "tflops": flops / (ms / 1e3) / 1e12,
                          "frac": flops / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "of": peaks["source"]}),
              flush=True)
    return 0


def run_chunked_prefill(args) -> int:
    """One long prompt in portions (``--chunked-prefill lfm2-2.6b:32768x2048``): every portion
    timed with CUDA events, one JSON line with the whole prompt's rate and what the attention over
    the cached keys adds between the first and the last portion."""
    import torch
    from flyweight_b200.engine import ModelRunner
    from flyweight_b200.engine.runtime import Model
    name, _, shape = args.chunked_prefill.partition(":")
    if name not in MODELS or "x" not in shape:
        print(json.dumps({"error": f"--chunked-prefill wants MODEL:CONTEXTxPORTION with MODEL in {sorted(MODELS)}"}))
        return 1
    context, portion = (int(v) for v in shape.lower().split("x"))
    peaks = read_peaks()
    config = dict(MODELS[name])
    model = Model.random(config, seed=0, dtype="bfloat16", device="cuda:0").module
    runner = ModelRunner(model, num_pages=context // 64 + 2, num_slots=1, max_model_len=context + 64,
                         max_batched_tokens=portion, use_graphs=False)
    prompt = torch.randint(0, config["vocab_size"], (context,), generator=torch.Generator().manual_seed(0)).tolist()
    for _ in range(2):                                  # the second pass is the timed one
        events = []
        for start in range(0, context, portion):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            last = start + portion >= context
            runner.step([("p", prompt[start:start + portion], [len(prompt[start:start + portion]) - 1] if last else [])])
            end.record()
            events.append((begin, end))
        torch.cuda.synchronize()
        runner.finish("p")
    ms = [begin.elapsed_time(end) for begin, end in events]
    heads, head_dim, layers = config["num_attention_heads"], model.config.head_dim, len(config["full_attn_idxs"])
    attention = sum(4.0 * min(portion, context - s) * (s + min(portion, context - s) / 2) * heads * head_dim * layers
                    for s in range(0, context, portion))
    flops = model_flops_per_token(model) * context + attention
    total = sum(ms)
    print(json.dumps({"chunked_prefill": True, "model": name, "context": context, "portion": portion,
                      "ms": total, "tokens_per_s": context / (total / 1e3), "tflops": flops / (total / 1e3) / 1e12,
                      "frac": flops / (total / 1e3) / (peaks["bf16_tflops"] * 1e12), "of": peaks["source"],
                      "first_portion_ms": ms[0], "last_portion_ms": ms[-1],
                      "attention_tflop": attention / 1e12, "portions_ms": [round(m, 2) for m in ms]}))
    return 0


def run_profile_step(args) -> int:
    """One step (decode at batch 8 / context 4,096, or a 2,048-token prefill) between
    cudaProfilerStart/Stop after warm-up, with CUDA graphs off so that every kernel is a launch
    of its own: the target of ``ncu --profile-from-start off`` for a per-kernel launch list."""
    import torch
    from flyweight_b200.engine import ModelRunner
    from flyweight_b200.engine.runtime import Model
    from flyweight_b200.sampling import sampler
    model = Model.random(dict(LFM2_1P2B), seed=0, dtype="bfloat16", device="cuda:0").module
    vocab = LFM2_1P2B["vocab_size"]
    rng = torch.Generator().manual_seed(0)
    if args.profile == "decode":
        total = CONTEXT + 16
        runner = ModelRunner(model, num_pages=BATCH * (-(-total // 64)), num_slots=BATCH,
                             max_model_len=total, max_batched_tokens=2048, use_graphs=False)
        requests = [f"b{i}" for i in range(BATCH)]
        fill_context(runner, requests, CONTEXT, vocab, rng)

        def step():
            sampler.argmax(runner.step([(r, [7], [0]) for r in requests]))
    else:
        runner = ModelRunner(model, num_pages=PREFILL_TOKENS // 64 + 2, num_slots=1,
                             max_model_len=PREFILL_TOKENS + 64, max_batched_tokens=PREFILL_TOKENS,
                             use_graphs=False)
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=rng).tolist()

        def step():
            runner.step([("p", prompt, [PREFILL_TOKENS - 1])])
            runner.finish("p")
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(json.dumps({"profiled": args.profile, "launches_per_step": "see the profiler's list"}))
    return 0


def run_mixed(args) -> int:
    """``--mixed lfm2-350m``: the baseline's mixed workload through the public runtime.  64 requests
    with prompt lengths drawn uniformly from 128 to 8,192 tokens are queued at once; the scheduler
    reads the prompts in portions under a budget of 512 tokens a step beside the requests that
    already decode; every request generates 256 tokens (greedy).  One JSON line: end-to-end tokens
    a second (prompt and generated tokens over the wall time), generated tokens a second, and per
    step the host's share (the time ``engine_step`` spends before it waits for the device) and
    the wait."""
    import random
    import torch
    from flyweight_b200.engine.runtime import Model
    name = args.mixed
    if name not in MODELS:
        print(json.dumps({"error": f"--mixed wants one of {sorted(MODELS)}"}))
        return 1
    config = dict(MODELS[name])
    model = Model.random(config, seed=0, dtype="bfloat16", device="cuda:0")
    requests, new_tokens, budget = 64, 256, 512
    rnd = random.Random(0)
    lengths = [rnd.randint(128, 8192) for _ in range(requests)]
    generator = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, config["vocab_size"], (n,), generator=generator).tolist() for n in lengths]
    results = []
    for attempt in range(2):                      # the first pass warms up (graphs are recorded), the second counts
        runtime = model.native_runtime(context_limit=8192 + new_tokens + 8, parallel_sequences=requests,
                                       max_batched_tokens=budget)
        for prompt in prompts:
            runtime.task_submit(prompt, new_tokens, temperature=0.0)
        torch.cuda.synchronize()
        clock = ClockSampler(0)
        clock.start()
        begun = time.perf_counter()
        steps = generated = 0
        while runtime.has_work():
            for _, _, kind in runtime.engine_step():
                generated += kind == 0
            steps += 1
        torch.cuda.synchronize()
        wall = time.perf_counter() - begun
        clocks = clock.stop()
        info = runtime.info
        runtime.close()
        results.append((wall, steps, generated, info, clocks))
    wall, steps, generated, info, clocks = results[-1]
    waited = info["sampling_seconds"]
    print(json.dumps({
        "mixed": name, "parameters": model.module.parameter_count(), "requests": requests,
        "prompt_tokens": sum(lengths), "generated_tokens": generated, "token_budget": budget,
        "seconds": round(wall, 4), "steps": steps,
        "tokens_per_s": round((sum(lengths) + generated) / wall, 1),
        "generated_tokens_per_s": round(generated / wall, 1),
        "ms_per_step": round(1e3 * wall / steps, 4),
        "host_ms_per_step": round(1e3 * (info["step_seconds"] - waited) / steps, 4),
        "wait_ms_per_step": round(1e3 * waited / steps, 4),
        "steady_steps": info["steady_steps"], "preemptions": info["preemptions"],
        "graphs_recorded": info["graphs_recorded"],
        "first_pass_seconds": round(results[0][0], 4), "clocks": clocks,
        "dtype": "bf16", "data": "synthetic: uniform-random token ids, seeded random weights"}))
    return 0


def run_kernel_times(args) -> int:
    """``--kernel-times [MODEL:]decode|prefill|TOKENS``: one step (of LFM2-1.2B unless another of the
    models is named, e.g. ``lfm2-350m:512``) launched kernel by kernel with
    a pair of CUDA events around every launch; prints {kernel, calls, us, share} by falling time,
    launches per step and the host time spent inside the launchers, as one JSON line.  The events
    keep kernels from overlapping their neighbours and every bracket includes the gap before its
    kernel starts; ``net_us`` takes the bracket of an empty kernel off every launch, and the
    step's real time (a second, unbracketed run) is printed beside the sums."""
    import torch
    from flyweight_b200.engine import ModelRunner
    from flyweight_b200.engine.runtime import Model
    from flyweight_b200.kernels import lib as kernel_lib
    from flyweight_b200.sampling import sampler
    name, _, what = args.kernel_times.rpartition(":")
    name = name or "lfm2-1.2b"
    batch, context = BATCH, CONTEXT
    if what.startswith("decode@"):                    # decode@BATCHxCONTEXT
        shape = what[len("decode@"):].split("x")
        if len(shape) == 2 and all(part.isdigit() for part in shape):
            batch, context, what = int(shape[0]), int(shape[1]), "decode"
    if name not in MODELS or not (what in ("decode", "prefill") or what.isdigit()):
        print(json.dumps({"error": "--kernel-times wants [MODEL:]decode|decode@BATCHxCONTEXT|prefill|TOKENS "
                                   f"with MODEL in {sorted(MODELS)}"}))
        return 1
    config = dict(MODELS[name])
    model = Model.random(config, seed=0, dtype="bfloat16", device="cuda:0").module
    vocab = config["vocab_size"]
    rng = torch.Generator().manual_seed(0)
    if what == "decode":
        total = context + 16
        runner = ModelRunner(model, num_pages=batch * (-(-total // 64)), num_slots=batch, max_model_len=total,
                             max_batched_tokens=2048, use_graphs=False, use_plan=False)
        requests = [f"b{i}" for i in range(batch)]
        fill_context(runner, requests, context, vocab, rng)
        tokens = batch

        def step():
            sampler.argmax(runner.step([(r, [7], [0]) for r in requests]))
    else:
        tokens = PREFILL_TOKENS if what == "prefill" else int(what)
        runner = ModelRunner(model, num_pages=tokens // 64 + 2, num_slots=1, max_model_len=tokens + 64,
                             max_batched_tokens=tokens, use_graphs=False, use_plan=False)
        prompt = torch.randint(0, vocab, (tokens,), generator=rng).tolist()

        def step():
            runner.step([("p", prompt, [tokens - 1])])
            runner.finish("p")
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    step()
    stop.record()
    torch.cuda.synchronize()
    kernel_lib.profile_start()
    step()
    report = kernel_lib.profile_stop()
    # what a pair of events costs around a kernel that does next to nothing (launched one by one,
    # a kernel starts a few microseconds after the one before it ended): taken off every call
    from flyweight_b200.kernels import ops
    tiny_x = torch.zeros(8, device="cuda:0")
    tiny_d = torch.zeros(8, device="cuda:0")
    rounds = []
    for _ in range(7):                   # the least of several rounds: a stall of the host inflates a round
        kernel_lib.profile_start()
        for _ in range(20):
            ops.add_(tiny_x, tiny_d)
        gap = kernel_lib.profile_stop()["kernels"][0]
        rounds.append(gap["us"] / gap["calls"])
    overhead = min(rounds)
    net_total = 0.0
    for entry in report["kernels"]:
        entry["net_us"] = round(max(0.0, entry["us"] - overhead * entry["launches"]), 2)
        net_total += entry["net_us"]
    for entry in report["kernels"]:
        entry["net_share"] = round(entry["net_us"] / (net_total or 1.0), 4)
    report["kernels"].sort(key=lambda entry: -entry["net_us"])
    report.update({"kernel_times": what, "model": name, "tokens": tokens, "bracket_overhead_us": round(overhead, 2),
                   "net_device_us": round(net_total, 1),
                   "step_us_unbracketed": round(1e3 * start.elapsed_time(stop), 1)})
    print(json.dumps(report))
    return 0


def run_reference(args) -> int:
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        from reference_arm import run as run_reference_arm
    except Exception as error:                                     # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable":
                          f"reference arm not set up: {type(error).__name__}: {error}"}))
        return 0
    return run_reference_arm(args, LFM2_1P2B, BATCH, CONTEXT)


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--layers", type=int, default=0,
                        help="run fewer layers than the configuration has (both counts are reported)")
    parser.add_argument("--sizes", default=None, metavar="MODEL:BxCTX[,BxCTX...]",
                        help="decode steps of lfm2-350m / lfm2-1.2b / lfm2-2.6b at other batches and contexts")
    parser.add_argument("--sampling", choices=sorted(SAMPLING_PRESETS), default="greedy",
                        help="with --sizes: how the requests of the runtime's column sample (greedy; topk: "
                             "temperature 0.8, top-k 20, top-p 0.95; topp: the same over the whole vocabulary; "
                             "penalty: topk with a repetition penalty)")
    parser.add_argument("--prefill-lengths", default=None, metavar="N[,N...]",
                        help="time one prompt of each length through one step (lfm2-1.2b)")
    parser.add_argument("--chunked-prefill", default=None, metavar="MODEL:CONTEXTxPORTION",
                        help="one long prompt read in portions, e.g. lfm2-2.6b:32768x2048")
    parser.add_argument("--profile", choices=("decode", "prefill"), default=None,
                        help="run one step inside cudaProfilerStart/Stop (for a profiler) and exit")
    parser.add_argument("--mixed", default=None, metavar="MODEL",
                        help="64 requests, prompts of 128 to 8,192 tokens in portions of 512 beside decoding "
                             "requests, 256 new tokens each, through the public runtime (e.g. lfm2-350m)")
    parser.add_argument("--kernel-times", default=None, metavar="[MODEL:]decode[@BATCHxCONTEXT]|prefill|TOKENS",
                        help="one step with CUDA events around every launch: time per kernel as JSON")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured (N=1 only)")
        return 2
    args.warmup = max(3, args.warmup)
    if args.profile:
        return run_profile_step(args)
    if args.kernel_times:
        return run_kernel_times(args)
    if args.mixed:
        return run_mixed(args)
    if args.sizes:
        return run_sizes(args)
    if args.prefill_lengths:
        return run_prefill_lengths(args)
    if args.chunked_prefill:
        return run_chunked_prefill(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
