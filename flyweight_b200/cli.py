"""Command line, shaped after flyweight's (src/flyweight/cli.py:844-1236): the same
command names and option names where flyweight has them (``generate``, ``benchmark``,
``inspect``; ``--max-tokens``, ``--context``, ``--temperature``, ``--top-k``, ``--top-p``,
``--min-p``, ``--seed``, ``--parallel``, ``--device``, ``--warmup``, ``--iterations``,
``--tokens``), with token ids in place of text: this engine has no tokenizer.

    python -m flyweight_b200 generate MODEL --prompt 1,2,3 --max-tokens 16 --temperature 0
    python -m flyweight_b200 benchmark MODEL --tokens 1,2,3 --iterations 64
    python -m flyweight_b200 inspect MODEL
    python -m flyweight_b200 make-random CONFIG.json --seed 0 --out DIR
    python -m flyweight_b200 replay --model DIR --dtype float32 --out DIR --max-tokens N < trace
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path


def _ids(text: str):
    return [int(part) for part in text.replace(",", " ").split()]


def _add_model(parser):
    parser.add_argument("model", metavar="MODEL", help="folder with config.json and model.safetensors")


def _add_runtime(parser):
    group = parser.add_argument_group("runtime")
    group.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                       help="bfloat16 serving precision, or everything in true 32-bit")
    group.add_argument("--device", type=int, default=0, metavar="N", help="CUDA device index")
    group.add_argument("--parallel", type=int, default=1, dest="parallel_sequences", metavar="N",
                       help="requests that may be live at a time")
    group.add_argument("--cache-tokens", type=int, default=None, metavar="N",
                       help="size of the KV page pool in tokens (default: parallel x context)")
    group.add_argument("--max-batched-tokens", type=int, default=2048, metavar="N",
                       help="token budget of one step (portions of prompts are cut to fit)")


def _parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="flyweight_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    from . import __version__
    parser.add_argument("--version", action="version", version=f"flyweight_b200 {__version__}")
    commands = parser.add_subparsers(dest="command", required=True)

    generate = commands.add_parser("generate", help="print one response and exit")
    _add_model(generate)
    request = generate.add_argument_group("request")
    request.add_argument("--prompt", metavar="IDS", help="prompt token ids, e.g. 1,2,3")
    request.add_argument("--random-prompt", type=int, metavar="LEN",
                         help="a uniform-random prompt of LEN token ids (seeded by --seed)")
    request.add_argument("--max-tokens", "--max-new-tokens", dest="max_new_tokens", type=int,
                         default=64, metavar="N", help="maximum generated tokens")
    request.add_argument("--context", "--context-window", dest="context_window", type=int,
                         default=32768, metavar="N", help="maximum prompt + output tokens")
    request.add_argument("--stop", metavar="IDS", default="", help="stop token ids")
    sampling = generate.add_argument_group("sampling")
    sampling.add_argument("--temperature", type=float, default=0.8, metavar="X",
                          help="sampling temperature; 0 is greedy")
    sampling.add_argument("--top-k", type=int, default=40, metavar="N",
                          help="how many candidates the sampler considers")
    sampling.add_argument("--top-p", type=float, default=0.95, metavar="X",
                          help="nucleus cut over those candidates, in (0, 1]")
    sampling.add_argument("--min-p", type=float, default=0.05, metavar="X",
                          help="drop candidates below this fraction of the best one's probability")
    sampling.add_argument("--seed", type=int, metavar="N", help="fixed RNG seed")
    sampling.add_argument("--repetition-penalty", type=float, default=1.0, metavar="X")
    sampling.add_argument("--presence-penalty", type=float, default=0.0, metavar="X")
    sampling.add_argument("--frequency-penalty", type=float, default=0.0, metavar="X")
    sampling.add_argument("--penalty-window", type=int, default=64, metavar="N")
    _add_runtime(generate)

    bench = commands.add_parser("benchmark", help="time prompt ingestion and decoding")
    _add_model(bench)
    bench.add_argument("--tokens", default="0", metavar="IDS", help="prompt token ids")
    bench.add_argument("--warmup", type=int, default=3, metavar="N")
    bench.add_argument("--iterations", type=int, default=128, metavar="N",
                       help="decoded tokens that are timed")
    bench.add_argument("--context", type=int, default=2048, metavar="N")
    _add_runtime(bench)

    inspect = commands.add_parser("inspect", help="print configuration and tensor table as JSON")
    _add_model(inspect)

    make = commands.add_parser("make-random",
                               help="write a model folder with seeded random weights")
    make.add_argument("config", metavar="CONFIG.json")
    make.add_argument("--seed", type=int, default=0)
    make.add_argument("--out", required=True, metavar="DIR")
    make.add_argument("--preset", choices=("baseline", "unit"), default="baseline")
    make.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                      help="dtype the tensors are stored in")

    replay = commands.add_parser("replay", help="trace replay (same as bin/trace_run)",
                                 add_help=False)
    replay.add_argument("rest", nargs=argparse.REMAINDER)
    return parser


def _open_runtime(args, context):
    from .engine.runtime import Model
    model = Model(args.model, dtype=args.dtype, device=f"cuda:{args.device}")
    return model, model.native_runtime(context_limit=context,
                                       parallel_sequences=args.parallel_sequences,
                                       cache_tokens=args.cache_tokens,
                                       max_batched_tokens=args.max_batched_tokens)


def _generate(args) -> int:
    import random
    from .config.registry import read_config_json
    if args.prompt:
        prompt = _ids(args.prompt)
    elif args.random_prompt:
        vocab = int(read_config_json(args.model)["vocab_size"])
        rng = random.Random(args.seed or 0)
        prompt = [rng.randrange(vocab) for _ in range(args.random_prompt)]
    else:
        print("generate needs --prompt IDS or --random-prompt LEN", file=sys.stderr)
        return 2
    context = min(args.context_window, len(prompt) + args.max_new_tokens)
    model, runtime = _open_runtime(args, context)
    with runtime:
        task = runtime.task_submit(
            prompt, args.max_new_tokens, _ids(args.stop), temperature=args.temperature,
            top_k=args.top_k, top_p=args.top_p, min_p=args.min_p, seed=args.seed,
            repetition_penalty=args.repetition_penalty, presence_penalty=args.presence_penalty,
            frequency_penalty=args.frequency_penalty, penalty_window=args.penalty_window)
        out = []
        while runtime.has_work():
            for tid, token, kind in runtime.engine_step():
                if tid == task and kind == 0:
                    out.append(token)
                elif tid == task and kind == 2:
                    print(runtime.task_error(task), file=sys.stderr)
                    return 1
    print(" ".join(str(t) for t in out))
    return 0


def _benchmark(args) -> int:
    """Prepare time, prompt + first token time, then per-token intervals with median and
    p90/p99, as flyweight's benchmark reports them (src/flyweight/cli.py:1749-1794)."""
    import torch
    started = time.perf_counter()
    prompt = _ids(args.tokens)
    total = args.warmup + args.iterations
    model, runtime = _open_runtime(args, min(args.context, len(prompt) + total + 1)
                                   if args.context < len(prompt) + total + 1 else args.context)
    torch.cuda.synchronize()
    prepared = time.perf_counter() - started
    stamps = []
    with runtime:
        begin = time.perf_counter()
        runtime.generate(prompt, total, lambda token: stamps.append(time.perf_counter()))
    first = stamps[0] - begin
    intervals = [b - a for a, b in zip(stamps[args.warmup:], stamps[args.warmup + 1:])]
    intervals.sort()
    pick = lambda q: intervals[min(len(intervals) - 1, int(q * len(intervals)))] if intervals else 0.0
    report = {
        "model": str(args.model), "dtype": args.dtype, "prompt_tokens": len(prompt),
        "prepare_seconds": prepared, "prompt_and_first_token_seconds": first,
        "decoded_tokens": len(intervals),
        "median_token_seconds": statistics.median(intervals) if intervals else None,
        "p90_token_seconds": pick(0.90), "p99_token_seconds": pick(0.99),
        "tokens_per_second": (len(intervals) / sum(intervals)) if intervals else None,
    }
    print(json.dumps(report))
    return 0


def _inspect(args) -> int:
    from . import models  # noqa: F401
    from .config.registry import load_config
    from .weights.safetensors_io import read_header
    arch, config = load_config(args.model)
    entries = read_header(Path(args.model) / "model.safetensors")
    tensors = {name: {"dtype": str(e.dtype).replace("torch.", ""), "shape": list(e.shape),
                      "bytes": e.end - e.begin} for name, e in sorted(entries.items())}
    report = {"architecture": arch.name, "config": config.to_dict(),
              "derived": {"head_dim": getattr(config, "head_dim", None),
                          "ffn_dim": getattr(config, "ffn_dim", None)},
              "tensor_count": len(tensors), "bytes": sum(t["bytes"] for t in tensors.values()),
              "tensors": tensors}
    print(json.dumps(report, indent=2))
    return 0


def _make_random(args) -> int:
    import torch
    from . import models  # noqa: F401
    from .config.registry import architecture_name, lookup
    from .parts.base import Precision
    from .weights.random_init import random_tensors, write_model_dir
    raw = json.loads(Path(args.config).read_text())
    arch = lookup(architecture_name(raw))
    config = arch.config_class.from_dict(raw)
    model = arch.model_class(config, Precision("float32"), torch.device("cpu"))
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    tensors = random_tensors(model.declare(), args.seed, args.preset, dtype, "cpu")
    out = write_model_dir(args.out, config.to_dict(), tensors, args.seed)
    print(json.dumps({"out": str(out), "tensors": len(tensors),
                      "parameters": sum(t.numel() for t in tensors.values())}))
    return 0


def main(argv=None) -> int:
    from .engine.loading import NoGpu
    try:
        return _run(_parser().parse_args(argv))
    except NoGpu as error:
        print(f"flyweight_b200: {error}", file=sys.stderr)
        return 3


def _run(args) -> int:
    if args.command == "generate":
        return _generate(args)
    if args.command == "benchmark":
        return _benchmark(args)
    if args.command == "inspect":
        return _inspect(args)
    if args.command == "make-random":
        return _make_random(args)
    if args.command == "replay":
        from .replay import main as replay_main
        return replay_main(args.rest)
    return 2
