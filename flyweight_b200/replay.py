"""Trace replay (the program behind ``bin/trace_run``).

It owns no forward pass, cache or loader: it builds the same ``ModelRunner`` that the
engine uses for generation and calls its ``step`` with the tokens the trace gives.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__)
    parser.add_argument("--model", required=True, metavar="DIR",
                        help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                        help="bfloat16: the kernels and precisions serving uses; "
                             "float32: everything in true 32-bit")
    parser.add_argument("--out", required=True, metavar="DIR", help="where <step>.f32 files go")
    parser.add_argument("--max-tokens", type=int, required=True, metavar="N",
                        help="most tokens live requests hold at any time, each request's count "
                             "rounded up to a multiple of the page size (64)")
    parser.add_argument("--max-live", type=int, default=4, metavar="N",
                        help="most requests live at a time (state slots)")
    parser.add_argument("--device", default="cuda:0")
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from .cache.manager import PAGE_SIZE
    from .engine.loading import NoGpu, load_model
    from .engine.runner import ModelRunner

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    try:
        model = load_model(args.model, args.dtype, args.device)
    except NoGpu as error:
        print(f"trace_run: {error}", file=sys.stderr)
        return 3
    num_pages = max(1, args.max_tokens // PAGE_SIZE)
    max_len = min(model.spec.max_positions, num_pages * PAGE_SIZE)
    runner = ModelRunner(model, num_pages=num_pages, num_slots=max(1, args.max_live),
                         max_model_len=max_len, max_batched_tokens=max(num_pages * PAGE_SIZE, 1))
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in record.get("entries", [])]
        logits = runner.step(entries)
        if logits.shape[0]:
            data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
            runner.check_health()          # a kernel that gave up must not leave a file that looks fine
            data.tofile(out_dir / f"{step}.f32")
        for request in record.get("end", []):
            runner.finish(request)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
