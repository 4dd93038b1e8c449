"""Helpers shared by the GPU tests: model folders, the plain oracle, tolerances, traces."""
from __future__ import annotations

import functools
import random
import tempfile
from pathlib import Path

import numpy as np
import torch

import plain_lfm2 as P
from tiny_configs import TINY, make_model_dir

DTYPES = ("float32", "bfloat16")
STORED = {"float32": torch.float32, "bfloat16": torch.bfloat16}

# Tolerances, relative to scale = max(1, max|logit|).
# Against the float64 oracle: float32 is the acceptance bound of the 32-bit path; bfloat16 is
# ten unit roundoffs (2^-9 each) of the logit scale, on the same bfloat16 weights.
# Between two ways of cutting the same work: the float32 kernels sum every output element in
# one fixed order, so 1e-5 (in practice they agree bit for bit).  In bfloat16 the split-K factor
# of the tensor-core products follows the number of tokens in the step, so the fp32 sums differ
# in their last bits, an activation now and then rounds to the neighbouring bfloat16, and two
# cuts are two independent bfloat16 computations of the same value: they agree as well as each
# agrees with the oracle (same bound).  With the split factor pinned (TOL_CUTS_PINNED) the
# bfloat16 path is summed in one order too and must agree to one unit roundoff.
TOL_ORACLE = {"float32": 1e-4, "bfloat16": 10 * 2.0 ** -9}
TOL_CUTS = {"float32": 1e-5, "bfloat16": 10 * 2.0 ** -9}
TOL_CUTS_PINNED = {"float32": 1e-5, "bfloat16": 2.0 ** -9}

_TMP = tempfile.TemporaryDirectory(prefix="fwb200-tests-")


@functools.lru_cache(maxsize=None)
def model_dir(name: str, dtype: str, seed: int = 3) -> Path:
    """A folder with the tiny configuration ``name`` stored in ``dtype`` (made once)."""
    path = Path(_TMP.name) / f"{name}-{dtype}-{seed}"
    make_model_dir(path, TINY[name], seed=seed, preset="unit", dtype=STORED[dtype])
    return path


@functools.lru_cache(maxsize=None)
def plain_model(name: str, dtype: str, seed: int = 3):
    return P.load_model_dir(model_dir(name, dtype, seed))


@functools.lru_cache(maxsize=None)
def _plain_logits_cached(name, dtype, seed, tokens):
    cfg, w = plain_model(name, dtype, seed)
    return P.forward(cfg, w, list(tokens))


def plain_logits(name: str, dtype: str, tokens, seed: int = 3) -> np.ndarray:
    return _plain_logits_cached(name, dtype, seed, tuple(int(t) for t in tokens))


def random_tokens(name: str, length: int, seed: int) -> list:
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, TINY[name]["vocab_size"], size=length)]


@functools.lru_cache(maxsize=None)
def engine_model(name: str, dtype: str, seed: int = 3):
    from flyweight_b200.engine import load_model
    return load_model(model_dir(name, dtype, seed), dtype)


def new_runner(name: str, dtype: str, num_pages: int = 16, num_slots: int = 4,
               max_model_len: int = 1024, seed: int = 3):
    from flyweight_b200.engine import ModelRunner
    return ModelRunner(engine_model(name, dtype, seed), num_pages=num_pages, num_slots=num_slots,
                       max_model_len=max_model_len, max_batched_tokens=4096)


def assert_close(got: np.ndarray, want: np.ndarray, rel: float, what: str = "") -> None:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    scale = max(1.0, float(np.abs(want).max()))
    err = np.abs(got - want)
    worst = float(err.max()) if err.size else 0.0
    if worst > rel * scale:
        row = int(np.unravel_index(err.argmax(), err.shape)[0])
        first_bad = int(np.argmax(err.max(axis=-1) > rel * scale)) if err.ndim > 1 else row
        raise AssertionError(f"{what}: max|delta| {worst:.3e} > {rel:.1e} * {scale:.3g} "
                             f"(worst row {row}, first row over the bound {first_bad})")


def run_whole(runner, rid, tokens) -> np.ndarray:
    out = runner.step([(rid, tokens, list(range(len(tokens))))])
    runner.finish(rid)
    return out.cpu().numpy()


def run_portions(runner, rid, tokens, sizes) -> np.ndarray:
    """Feed ``tokens`` in portions of the given sizes (cycled), all logits wanted."""
    outs, pos, i = [], 0, 0
    while pos < len(tokens):
        n = min(sizes[i % len(sizes)], len(tokens) - pos)
        outs.append(runner.step([(rid, tokens[pos:pos + n], list(range(n)))]).cpu().numpy())
        pos += n
        i += 1
    runner.finish(rid)
    return np.concatenate(outs)


def mixed_trace(lengths, vocab, num_pages, max_live=4, seed=0, tail=32, name_prefix="r",
                sizes=(1, 2, 3, 7, 16, 33, 64, 2, 5)):
    """A trace of steps over several requests: up to ``max_live`` live at a time, portions of
    changing size for the body of each request and its last ``tail`` tokens one by one,
    requests starting as soon as the pool has pages for their whole length (so pages and
    slots of finished requests are used again).  Returns (steps, tokens by request); a step is
    a dict like a trace_run line, with every position wanted."""
    rng = random.Random(seed)
    nprng = np.random.default_rng(seed)
    tokens = {f"{name_prefix}{i}": [int(t) for t in nprng.integers(0, vocab, size=n)]
              for i, n in enumerate(lengths)}
    pages_of = {k: -(-len(v) // 64) for k, v in tokens.items()}
    waiting = list(tokens)
    live, done_pos = [], {}
    free = num_pages
    steps = []
    sizes = list(sizes)
    while waiting or live:
        while waiting and len(live) < max_live and pages_of[waiting[0]] <= free:
            rid = waiting.pop(0)
            free -= pages_of[rid]
            live.append(rid)
            done_pos[rid] = 0
        assert live, "the pool is too small for the next request"
        entries, ended = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                  # left out of this step, goes on later
            total = len(tokens[rid])
            pos = done_pos[rid]
            body = max(0, total - tail)
            n = min(rng.choice(sizes), body - pos) if pos < body else 1
            entries.append({"id": rid, "tokens": tokens[rid][pos:pos + n],
                            "want": list(range(n))})
            done_pos[rid] = pos + n
            if done_pos[rid] == total:
                ended.append(rid)
        if not entries:
            continue
        for rid in ended:
            live.remove(rid)
            free += pages_of[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps, tokens


def replay_in_process(runner, steps):
    """Run a trace through ``runner``; returns logits by request, in position order."""
    out = {}
    for step in steps:
        logits = runner.step([(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
        logits = logits.cpu().numpy()
        row = 0
        for e in step["entries"]:
            out.setdefault(e["id"], []).append(logits[row:row + len(e["want"])])
            row += len(e["want"])
        for rid in step["end"]:
            runner.finish(rid)
        runner.cache.check()
    return {rid: np.concatenate(parts) for rid, parts in out.items()}


class GuardedOutputs:
    """Guard bands around everything a kernel's Python face allocates (the stand-in for a memory
    checker): while active, every CUDA tensor that Python code makes with ``torch.empty`` or
    ``torch.empty_like`` lies in the middle of a larger buffer whose margins hold a canary byte,
    and is itself filled with 0xFF bytes (NaN in fp32 and bfloat16, -1 in int32), so an output
    element that no thread wrote shows up in the comparison.  ``check()`` waits for the device and
    fails if a byte of any margin changed: a kernel wrote before or past its output."""
    MARGIN = 1 << 16
    CANARY = 0xA5

    def __init__(self):
        self._empty = torch.empty
        self._empty_like = torch.empty_like
        self._held = []

    def _guarded(self, shape, dtype, device):
        count = 1
        for extent in shape:
            count *= int(extent)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        padded = -(-nbytes // 256) * 256
        buffer = self._empty(2 * self.MARGIN + padded, dtype=torch.uint8, device=device)
        buffer.fill_(self.CANARY)
        buffer[self.MARGIN:self.MARGIN + nbytes].fill_(0xFF)
        self._held.append((buffer, nbytes, tuple(shape), dtype))
        return buffer[self.MARGIN:self.MARGIN + nbytes].view(dtype).view(tuple(shape))

    def __enter__(self):
        def empty(*size, dtype=None, device=None, **kwargs):
            if device is None or torch.device(device).type != "cuda" or kwargs.get("pin_memory"):
                return self._empty(*size, dtype=dtype, device=device, **kwargs)
            shape = tuple(size[0]) if len(size) == 1 and not isinstance(size[0], int) else tuple(size)
            return self._guarded(shape, dtype or torch.get_default_dtype(), device)

        def empty_like(other, **kwargs):
            if not other.is_cuda or kwargs:
                return self._empty_like(other, **kwargs)
            return self._guarded(tuple(other.shape), other.dtype, other.device)

        torch.empty, torch.empty_like = empty, empty_like
        return self

    def __exit__(self, *exc):
        torch.empty, torch.empty_like = self._empty, self._empty_like
        return False

    def check(self):
        torch.cuda.synchronize()
        for buffer, nbytes, shape, dtype in self._held:
            for name, band in (("before", buffer[:self.MARGIN]), ("after", buffer[self.MARGIN + nbytes:])):
                bad = (band != self.CANARY).nonzero()
                if bad.numel():
                    at = int(bad[0])
                    where = at - self.MARGIN if name == "before" else at
                    raise AssertionError(f"a kernel wrote {name} its output of shape {shape} ({dtype}): "
                                         f"{bad.numel()} bytes changed, the first at offset {where} "
                                         f"{'from its start' if name == 'before' else 'past its end'}")

    def forget(self):
        self._held.clear()
