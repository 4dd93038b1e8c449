"""The engine against the plain implementation under every way of cutting the work:
whole, a long first step then the last 32 tokens one by one, portions of changing size
down to two tokens, and mixed batches with so few pages that they are used again --
for both tiny configurations, in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from gpu_util import (DTYPES, TOL_CUTS, TOL_CUTS_PINNED, TOL_ORACLE, assert_close, mixed_trace, model_dir,
                      new_runner, plain_logits, random_tokens, replay_in_process, run_portions,
                      run_whole)
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

CASES = [(name, dtype) for name in ("A", "B") for dtype in DTYPES]
LENGTHS = (5, 67, 150)
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(name, dtype):
    runner = new_runner(name, dtype)
    for i, length in enumerate(LENGTHS):
        tokens = random_tokens(name, length, seed=10 + i)
        got = run_whole(runner, f"w{i}", tokens)
        assert_close(got, plain_logits(name, dtype, tokens), TOL_ORACLE[dtype],
                     f"{name} {dtype} whole request of {length}")
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_one_long_step_then_the_last_32_one_by_one(name, dtype):
    runner = new_runner(name, dtype)
    tokens = random_tokens(name, 150, seed=12)
    want = plain_logits(name, dtype, tokens)
    whole = run_whole(runner, "whole", tokens)
    head = len(tokens) - 32
    parts = [runner.step([("d", tokens[:head], list(range(head)))]).cpu().numpy()]
    for token in tokens[head:]:
        parts.append(runner.step([("d", [token], [0])]).cpu().numpy())
    runner.finish("d")
    got = np.concatenate(parts)
    assert_close(got, want, TOL_ORACLE[dtype], f"{name} {dtype} decode of the last 32")
    assert_close(got, whole, TOL_CUTS[dtype], f"{name} {dtype} decode vs whole")


@pytest.mark.parametrize("name", ["A", "B"])
def test_norms_and_residual_sums_folded_into_the_products_at_every_size(name):
    """Below 16 tokens a step runs the norm kernels by default; here the folded forms (the norm
    inside the next product, the residual sum in the epilogue) run for single tokens and small
    portions too, through CUDA graphs and without."""
    from flyweight_b200.kernels import tensorcore
    tensorcore.fuse_always(True)
    try:
        for use_graphs in (True, False):
            runner = new_runner(name, "bfloat16")
            runner.use_graphs = use_graphs
            tokens = random_tokens(name, 150, seed=14)
            want = plain_logits(name, "bfloat16", tokens)
            head = len(tokens) - 32
            parts = [runner.step([("d", tokens[:head], list(range(head)))]).cpu().numpy()]
            for token in tokens[head:]:
                parts.append(runner.step([("d", [token], [0])]).cpu().numpy())
            runner.finish("d")
            assert_close(np.concatenate(parts), want, TOL_ORACLE["bfloat16"], f"{name} folded, decode of the last 32")
            got = run_portions(runner, "p", tokens, [3, 2, 9, 40, 1, 14])
            assert_close(got, want, TOL_ORACLE["bfloat16"], f"{name} folded, small portions")
            runner.cache.check()
    finally:
        tensorcore.fuse_always(False)


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(name, dtype):
    runner = new_runner(name, dtype)
    tokens = random_tokens(name, 200, seed=13)
    want = plain_logits(name, dtype, tokens)
    whole = run_whole(runner, "whole", tokens)
    for sizes in ([16, 2, 7, 64, 3, 2, 1, 30], [2], [63, 1, 64, 2], [3, 65]):
        got = run_portions(runner, "p", tokens, sizes)
        assert_close(got, want, TOL_ORACLE[dtype], f"{name} {dtype} portions {sizes}")
        assert_close(got, whole, TOL_CUTS[dtype], f"{name} {dtype} portions {sizes} vs whole")
    runner.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_with_pages_used_again(name, dtype):
    lengths = [150, 90, 200, 70, 130, 64, 33, 180]
    num_pages = 9                         # 8 requests need 18 pages in all: pages come back
    steps, tokens = mixed_trace(lengths, TINY[name]["vocab_size"], num_pages, seed=5)
    runner = new_runner(name, dtype, num_pages=num_pages, num_slots=4)
    got = replay_in_process(runner, steps)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"])
    # 18 pages of requests went through a pool of 9: every page id was handed out again
    assert 7 <= runner.cache.groups[0].pool.high_water <= num_pages
    assert runner.cache.slots_high_water == 4
    for rid, toks in tokens.items():
        assert_close(got[rid], plain_logits(name, dtype, toks), TOL_ORACLE[dtype],
                     f"{name} {dtype} mixed, request {rid} of {len(toks)}")
    assert runner.cache.groups[0].pool.n_used == 0 and runner.cache.free_slots == 4


@pytest.mark.parametrize("name,dtype", CASES)
def test_long_decoding(name, dtype):
    runner = new_runner(name, dtype)
    tokens = random_tokens(name, 330, seed=14)
    want = plain_logits(name, dtype, tokens)
    parts = [runner.step([("l", tokens[:3], [0, 1, 2])]).cpu().numpy()]
    for token in tokens[3:]:
        parts.append(runner.step([("l", [token], [0])]).cpu().numpy())
    runner.finish("l")
    assert_close(np.concatenate(parts), want, TOL_ORACLE[dtype], f"{name} {dtype} 327 decode steps")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_decoding_at_a_context_of_four_thousand_tokens(name, dtype):
    """Sixty-two pages of context: a prompt of 3,900 tokens in portions of 1,000, then 60 tokens
    one by one, the context cut into slices that a cluster merges, graphs of a wide block table;
    another request decodes beside it at a short context (its rows of the table are mostly empty)."""
    runner = new_runner(name, dtype, num_pages=70, num_slots=2, max_model_len=4000)
    tokens = random_tokens(name, 3960, seed=31)
    short = random_tokens(name, 80, seed=32)
    want, want_short = plain_logits(name, dtype, tokens), plain_logits(name, dtype, short)
    got = []
    for start in range(0, 3900, 1000):
        stop = min(start + 1000, 3900)
        got.append(runner.step([("l", tokens[start:stop], [0, stop - start - 1])]).cpu().numpy())
    assert_close(np.concatenate(got), want[[0, 999, 1000, 1999, 2000, 2999, 3000, 3899]], TOL_ORACLE[dtype],
                 f"{name} {dtype} portions of a long prompt")
    runner.step([("s", short[:20], [])])
    got_long, got_short = [], []
    for i in range(60):
        out = runner.step([("l", [tokens[3900 + i]], [0]), ("s", [short[20 + i]], [0])]).cpu().numpy()
        got_long.append(out[0])
        got_short.append(out[1])
    assert_close(np.stack(got_long), want[3900:], TOL_ORACLE[dtype], f"{name} {dtype} decoding at 3,900 tokens")
    assert_close(np.stack(got_short), want_short[20:], TOL_ORACLE[dtype], f"{name} {dtype} its short neighbour")
    runner.finish("l")
    runner.finish("s")
    runner.cache.check()
    runner.check_health()


@pytest.mark.parametrize("name,dtype", CASES)
def test_the_first_tokens_of_a_sequence(name, dtype):
    runner = new_runner(name, dtype)
    tokens = random_tokens(name, 6, seed=15)
    want = plain_logits(name, dtype, tokens)
    for length in (1, 2, 3):
        got = run_whole(runner, f"f{length}", tokens[:length])
        assert_close(got, want[:length], TOL_ORACLE[dtype], f"{name} {dtype} prompt of {length}")
    got = run_portions(runner, "one", tokens, [1])
    assert_close(got, want, TOL_ORACLE[dtype], f"{name} {dtype} token by token from position 0")
    # several one-token requests in one batch
    out = runner.step([(f"s{i}", [tokens[0]], [0]) for i in range(4)]).cpu().numpy()
    for i in range(4):
        runner.finish(f"s{i}")
        assert_close(out[i:i + 1], want[:1], TOL_ORACLE[dtype], f"{name} {dtype} batch of first tokens")


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("A", "bfloat16")])
def test_trace_run_program(name, dtype, tmp_path):
    lengths = [100, 70, 130, 66, 40]
    num_pages = 6
    steps, tokens = mixed_trace(lengths, TINY[name]["vocab_size"], num_pages, seed=8)
    trace = "".join(json.dumps(step) + "\n" for step in steps)
    out_dir = tmp_path / "logits"
    env = dict(os.environ)
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir(name, dtype)),
         "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(num_pages * 64)],
        input=trace, capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    vocab = TINY[name]["vocab_size"]
    got = {}
    for step in steps:
        data = np.fromfile(out_dir / f"{step['step']}.f32", dtype="<f4").reshape(-1, vocab)
        row = 0
        for e in step["entries"]:
            got.setdefault(e["id"], []).append(data[row:row + len(e["want"])])
            row += len(e["want"])
        assert row == data.shape[0]
    for rid, toks in tokens.items():
        assert_close(np.concatenate(got[rid]), plain_logits(name, dtype, toks), TOL_ORACLE[dtype],
                     f"trace_run {name} {dtype} request {rid}")


def test_a_step_that_wants_nothing_writes_nothing_and_refusals_are_clean(tmp_path):
    from flyweight_b200.cache import OutOfPages
    from flyweight_b200.engine import StepError
    runner = new_runner("A", "float32", num_pages=2)
    tokens = random_tokens("A", 70, seed=1)
    assert runner.step([("q", tokens[:10], [])]).shape == (0, 256)
    with pytest.raises(StepError, match="outside"):
        runner.step([("q", [999], [0])])
    with pytest.raises(StepError, match="brings no tokens"):
        runner.step([("q", [], [])])
    with pytest.raises(OutOfPages):
        runner.step([("q", tokens[10:], []), ("z", tokens * 2, [])])
    assert runner.cache.length("q") == 10 and not runner.cache.has("z")
    got = runner.step([("q", tokens[10:], [59])]).cpu().numpy()
    assert_close(got, plain_logits("A", "float32", tokens)[-1:], TOL_ORACLE["float32"], "after refusals")


@pytest.mark.parametrize("name", ["A", "B"])
def test_bfloat16_cuts_agree_to_one_roundoff_when_the_sums_keep_one_order(name):
    """The bfloat16 kernels' own cache and batch logic, checked as sharply as in 32-bit: with
    the split-K factor pinned, whole, decoded, portioned and mixed runs must agree to one
    bfloat16 unit roundoff of the logit scale.  (The split-context decode kernel is checked
    against float64 in test_kernels_gpu.py and against the oracle in the tests above.)"""
    from flyweight_b200.kernels import attention, tensorcore
    dtype = "bfloat16"
    tensorcore.force_splits(1)
    tensorcore.set_norm_fusion(False)   # a norm folded into its product rounds bf16(x*w), the norm kernel bf16(x*r*w)
    attention.force_tiled(True)         # the decode kernel merges key slices in another order
    try:
        runner = new_runner(name, dtype)
        runner.use_graphs = False
        tokens = random_tokens(name, 200, seed=21)
        whole = run_whole(runner, "whole", tokens)
        for sizes in ([1], [2], [16, 2, 7, 64, 3, 2, 1, 30], [63, 1, 64, 2]):
            got = run_portions(runner, "p", tokens, sizes)
            assert_close(got, whole, TOL_CUTS_PINNED[dtype], f"{name} pinned portions {sizes}")
        steps, toks = mixed_trace([150, 90, 200, 70], TINY[name]["vocab_size"], 9, seed=6)
        got = replay_in_process(runner, steps)
        for rid, seq in toks.items():
            assert_close(got[rid], run_whole(runner, "w" + rid, seq), TOL_CUTS_PINNED[dtype],
                         f"{name} pinned mixed {rid}")
    finally:
        tensorcore.force_splits(None)
        tensorcore.set_norm_fusion(True)
        attention.force_tiled(False)


@pytest.mark.parametrize("name", ["A", "B"])
def test_decoding_requests_at_the_head_of_a_mixed_step(name):
    """Three requests decode beside portions of a fourth: their tokens, first in the step, run
    the split-context kernel and the portions the tiled one, into one output; with the split
    switched off the tiled kernel runs all of it.  Both follow the plain implementation."""
    from flyweight_b200.kernels import attention
    dtype = "bfloat16"
    seqs = [random_tokens(name, n, seed=40 + i) for i, n in enumerate((150, 97, 70, 130))]
    want = [plain_logits(name, dtype, s) for s in seqs]
    tail = 20
    results = {}
    for split in (True, False):
        attention.set_mixed_split(split)
        try:
            runner = new_runner(name, dtype, num_pages=16, num_slots=4)
            runner.use_graphs = False
            for i in range(3):
                runner.step([(f"d{i}", seqs[i][:-tail], [])])
            got = {i: [] for i in range(4)}
            pos = 0
            for k in range(tail):
                entries = [(f"d{i}", [seqs[i][len(seqs[i]) - tail + k]], [0]) for i in range(3)]
                portion = seqs[3][pos:pos + (7, 2, 16, 1, 9)[k % 5]]
                if portion:
                    entries.append(("p", portion, list(range(len(portion)))))
                    pos += len(portion)
                out = runner.step(entries).cpu().numpy()
                for i in range(3):
                    got[i].append(out[i:i + 1])
                if portion:
                    got[3].append(out[3:])
            for i in range(3):
                assert_close(np.concatenate(got[i]), want[i][-tail:], TOL_ORACLE[dtype],
                             f"{name} split={split}: decoding request {i} in mixed steps")
            assert_close(np.concatenate(got[3]), want[3][:pos], TOL_ORACLE[dtype],
                         f"{name} split={split}: portions beside decoding requests")
            results[split] = np.concatenate([np.concatenate(got[i]) for i in range(4)])
            runner.cache.check()
        finally:
            attention.set_mixed_split(True)
    assert_close(results[True], results[False], TOL_CUTS[dtype], f"{name} split on against off")
