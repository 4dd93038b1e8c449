"""The engine against the plain implementation at the layer sizes of LFM2-1.2B: hidden 2048,
32 heads on 8 KV heads of size 64, ``intermediate_size`` 12288 auto-adjusted to a feed-forward
width of 8192, 3 taps, vocabulary 65,536 -- the shapes at which 256-token product tiles, CTA
pairs, the wave cut, 8-way cluster split-K and the 128-row tcgen05 attention tiles all run.
LFM2-1.2B has 16 layers; this model has 4 of them (conv, attention, conv, attention) so that a
float64 forward of a few thousand tokens stays a matter of seconds.

The oracle is ``plain_lfm2_torch`` (float64, whole sequences, no cache; the same formulas as
``plain_lfm2``, checked against it on the CPU), reading the same model folder as the engine.
Requests are long enough to fill the large tiles (600 tokens and more) and run whole, as one
long step and the last 32 tokens singly, in portions down to two tokens, and mixed with up to
four live requests through a pool so small that pages come back; in 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

import plain_lfm2_torch as PT
from gpu_util import TOL_CUTS, TOL_ORACLE, assert_close, mixed_trace, replay_in_process
from tiny_configs import make_model_dir

pytestmark = pytest.mark.gpu

LAYERS_OF_LFM2_1P2B = 16
REAL = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "num_hidden_layers": 4,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"], "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "intermediate_size": 12288,
    "block_auto_adjust_ff_dim": True, "block_multiple_of": 256, "conv_L_cache": 3,
    "conv_bias": False, "vocab_size": 65536, "rope_theta": 1000000.0, "norm_eps": 1e-5,
    "max_position_embeddings": 128000, "tie_embedding": True,
}
DTYPES = ("float32", "bfloat16")
# The other two sizes of the family (their own feed-forward widths, head counts and groups), two
# layers each: LFM2-350M has 16 query heads on 8 KV heads (two per group: 64-token attention
# tiles) and a width of 4,608; LFM2-2.6B as the baseline states it has a width of 7,168.
OTHERS = {
    "lfm2-350m": dict(REAL, num_hidden_layers=2, layer_types=["full_attention", "conv"], hidden_size=1024,
                      num_attention_heads=16, intermediate_size=6656),
    "lfm2-2.6b": dict(REAL, num_hidden_layers=2, layer_types=["conv", "full_attention"], intermediate_size=10752),
}


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    assert REAL["num_hidden_layers"] < LAYERS_OF_LFM2_1P2B
    return make_model_dir(tmp_path_factory.mktemp("real"), REAL, seed=11, dtype=torch.bfloat16)


@pytest.fixture(scope="module")
def oracle(folder):
    cfg, weights = PT.load_model_dir(folder, "cuda")
    assert weights["model.layers.0.feed_forward.w1.weight"].shape == (8192, 2048)
    cache = {}

    def logits(tokens, rows):
        key = (tuple(tokens), tuple(rows))
        if key not in cache:
            cache[key] = PT.forward(cfg, weights, tokens, rows=rows)
        return cache[key]
    return logits


@pytest.fixture(scope="module")
def runners(folder):
    from flyweight_b200.engine import ModelRunner, load_model
    made = {}

    def runner(dtype):
        if dtype not in made:
            made[dtype] = ModelRunner(load_model(folder, dtype), num_pages=32, num_slots=4,
                                      max_model_len=2048, max_batched_tokens=4096)
        return made[dtype]
    return runner


def _tokens(length, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, REAL["vocab_size"], size=length)]


def _run(runner, rid, tokens, sizes, rows):
    """Feed ``tokens`` in steps of the given sizes (the last size repeats), asking for the logits
    at the positions ``rows``; returns them in position order."""
    outs, pos, i = [], 0, 0
    while pos < len(tokens):
        n = min(sizes[min(i, len(sizes) - 1)], len(tokens) - pos)
        want = [r - pos for r in rows if pos <= r < pos + n]
        out = runner.step([(rid, tokens[pos:pos + n], want)])
        if want:
            outs.append(out.cpu().numpy())
        pos += n
        i += 1
    runner.finish(rid)
    runner.cache.check()
    return np.concatenate(outs)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_then_decoded_then_in_portions(dtype, runners, oracle):
    from flyweight_b200.kernels import tensorcore
    runner = runners(dtype)
    tokens = _tokens(700, seed=21)
    rows = sorted(set(range(0, 700, 9)) | set(range(660, 700)))
    want = oracle(tokens, rows)
    whole = _run(runner, "whole", tokens, [700], rows)
    assert_close(whole, want, TOL_ORACLE[dtype], f"real sizes {dtype}: whole request")
    decoded = _run(runner, "decoded", tokens, [668, 1], rows)
    assert_close(decoded, want, TOL_ORACLE[dtype], f"real sizes {dtype}: 668 tokens, then 32 singly")
    assert_close(decoded, whole, TOL_CUTS[dtype], f"real sizes {dtype}: decoded against whole")
    # full 256-token tiles, a ragged middle, two-token portions, a page edge in a portion
    sizes = [256, 2, 130, 7, 64, 3, 2, 1, 129, 2, 40, 2, 2, 60]
    assert sum(sizes) == 700
    portions = _run(runner, "portions", tokens, sizes, rows)
    assert_close(portions, want, TOL_ORACLE[dtype], f"real sizes {dtype}: portions of changing size")
    assert_close(portions, whole, TOL_CUTS[dtype], f"real sizes {dtype}: portions against whole")
    assert tensorcore.status() == 0
    runner.check_health()


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_with_pages_that_come_back(dtype, runners, oracle):
    runner = runners(dtype)
    lengths = [300, 650, 130, 400, 700, 260, 520]
    steps, tokens = mixed_trace(lengths, REAL["vocab_size"], num_pages=32, seed=5, tail=12,
                                sizes=(1, 2, 3, 7, 16, 33, 64, 2, 5, 130, 256))
    assert sum(-(-n // 64) for n in lengths) > 32          # the pool is smaller than their sum
    rows = {rid: [] for rid in tokens}
    position = {rid: 0 for rid in tokens}
    for step in steps:                                    # the last place of every entry only
        for entry in step["entries"]:
            entry["want"] = [len(entry["tokens"]) - 1]
            position[entry["id"]] += len(entry["tokens"])
            rows[entry["id"]].append(position[entry["id"]] - 1)
    assert max(len(step["entries"]) for step in steps) == 4
    got = replay_in_process(runner, steps)
    for rid in tokens:
        assert_close(got[rid], oracle(tokens[rid], rows[rid]), TOL_ORACLE[dtype],
                     f"real sizes {dtype}: mixed, request {rid}")
    assert runner.cache.stats()["groups"][0]["pages_in_use"] == 0
    runner.check_health()


@pytest.mark.parametrize("size", sorted(OTHERS))
def test_the_other_sizes_of_the_family_in_bfloat16(size, tmp_path):
    """Layer sizes of LFM2-350M and LFM2-2.6B (two layers each): whole, decoded and in portions
    against the float64 oracle, in the precision that serves."""
    from flyweight_b200.engine import ModelRunner, load_model
    config = OTHERS[size]
    folder = make_model_dir(tmp_path / size, config, seed=13, dtype=torch.bfloat16)
    cfg, weights = PT.load_model_dir(folder, "cuda")
    assert weights["model.layers.0.feed_forward.w1.weight"].shape[0] == {"lfm2-350m": 4608, "lfm2-2.6b": 7168}[size]
    runner = ModelRunner(load_model(folder, "bfloat16"), num_pages=12, num_slots=2, max_model_len=1024,
                         max_batched_tokens=1024)
    tokens = _tokens(600, seed=22)
    rows = sorted(set(range(0, 600, 11)) | set(range(560, 600)))
    want = PT.forward(cfg, weights, tokens, rows=rows)
    whole = _run(runner, "whole", tokens, [600], rows)
    assert_close(whole, want, TOL_ORACLE["bfloat16"], f"{size}: whole request")
    decoded = _run(runner, "decoded", tokens, [568, 1], rows)
    assert_close(decoded, want, TOL_ORACLE["bfloat16"], f"{size}: 568 tokens, then 32 singly")
    portions = _run(runner, "portions", tokens, [300, 2, 100, 64, 129, 5], rows)
    assert_close(portions, want, TOL_ORACLE["bfloat16"], f"{size}: portions")
    assert_close(portions, whole, TOL_CUTS["bfloat16"], f"{size}: portions against whole")
    runner.check_health()
