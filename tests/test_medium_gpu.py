"""A middle-sized LFM2 (hidden 1024, 16 heads in 4 groups of head size 64, feed-forward width
2816, vocabulary 4099) at which the bfloat16 kernels run the tile shapes they run on real models:
256-token tiles, two accumulators, cluster split-K, 64-key attention tiles over a dozen pages.
The plain float64 implementation would take minutes here, so the oracle is the engine's own
32-bit path (itself checked against the plain implementation on the tiny configurations) on the
same bfloat16-rounded weights."""
import numpy as np
import pytest
import torch

from gpu_util import TOL_CUTS, TOL_ORACLE, assert_close, mixed_trace, replay_in_process
from tiny_configs import make_model_dir

pytestmark = pytest.mark.gpu

MEDIUM = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "num_hidden_layers": 3,
    "layer_types": ["conv", "full_attention", "conv"], "hidden_size": 1024,
    "num_attention_heads": 16, "num_key_value_heads": 4, "intermediate_size": 2816,
    "block_auto_adjust_ff_dim": False, "conv_L_cache": 3, "conv_bias": False, "vocab_size": 4099,
    "rope_theta": 1000000.0, "norm_eps": 1e-5, "max_position_embeddings": 8192,
    "tie_embedding": True,
}


@pytest.fixture(scope="module")
def runners(tmp_path_factory):
    from flyweight_b200.engine import ModelRunner, load_model
    folder = make_model_dir(tmp_path_factory.mktemp("medium"), MEDIUM, seed=4, dtype=torch.bfloat16)
    made = {}
    for dtype in ("float32", "bfloat16"):
        model = load_model(folder, dtype)
        made[dtype] = ModelRunner(model, num_pages=40, num_slots=4, max_model_len=2048,
                                  max_batched_tokens=4096)
    return made


def test_bfloat16_follows_the_32_bit_path_at_real_tile_shapes(runners):
    rng = np.random.default_rng(0)
    tokens = [int(t) for t in rng.integers(0, MEDIUM["vocab_size"], size=700)]
    want_rows = list(range(0, 700, 7)) + [699]
    oracle = runners["float32"].step([("o", tokens, want_rows)]).cpu().numpy()
    runners["float32"].finish("o")
    runner = runners["bfloat16"]
    whole = runner.step([("w", tokens, want_rows)]).cpu().numpy()
    runner.finish("w")
    assert_close(whole, oracle, TOL_ORACLE["bfloat16"], "medium, whole prompt")
    # 600 tokens in portions of 256 (full tiles) and a ragged tail, then 100 decode steps
    parts = []
    for start, stop in ((0, 256), (256, 512), (512, 600)):
        want = [r - start for r in want_rows if start <= r < stop]
        parts.append(runner.step([("p", tokens[start:stop], want)]).cpu().numpy())
    for position in range(600, 700):
        out = runner.step([("p", [tokens[position]], [0])]).cpu().numpy()
        if position in want_rows:
            parts.append(out)
    runner.finish("p")
    got = np.concatenate(parts)
    assert_close(got, oracle, TOL_ORACLE["bfloat16"], "medium, portions then decode")
    assert_close(got, whole, TOL_CUTS["bfloat16"], "medium, cuts")


def test_mixed_batches_at_real_tile_shapes(runners):
    steps, tokens = mixed_trace([300, 520, 130, 410, 260], MEDIUM["vocab_size"], 24, seed=3, tail=8)
    for step in steps:                       # fewer logits: the last place of every entry
        for entry in step["entries"]:
            entry["want"] = [len(entry["tokens"]) - 1]
    got = replay_in_process(runners["bfloat16"], steps)
    want = replay_in_process(runners["float32"], steps)
    for rid in tokens:
        assert_close(got[rid], want[rid], TOL_ORACLE["bfloat16"], f"medium mixed {rid}")


def test_a_hundred_tokens_against_a_wide_feed_forward(tmp_path):
    """A feed-forward width of 4,352: at 65 to a few hundred tokens its down projection (long K,
    few output tiles) runs 128-token tiles with K cut across a cluster; the 32-bit path is the
    oracle, and the portions must agree with the whole prompt."""
    from flyweight_b200.engine import ModelRunner, load_model
    from flyweight_b200.kernels import tensorcore
    config = dict(MEDIUM, num_hidden_layers=2, layer_types=["conv", "full_attention"],
                  intermediate_size=4352)
    assert tensorcore.mid_size_choice(100, 1024, 4352, 1, False)[2] > 1
    folder = make_model_dir(tmp_path / "wide", config, seed=6, dtype=torch.bfloat16)
    made = {dtype: ModelRunner(load_model(folder, dtype), num_pages=12, num_slots=2, max_model_len=512,
                               max_batched_tokens=512) for dtype in ("float32", "bfloat16")}
    rng = np.random.default_rng(1)
    tokens = [int(t) for t in rng.integers(0, config["vocab_size"], size=300)]
    rows = list(range(0, 300, 5)) + [299]
    oracle = made["float32"].step([("o", tokens, rows)]).cpu().numpy()
    runner = made["bfloat16"]
    whole = runner.step([("w", tokens, rows)]).cpu().numpy()
    runner.finish("w")
    assert_close(whole, oracle, TOL_ORACLE["bfloat16"], "wide feed-forward, 300 tokens at once")
    parts = []
    for start, stop in ((0, 100), (100, 228), (228, 300)):          # 100, 128 and 72 tokens
        want = [r - start for r in rows if start <= r < stop]
        parts.append(runner.step([("p", tokens[start:stop], want)]).cpu().numpy())
    runner.finish("p")
    got = np.concatenate(parts)
    assert_close(got, oracle, TOL_ORACLE["bfloat16"], "wide feed-forward, portions of about a hundred")
    assert_close(got, whole, TOL_CUTS["bfloat16"], "wide feed-forward, cuts")
    assert tensorcore.status() == 0
