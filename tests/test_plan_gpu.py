"""The native step plan against the Python path: the same model, the same steps, once launched
kernel by kernel from the parts' ``forward`` and once as one native call per step.  Both make
the same kernel choices by the same rules, so logits, key/value pages and conv states must be
equal bit for bit: at every token count that switches a rule (15/16/17 tokens, 32/33, 64/65,
128/129, 256+), for decoding requests beside prompt portions, with the switches that tests use
turned on, and in both precisions."""
import numpy as np
import pytest
import torch

from gpu_util import engine_model, mixed_trace, random_tokens
from tiny_configs import TINY, make_model_dir

pytestmark = pytest.mark.gpu


def pair_of_runners(model, num_pages=24, num_slots=6, max_model_len=1024, max_batched_tokens=1024):
    from flyweight_b200.engine import ModelRunner
    made = [ModelRunner(model, num_pages=num_pages, num_slots=num_slots, max_model_len=max_model_len,
                        max_batched_tokens=max_batched_tokens, use_graphs=False, use_plan=use_plan)
            for use_plan in (False, True)]
    assert made[0].step_plan is None and made[1].step_plan is not None, getattr(model, "not_plannable", "")
    return made


def same_steps(runners, steps, what):
    """Run the trace through both runners; every step's logits must be the same bits."""
    for index, step in enumerate(steps):
        outs = [r.step([(e["id"], e["tokens"], e["want"]) for e in step["entries"]]) for r in runners]
        assert torch.equal(outs[0], outs[1]), f"{what}: step {index} ({[len(e['tokens']) for e in step['entries']]} tokens)"
        for r in runners:
            for rid in step["end"]:
                r.finish(rid)
    eager, planned = runners
    for a, b in zip(eager.cache.layer_caches, planned.cache.layer_caches):
        for name in ("k_pool", "v_pool", "state"):
            ta, tb = getattr(a, name), getattr(b, name)
            if ta is not None:
                assert torch.equal(ta, tb), f"{what}: {name} differs after the trace"


def counted_steps(name, counts, seed):
    """One request fed in portions of the given sizes (all logits wanted), then ended."""
    tokens = random_tokens(name, sum(counts), seed)
    steps, at = [], 0
    for n in counts:
        steps.append({"entries": [{"id": "p", "tokens": tokens[at:at + n], "want": list(range(n))}], "end": []})
        at += n
    steps[-1]["end"] = ["p"]
    return steps


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_models_step_for_step(name, dtype):
    runners = pair_of_runners(engine_model(name, dtype))
    same_steps(runners, counted_steps(name, [150], 1), f"{name} {dtype} whole")
    same_steps(runners, counted_steps(name, [1, 1, 2, 15, 16, 17, 31, 33, 64, 65, 1, 1, 128, 129, 3], 2),
               f"{name} {dtype} portions")
    steps, _ = mixed_trace([70, 150, 33, 200, 90, 130], TINY[name]["vocab_size"], num_pages=9, seed=4, tail=20)
    same_steps(runners, steps, f"{name} {dtype} mixed")
    for r in runners:
        r.cache.check()
        r.check_health()
    assert runners[1].step_plan.n_ops > 10


def test_decoding_requests_at_the_head_of_a_step_beside_portions():
    """What the scheduler builds: single tokens of running requests first, portions behind them."""
    name = "B"
    runners = pair_of_runners(engine_model(name, "bfloat16"))
    vocab = TINY[name]["vocab_size"]
    rng = np.random.default_rng(7)
    draw = lambda n: [int(t) for t in rng.integers(0, vocab, size=n)]
    steps = [{"entries": [{"id": f"d{i}", "tokens": draw(40 + 30 * i), "want": []} for i in range(3)], "end": []}]
    for k in range(6):
        entries = [{"id": f"d{i}", "tokens": draw(1), "want": [0]} for i in range(3)]
        entries.append({"id": "p", "tokens": draw([70, 2, 64, 129, 1, 5][k]), "want": [0]})
        steps.append({"entries": entries, "end": []})
    steps[-1]["end"] = ["d0", "d1", "d2", "p"]
    same_steps(runners, steps, "singles then a portion")


@pytest.mark.parametrize("switch", ["fuse_always", "pinned", "no_tensor_cores", "no_mixed_split"])
def test_the_switches_reach_both_paths(switch):
    from flyweight_b200.kernels import attention, tensorcore
    name = "A"
    runners = pair_of_runners(engine_model(name, "bfloat16"))
    undo = []
    try:
        if switch == "fuse_always":
            tensorcore.fuse_always(True)
            undo.append(lambda: tensorcore.fuse_always(False))
        elif switch == "pinned":
            tensorcore.force_splits(1)
            attention.force_tiled(True)
            tensorcore.set_norm_fusion(False)
            undo += [lambda: tensorcore.force_splits(None), lambda: attention.force_tiled(False),
                     lambda: tensorcore.set_norm_fusion(True)]
        elif switch == "no_tensor_cores":
            tensorcore.set_enabled(False)
            attention.set_mma_enabled(False)
            undo += [lambda: tensorcore.set_enabled(True), lambda: attention.set_mma_enabled(True)]
        else:
            attention.set_mixed_split(False)
            undo.append(lambda: attention.set_mixed_split(True))
        same_steps(runners, counted_steps(name, [3, 16, 1, 40, 1, 1, 70, 130], 5), switch)
        steps, _ = mixed_trace([70, 150, 33, 90], TINY[name]["vocab_size"], num_pages=8, seed=6, tail=10)
        same_steps(runners, steps, f"{switch}, mixed")
    finally:
        for step in undo:
            step()


MEDIUM = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2", "num_hidden_layers": 3,
    "layer_types": ["conv", "full_attention", "conv"], "hidden_size": 1024,
    "num_attention_heads": 16, "num_key_value_heads": 4, "intermediate_size": 4352,
    "block_auto_adjust_ff_dim": False, "conv_L_cache": 3, "conv_bias": False, "vocab_size": 4099,
    "rope_theta": 1000000.0, "norm_eps": 1e-5, "max_position_embeddings": 8192, "tie_embedding": True,
}


def test_real_tile_shapes_step_for_step(tmp_path):
    """Hidden 1024, a feed-forward of 4,352: CTA pairs, the wave cut, 128-token tiles with a split K,
    the tcgen05 attention kernel and the split decode kernel with a merge kernel (a context of a
    few thousand tokens) all run, chosen once by Python and once by the library."""
    from flyweight_b200.engine import load_model
    folder = make_model_dir(tmp_path / "medium", MEDIUM, seed=8, dtype=torch.bfloat16)
    model = load_model(folder, "bfloat16")
    runners = pair_of_runners(model, num_pages=80, num_slots=4, max_model_len=4096, max_batched_tokens=2048)
    rng = np.random.default_rng(3)
    draw = lambda n: [int(t) for t in rng.integers(0, MEDIUM["vocab_size"], size=n)]
    steps = []
    for n in (700, 256, 100, 64, 33, 17, 16, 8, 1, 300, 513, 2048):
        steps.append({"entries": [{"id": "a", "tokens": draw(n), "want": sorted({0, n - 1})}], "end": []})
    steps[-1]["end"] = ["a"]
    same_steps(runners, steps, "medium, one request")
    # three requests decoding at a long context beside a portion of a fourth
    steps = [{"entries": [{"id": f"d{i}", "tokens": draw(900 + 100 * i), "want": []}], "end": []} for i in range(3)]
    for k in range(4):
        entries = [{"id": f"d{i}", "tokens": draw(1), "want": [0]} for i in range(3)]
        if k < 3:
            entries.append({"id": "p", "tokens": draw([300, 40, 129][k]), "want": [0]})
        steps.append({"entries": entries, "end": []})
    steps[-1]["end"] = ["d0", "d1", "d2", "p"]
    same_steps(runners, steps, "medium, mixed")
    for r in runners:
        r.check_health()


def test_decoding_requests_whose_slices_a_second_kernel_merges(tmp_path):
    """Two requests of 8,300 cached tokens decode together: few CTAs and a long context, so it is cut into
    more slices than a cluster merges, and the slices go through scratch memory (the plan's own, inside
    its arena) and a merge kernel.  And 36 requests of 1,900 tokens: slices that a cluster merges."""
    from flyweight_b200.engine import load_model
    from flyweight_b200.kernels import attention
    folder = make_model_dir(tmp_path / "medium", dict(MEDIUM, num_hidden_layers=2, layer_types=["full_attention", "conv"],
                                                      max_position_embeddings=16384),
                            seed=9, dtype=torch.bfloat16)
    model = load_model(folder, "bfloat16")
    n_kv, head_dim = MEDIUM["num_key_value_heads"], MEDIUM["hidden_size"] // MEDIUM["num_attention_heads"]
    rng = np.random.default_rng(5)
    draw = lambda n: [int(t) for t in rng.integers(0, MEDIUM["vocab_size"], size=n)]
    for count, length, merged_by_cluster in ((2, 8300, False), (36, 1900, True)):
        splits, _, in_cluster = attention.decode_splits(count, n_kv, -(-(length + 3) // 64), head_dim)
        assert splits > 1 and in_cluster == merged_by_cluster, (count, length, splits, in_cluster)
        runners = pair_of_runners(model, num_pages=count * (length // 64 + 2), num_slots=40, max_model_len=8400,
                                  max_batched_tokens=4096)
        steps = []
        for i in range(count):
            prompt = draw(length)
            for start in range(0, length, 4096):
                steps.append({"entries": [{"id": f"d{i}", "tokens": prompt[start:start + 4096], "want": []}], "end": []})
        for _ in range(3):
            steps.append({"entries": [{"id": f"d{i}", "tokens": draw(1), "want": [0]} for i in range(count)], "end": []})
        steps[-1]["end"] = [f"d{i}" for i in range(count)]
        same_steps(runners, steps, f"{count} decoding requests of {length} tokens")


def test_a_model_with_a_part_defined_elsewhere_keeps_the_python_path():
    from test_parts_gpu import toy_architecture
    from flyweight_b200.engine import ModelRunner, random_model
    raw = toy_architecture()
    model = random_model(raw, seed=1, dtype="float32", preset="unit", stored_dtype=torch.float32)
    runner = ModelRunner(model, num_pages=4, num_slots=2, max_model_len=128)
    assert runner.step_plan is None and "toy_decay" in model.not_plannable
    out = runner.step([("a", [1, 2, 3], [2])])
    assert out.shape == (1, raw["vocab_size"]) and torch.isfinite(out).all()
