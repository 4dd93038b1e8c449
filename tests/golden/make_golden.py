"""Anchor the plain implementation on yairpatch/flyweight's own float64 LFM2 forward.

Run once, where the reference tree is at hand:

    python tests/golden/make_golden.py /path/to/flyweight

It imports ``tests/lfm2_gguf_fixture.py`` FROM THAT TREE (nothing of it is copied
here), lets it draw the weights of two small dense-LFM2 geometries and run its own
``reference_greedy``, renames the tensors from their GGUF names to the checkpoint
names the plain implementation reads, and stores weights, prompts and the reference's
greedy tokens in ``lfm2_reference_greedy.npz``.  ``tests/test_plain_reference.py``
then checks, without the reference tree, that ``plain_lfm2`` gives the same tokens.

What this anchors: layer order, the B|C|x split, tap order, half-split rope pairing
and frequencies, q/k norm placement, the GQA head mapping, the tied head and the
final norm.  What the reference's fixture cannot express (conv bias, untied head,
another eps, logits) rests on the formulas cited in ``plain_lfm2.py``.
"""
import importlib.util
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

import plain_lfm2  # noqa: E402

GEOMETRIES = {
    # name: (fixture keyword arguments, attention layers)
    "g1": (dict(hidden=32, layers=4, dense_intermediate=48, heads=4, kv_heads=2, conv_kernel=3,
                rope_theta=100.0), (1, 3)),
    "g2": (dict(hidden=48, layers=5, dense_intermediate=80, heads=3, kv_heads=1, conv_kernel=4,
                rope_theta=10000.0), (0, 2, 4)),
}


def gguf_to_hf(name: str) -> str:
    table = {
        "token_embd.weight": "model.embed_tokens.weight",
        "token_embd_norm.weight": "model.embedding_norm.weight",
    }
    if name in table:
        return table[name]
    _, layer, rest = name.split(".", 2)
    rest = {
        "attn_norm.weight": "operator_norm.weight",
        "attn_q.weight": "self_attn.q_proj.weight",
        "attn_k.weight": "self_attn.k_proj.weight",
        "attn_v.weight": "self_attn.v_proj.weight",
        "attn_output.weight": "self_attn.out_proj.weight",
        "attn_q_norm.weight": "self_attn.q_layernorm.weight",
        "attn_k_norm.weight": "self_attn.k_layernorm.weight",
        "shortconv.in_proj.weight": "conv.in_proj.weight",
        "shortconv.out_proj.weight": "conv.out_proj.weight",
        "shortconv.conv.weight": "conv.conv.weight",
        "ffn_norm.weight": "ffn_norm.weight",
        "ffn_gate.weight": "feed_forward.w1.weight",
        "ffn_up.weight": "feed_forward.w3.weight",
        "ffn_down.weight": "feed_forward.w2.weight",
    }[rest]
    return f"model.layers.{layer}.{rest}"


def main(reference_root: str) -> None:
    path = Path(reference_root) / "tests" / "lfm2_gguf_fixture.py"
    spec = importlib.util.spec_from_file_location("lfm2_gguf_fixture", path)
    fixture = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fixture)
    out = {}
    for name, (kwargs, attention_layers) in GEOMETRIES.items():
        class Spec(fixture.Lfm2Spec):
            def is_attention(self, layer, _layers=attention_layers):
                return layer in _layers
        geometry = Spec(architecture="lfm2", **kwargs)
        with tempfile.TemporaryDirectory() as tmp:
            geometry, weights = fixture.build_lfm2_gguf(Path(tmp) / "m.gguf", geometry, seed=11)
        rng = np.random.default_rng(3)
        prompt = [int(v) for v in rng.integers(0, geometry.vocabulary, size=19)]
        tokens = fixture.reference_greedy(geometry, weights, prompt, 12)
        config = {
            "architectures": ["Lfm2ForCausalLM"], "num_hidden_layers": geometry.layers,
            "layer_types": ["full_attention" if geometry.is_attention(i) else "conv"
                            for i in range(geometry.layers)],
            "hidden_size": geometry.hidden, "num_attention_heads": geometry.heads,
            "num_key_value_heads": geometry.kv_heads,
            "intermediate_size": geometry.dense_intermediate, "block_auto_adjust_ff_dim": False,
            "conv_L_cache": geometry.conv_kernel, "conv_bias": False,
            "vocab_size": geometry.vocabulary, "rope_theta": geometry.rope_theta,
            "norm_eps": 1e-5, "tie_embedding": True,
        }
        hf = {gguf_to_hf(k): v.astype(np.float32) for k, v in weights.items()}
        mine = plain_lfm2.greedy_generate(config, {k: v.astype(np.float64) for k, v in hf.items()},
                                          prompt, 12)
        print(name, "reference", tokens, "plain", mine)
        assert mine == tokens, "the plain implementation disagrees with the reference forward"
        import json
        out[f"{name}.config"] = np.frombuffer(json.dumps(config).encode(), dtype=np.uint8)
        out[f"{name}.prompt"] = np.asarray(prompt, dtype=np.int32)
        out[f"{name}.tokens"] = np.asarray(tokens, dtype=np.int32)
        for k, v in hf.items():
            out[f"{name}.w.{k}"] = v
    np.savez_compressed(HERE / "lfm2_reference_greedy.npz", **out)
    print("wrote", HERE / "lfm2_reference_greedy.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/flyweight")
    main(sys.argv[1])
