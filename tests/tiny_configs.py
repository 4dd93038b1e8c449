"""The two tiny LFM2 configurations of the test-suite and helpers to make model folders.

They differ in every size and option: layer order and count, hidden size, heads and
groups (2 and 3 query heads per KV head), head size, feed-forward width (no power of
two), taps, conv bias, vocabulary, rope theta, eps, tied or untied head.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

TINY_A = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "num_hidden_layers": 4, "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 192, "block_auto_adjust_ff_dim": False, "block_multiple_of": 32,
    "conv_L_cache": 3, "conv_bias": False, "vocab_size": 256, "rope_theta": 10000.0,
    "norm_eps": 1e-5, "max_position_embeddings": 4096, "tie_embedding": True,
}

TINY_B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "num_hidden_layers": 6,
    "layer_types": ["full_attention", "conv", "full_attention", "conv", "conv", "full_attention"],
    "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "intermediate_size": 320, "block_auto_adjust_ff_dim": False, "block_multiple_of": 32,
    "conv_L_cache": 4, "conv_bias": True, "vocab_size": 384, "rope_theta": 1000000.0,
    "norm_eps": 1e-6, "max_position_embeddings": 4096, "tie_embedding": False,
}

TINY = {"A": TINY_A, "B": TINY_B}


def make_model_dir(path, config: dict, seed: int, preset: str = "unit",
                   dtype: torch.dtype = torch.float32, edit=None) -> Path:
    """Write config.json + model.safetensors with seeded random weights through the
    framework's own random-weights mode.  ``edit(tensors)`` may change tensors first."""
    from flyweight_b200.config import architecture_name, lookup
    from flyweight_b200.parts import Precision
    from flyweight_b200.weights import random_tensors, write_model_dir
    import flyweight_b200.models  # noqa: F401

    arch = lookup(architecture_name(config))
    typed = arch.config_class.from_dict(config)
    model = arch.model_class(typed, Precision("float32"), torch.device("cpu"))
    tensors = random_tensors(model.declare(), seed, preset, dtype, "cpu")
    if edit is not None:
        edit(tensors)
    return write_model_dir(path, typed.to_dict(), tensors, seed)
