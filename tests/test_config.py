"""Configuration, registry and the model description built from it (no GPU)."""
import json

import pytest

from flyweight_b200.config import (ConfigError, Lfm2Config, UnknownArchitecture, load_config,
                                   lookup)
import flyweight_b200.models  # noqa: F401
from tiny_configs import TINY_A, TINY_B


def base(**over):
    raw = dict(TINY_A)
    raw.update(over)
    return raw


@pytest.mark.parametrize("intermediate,auto,expected", [
    (12288, True, 8192),      # LFM2-1.2B
    (6656, True, 4608),       # LFM2-350M: 4437 -> 4608
    (10752, True, 7168),      # LFM2-2.6B as the benchmark configuration states it
    (192, False, 192),
    (320, False, 320),
    (10752, False, 10752),
])
def test_ffn_width_rule(intermediate, auto, expected):
    cfg = Lfm2Config.from_dict(base(intermediate_size=intermediate, block_auto_adjust_ff_dim=auto,
                                    block_multiple_of=256))
    assert cfg.ffn_dim == expected


def test_ffn_multiplier_applies_after_two_thirds():
    cfg = Lfm2Config.from_dict(base(intermediate_size=3000, block_auto_adjust_ff_dim=True,
                                    block_ffn_dim_multiplier=1.5, block_multiple_of=64))
    assert cfg.ffn_dim == 3008          # 2000 * 1.5 = 3000 -> next multiple of 64


def test_defaults_follow_the_reference():
    raw = base()
    for key in ("norm_eps", "rope_theta", "conv_L_cache", "conv_bias", "tie_embedding"):
        raw.pop(key, None)
    cfg = Lfm2Config.from_dict(raw)
    assert cfg.norm_eps == 1e-6 and cfg.rope_theta == 1e6
    assert cfg.conv_L_cache == 3 and cfg.conv_bias is False and cfg.tie_embedding is True


def test_layer_types_and_full_attn_idxs_agree():
    a = Lfm2Config.from_dict(base())
    raw = base()
    raw.pop("layer_types")
    raw["full_attn_idxs"] = [1, 3]
    b = Lfm2Config.from_dict(raw)
    assert a.layer_types == b.layer_types == ("conv", "full_attention", "conv", "full_attention")
    assert a.attention_layers == (1, 3)


@pytest.mark.parametrize("over,match", [
    (dict(num_attention_heads=5), "multiple of num_attention_heads"),
    (dict(num_key_value_heads=3), "multiple of"),
    (dict(conv_L_cache=1), "conv_L_cache"),
    (dict(layer_types=["conv"]), "layer_types has 1"),
    (dict(layer_types=["conv", "mamba", "conv", "conv"]), "unknown LFM2 layer type"),
    (dict(hidden_size=None), "missing: hidden_size"),
    (dict(full_attn_idxs=[9], layer_types=None), "outside"),
])
def test_bad_configs_are_refused(over, match):
    with pytest.raises(ConfigError, match=match):
        Lfm2Config.from_dict(base(**over))


def test_registry_picks_by_architecture_name(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Lfm2ForCausalLM" and cfg.hidden_size == 96
    assert lookup("Lfm2ForCausalLM").model_class.__name__ == "Lfm2ForCausalLM"


def test_unknown_architecture_names_what_is_supported(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_A, architectures=["Nope"])))
    with pytest.raises(UnknownArchitecture, match="Lfm2ForCausalLM"):
        load_config(tmp_path)


def test_round_trip_through_dict():
    cfg = Lfm2Config.from_dict(TINY_B)
    again = Lfm2Config.from_dict(cfg.to_dict())
    assert cfg == again


def test_model_spec_is_put_together_from_parts():
    spec = Lfm2Config.from_dict(TINY_B).model_spec()
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["gqa_attention", "gated_short_conv", "gqa_attention", "gated_short_conv",
                     "gated_short_conv", "gqa_attention"]
    attn = spec.layers[0].mixer.params
    assert (attn["num_heads"], attn["num_kv_heads"], attn["head_dim"]) == (3, 1, 32)
    assert attn["position"].params["theta"] == 1e6 and attn["qk_norm_eps"] == 1e-6
    conv = spec.layers[1].mixer
    assert conv.params["taps"] == 4 and conv.params["bias"] and "bias" in conv.tensors
    assert spec.head_tensor == "lm_head.weight"
    assert [e.layer for e in spec.schedule] == list(range(6))
    assert Lfm2Config.from_dict(TINY_A).model_spec().head_tensor is None


def test_schedule_validation():
    from dataclasses import replace
    from flyweight_b200.config import ScheduleEntry
    spec = Lfm2Config.from_dict(TINY_A).model_spec()
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0))
            ).validate()                       # a layer may run twice
    with pytest.raises(ValueError, match="does not run before"):
        replace(spec, schedule=(ScheduleEntry(0, cache_of=1), ScheduleEntry(1))).validate()
    with pytest.raises(ValueError, match="names layer 7"):
        replace(spec, schedule=(ScheduleEntry(7),)).validate()


def test_a_checkpoint_with_another_feed_forward_width_is_believed_over_the_rule(tmp_path):
    """The width rule restates the config keys; a folder whose gate matrices have another number of
    rows (here: written without the rounding) loads with the stored width, as flyweight reads the
    width off the tensor (native/src/v2_runtime.cpp:3527-3535)."""
    import torch
    from flyweight_b200.config import Lfm2Config
    from flyweight_b200.weights.safetensors_io import stored_shapes
    from tiny_configs import TINY_A, make_model_dir
    raw = dict(TINY_A, intermediate_size=200, block_auto_adjust_ff_dim=True, block_multiple_of=32)
    config = Lfm2Config.from_dict(raw)
    assert config.ffn_dim == 160                                   # 200 * 2 / 3 = 133 -> 160
    folder = make_model_dir(tmp_path / "m", dict(TINY_A, intermediate_size=133), seed=1, dtype=torch.float32)
    shapes = stored_shapes(folder)
    assert shapes["model.layers.0.feed_forward.w1.weight"] == (133, 64)
    reconciled = config.reconciled_with(shapes)
    assert reconciled.ffn_dim == 133 and reconciled.model_spec().layers[0].feed_forward.params["ffn_dim"] == 133
    assert config.reconciled_with({}) is config
    assert "ffn_dim_from_checkpoint" not in reconciled.to_dict()
