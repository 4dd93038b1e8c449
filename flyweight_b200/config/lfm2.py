"""Typed configuration of dense LFM2 (gated short convolution + GQA hybrid).

Keys are the ones an LFM2 ``config.json`` carries.  Defaults are the ones
yairpatch/flyweight applies when a key is absent: norm eps 1e-6
(native/src/v2_runtime.cpp:27558), rope base 1e6 (native/src/v2_runtime.cpp:4235),
head size = hidden / heads (native/src/v2_runtime.cpp:4222).  Validation mirrors
``build_lfm2_plan`` (native/src/v2_runtime.cpp:4185-4282) and the post-parse checks
(native/src/v2_runtime.cpp:3195-3209).
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Any, Mapping, Optional, Tuple

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


class ConfigError(ValueError):
    """A configuration that cannot describe a model."""


_ATTENTION_NAMES = ("full_attention", "attention", "attn")
_CONV_NAMES = ("conv", "short_conv", "shortconv")


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    layer_types: Tuple[str, ...]                 # "conv" | "full_attention", one per layer
    block_multiple_of: int = 256
    block_ffn_dim_multiplier: Optional[float] = None
    block_auto_adjust_ff_dim: bool = False
    conv_L_cache: int = 3
    conv_bias: bool = False
    rope_theta: float = 1_000_000.0
    norm_eps: float = 1e-6
    max_position_embeddings: int = 128_000
    tie_embedding: bool = True
    architectures: Tuple[str, ...] = ("Lfm2ForCausalLM",)
    model_type: str = "lfm2"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)
    # the feed-forward width read off the checkpoint's gate matrix when it differs from the rule
    # below (flyweight never applies a rule: native/src/v2_runtime.cpp:3527-3535)
    ffn_dim_from_checkpoint: Optional[int] = None

    # ------------------------------------------------------------------ derived sizes
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def ffn_dim(self) -> int:
        """SwiGLU width.  flyweight reads it off the gate tensor
        (native/src/v2_runtime.cpp:3527-3535); a config.json states it through
        ``intermediate_size`` and the three ``block_*`` keys: with auto-adjust the
        width is 2/3 of it, times the optional multiplier, rounded up to a multiple
        of ``block_multiple_of``."""
        if self.ffn_dim_from_checkpoint is not None:
            return self.ffn_dim_from_checkpoint
        width = self.intermediate_size
        if self.block_auto_adjust_ff_dim:
            width = int(2 * width / 3)
            if self.block_ffn_dim_multiplier is not None:
                width = int(self.block_ffn_dim_multiplier * width)
            width = self.block_multiple_of * ((width + self.block_multiple_of - 1)
                                              // self.block_multiple_of)
        return width

    @property
    def attention_layers(self) -> Tuple[int, ...]:
        return tuple(i for i, kind in enumerate(self.layer_types) if kind == "full_attention")

    # ------------------------------------------------------------------ reading / writing
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Lfm2Config":
        known = {
            "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "intermediate_size", "layer_types", "full_attn_idxs",
            "block_multiple_of", "block_ffn_dim_multiplier", "block_auto_adjust_ff_dim",
            "conv_L_cache", "conv_bias", "rope_theta", "norm_eps", "max_position_embeddings",
            "tie_embedding", "tie_word_embeddings", "architectures", "model_type",
        }
        required = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "intermediate_size")
        missing = [key for key in required if raw.get(key) is None]
        if missing:
            raise ConfigError("LFM2 config.json is missing: " + ", ".join(missing))
        layers = int(raw["num_hidden_layers"])
        if raw.get("layer_types") is not None:
            kinds = []
            for name in raw["layer_types"]:
                if name in _ATTENTION_NAMES:
                    kinds.append("full_attention")
                elif name in _CONV_NAMES:
                    kinds.append("conv")
                else:
                    raise ConfigError(f"unknown LFM2 layer type {name!r} "
                                      "(known: conv, full_attention)")
        elif raw.get("full_attn_idxs") is not None:
            full = {int(i) for i in raw["full_attn_idxs"]}
            bad = sorted(i for i in full if not 0 <= i < layers)
            if bad:
                raise ConfigError(f"full_attn_idxs {bad} outside 0..{layers - 1}")
            kinds = ["full_attention" if i in full else "conv" for i in range(layers)]
        else:
            raise ConfigError("LFM2 config.json needs layer_types or full_attn_idxs")
        tie = raw.get("tie_embedding", raw.get("tie_word_embeddings", True))
        eps = raw.get("norm_eps")
        theta = raw.get("rope_theta")
        mult = raw.get("block_ffn_dim_multiplier")
        config = cls(
            vocab_size=int(raw["vocab_size"]),
            hidden_size=int(raw["hidden_size"]),
            num_hidden_layers=layers,
            num_attention_heads=int(raw["num_attention_heads"]),
            num_key_value_heads=int(raw["num_key_value_heads"]),
            intermediate_size=int(raw["intermediate_size"]),
            layer_types=tuple(kinds),
            block_multiple_of=int(raw.get("block_multiple_of", 256)),
            block_ffn_dim_multiplier=None if mult is None else float(mult),
            block_auto_adjust_ff_dim=bool(raw.get("block_auto_adjust_ff_dim", False)),
            conv_L_cache=int(raw.get("conv_L_cache", 3)),
            conv_bias=bool(raw.get("conv_bias", False)),
            rope_theta=float(theta) if theta else 1_000_000.0,
            norm_eps=float(eps) if eps else 1e-6,
            max_position_embeddings=int(raw.get("max_position_embeddings", 128_000)),
            tie_embedding=bool(tie),
            architectures=tuple(raw.get("architectures") or ("Lfm2ForCausalLM",)),
            model_type=str(raw.get("model_type", "lfm2")),
            extra={k: v for k, v in raw.items() if k not in known},
        )
        config.validate()
        return config

    def reconciled_with(self, stored_shapes: Mapping[str, Tuple[int, ...]]) -> "Lfm2Config":
        """This configuration, with the feed-forward width taken from the checkpoint where the two
        disagree.  The width rule (2/3, multiplier, rounding) is restated from the config keys; a
        checkpoint whose gate matrix has another number of rows (a config written with other
        rounding habits) is believed over the rule, as flyweight believes the tensor
        (native/src/v2_runtime.cpp:3527-3535).  Every layer must agree on the width."""
        widths = {shape[0] for name, shape in stored_shapes.items()
                  if name.startswith("model.layers.") and name.endswith(".feed_forward.w1.weight")
                  and len(shape) == 2 and shape[1] == self.hidden_size}
        if len(widths) != 1:
            return self
        (width,) = widths
        if width == self.ffn_dim:
            return self
        from dataclasses import replace
        return replace(self, ffn_dim_from_checkpoint=int(width))

    def to_dict(self) -> dict:
        out = asdict(self)
        out.pop("extra")
        out.pop("ffn_dim_from_checkpoint")
        out["layer_types"] = list(self.layer_types)
        out["full_attn_idxs"] = list(self.attention_layers)
        out["architectures"] = list(self.architectures)
        out["tie_word_embeddings"] = self.tie_embedding
        out.update(self.extra)
        return out

    def validate(self) -> None:
        def need(ok: bool, message: str) -> None:
            if not ok:
                raise ConfigError(message)
        need(self.vocab_size > 0 and self.hidden_size > 0 and self.num_hidden_layers > 0,
             "vocab_size, hidden_size and num_hidden_layers must be positive")
        need(self.num_attention_heads > 0 and self.num_key_value_heads > 0,
             "LFM2 attention geometry is incomplete")              # v2_runtime.cpp:4220-4221
        need(self.hidden_size % self.num_attention_heads == 0,
             f"hidden_size {self.hidden_size} is not a multiple of num_attention_heads "
             f"{self.num_attention_heads}")
        need(self.num_attention_heads % self.num_key_value_heads == 0,
             f"num_attention_heads {self.num_attention_heads} is not a multiple of "
             f"num_key_value_heads {self.num_key_value_heads}")
        need(self.head_dim % 2 == 0, f"head size {self.head_dim} must be even for rotary pairs")
        need(len(self.layer_types) == self.num_hidden_layers,
             f"layer_types has {len(self.layer_types)} entries for "
             f"{self.num_hidden_layers} layers")
        need(self.conv_L_cache >= 2,                                 # v2_runtime.cpp:3205-3207
             f"conv_L_cache must be at least 2, got {self.conv_L_cache}")
        need(self.intermediate_size > 0 and self.block_multiple_of > 0,
             "intermediate_size and block_multiple_of must be positive")
        need(self.norm_eps > 0 and self.rope_theta > 0, "norm_eps and rope_theta must be positive")
        need(self.max_position_embeddings > 0, "max_position_embeddings must be positive")

    # ------------------------------------------------------------------ the model it describes
    def model_spec(self) -> ModelSpec:
        """Layers from parts.  Tensor names are the checkpoint's own
        (``model.layers.{i}.conv.in_proj.weight`` and so on)."""
        def norm(tensor: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.norm_eps},
                            {"weight": tensor})

        layers = []
        for index, kind in enumerate(self.layer_types):
            prefix = f"model.layers.{index}."
            if kind == "full_attention":
                mixer = PartSpec(
                    "gqa_attention",
                    {
                        "hidden_size": self.hidden_size,
                        "num_heads": self.num_attention_heads,
                        "num_kv_heads": self.num_key_value_heads,
                        "head_dim": self.head_dim,
                        "qk_norm_eps": self.norm_eps,          # same eps as the block norms
                        "position": PartSpec("rope_half_split",
                                             {"theta": self.rope_theta,
                                              "rotary_dim": self.head_dim}),
                        "window": 0,
                    },
                    {
                        "q": prefix + "self_attn.q_proj.weight",
                        "k": prefix + "self_attn.k_proj.weight",
                        "v": prefix + "self_attn.v_proj.weight",
                        "o": prefix + "self_attn.out_proj.weight",
                        "q_norm": prefix + "self_attn.q_layernorm.weight",
                        "k_norm": prefix + "self_attn.k_layernorm.weight",
                    })
            else:
                tensors = {
                    "in_proj": prefix + "conv.in_proj.weight",
                    "taps": prefix + "conv.conv.weight",
                    "out_proj": prefix + "conv.out_proj.weight",
                }
                if self.conv_bias:
                    tensors["bias"] = prefix + "conv.conv.bias"
                mixer = PartSpec(
                    "gated_short_conv",
                    {"hidden_size": self.hidden_size, "taps": self.conv_L_cache,
                     "bias": self.conv_bias},
                    tensors)
            ffn = PartSpec(
                "swiglu",
                {"hidden_size": self.hidden_size, "ffn_dim": self.ffn_dim},
                {"gate": prefix + "feed_forward.w1.weight",
                 "up": prefix + "feed_forward.w3.weight",
                 "down": prefix + "feed_forward.w2.weight"})
            layers.append(LayerSpec(
                arrangement="prenorm_residual",
                mixer_norm=norm(prefix + "operator_norm.weight"),
                mixer=mixer,
                ffn_norm=norm(prefix + "ffn_norm.weight"),
                feed_forward=ffn))
        spec = ModelSpec(
            architecture=self.architectures[0],
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding_tensor="model.embed_tokens.weight",
            final_norm=norm("model.embedding_norm.weight"),
            head_tensor=None if self.tie_embedding else "lm_head.weight",
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        )
        spec.validate()
        return spec
