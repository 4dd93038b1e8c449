"""LFM2 (dense): registration of the architecture name with its configuration and model.

The model itself is the generic ``DecoderModel`` built from ``Lfm2Config.model_spec()``;
this class only fixes the pairing, so that ``config.json``'s ``architectures[0]`` picks
it (flyweight gates on the architecture string the same way, native/src/v2_runtime.cpp:19903-19915,
and builds the per-layer plan in build_lfm2_plan, native/src/v2_runtime.cpp:4185-4282).
"""
from __future__ import annotations

from ..config.lfm2 import Lfm2Config
from ..config.registry import register_architecture
from ..parts.base import Precision
from ..parts.model import DecoderModel


class Lfm2ForCausalLM(DecoderModel):
    config_class = Lfm2Config

    def __init__(self, config: Lfm2Config, precision: Precision, device):
        self.config = config
        super().__init__(config.model_spec(), precision, device)


register_architecture("Lfm2ForCausalLM", Lfm2Config, Lfm2ForCausalLM)
