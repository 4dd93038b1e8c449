"""From a model folder, or from a configuration and a seed, to a model on the device."""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from .. import models as _models  # noqa: F401  (registers the architectures)
from ..config.registry import architecture_name, load_config, lookup
from ..parts.base import Precision
from ..weights.loader import load_checkpoint
from ..weights.safetensors_io import stored_shapes
from ..weights.random_init import random_tensors


def parse_dtype(dtype) -> Precision:
    if isinstance(dtype, Precision):
        return dtype
    if isinstance(dtype, torch.dtype):
        dtype = {torch.float32: "float32", torch.bfloat16: "bfloat16"}.get(dtype, str(dtype))
    names = {"float32": "float32", "fp32": "float32", "f32": "float32",
             "bfloat16": "bfloat16", "bf16": "bfloat16"}
    try:
        return Precision(names[str(dtype).lower()])
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


class NoGpu(RuntimeError):
    """The engine was asked for a CUDA device where there is none: it has no other path."""


def require_gpu(device) -> None:
    """One clear error instead of whatever the first CUDA call would say.  (A model may still be
    put together on ``cpu`` -- the random-weights mode and the tests do -- but nothing runs there.)"""
    if torch.device(device).type == "cuda" and not torch.cuda.is_available():
        raise NoGpu("flyweight_b200 runs on an NVIDIA GPU (B200, sm_100a) only and found no CUDA device; "
                    "there is no CPU path")


def load_model(model_dir, dtype="bfloat16", device="cuda:0"):
    """The model that ``config.json`` names, with ``model.safetensors`` bound by name."""
    require_gpu(device)
    arch, config = load_config(model_dir)
    reconcile = getattr(config, "reconciled_with", None)
    if reconcile is not None:
        # sizes the config only states through a rule may be read off the stored tensors instead
        config = reconcile(stored_shapes(model_dir))
    model = arch.model_class(config, parse_dtype(dtype), torch.device(device))
    model.load(load_checkpoint(model_dir, model.declare()))
    return model


def random_model(config: Any, seed: int, dtype="bfloat16", device="cuda:0",
                 preset: str = "baseline", stored_dtype: Optional[torch.dtype] = None):
    """A model with seeded random weights, drawn on the device (no file is written).
    ``config`` is a typed configuration or a ``config.json`` mapping."""
    if isinstance(config, Mapping):
        arch = lookup(architecture_name(config))
        config = arch.config_class.from_dict(config)
    else:
        arch = lookup(config.architectures[0])
    precision = parse_dtype(dtype)
    require_gpu(device)
    device = torch.device(device)
    model = arch.model_class(config, precision, device)
    if stored_dtype is None:
        stored_dtype = torch.bfloat16
    model.load(random_tensors(model.declare(), seed, preset, stored_dtype, device))
    return model
