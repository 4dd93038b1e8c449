"""Random weights for a model, from a configuration and a seed.

Every tensor is drawn from its own generator, keyed by (seed, tensor name), so any
tensor can be reproduced alone.  Two presets:

* ``"baseline"``: every matrix and table N(0, 0.02), norm weights 1 + N(0, 0.1),
  biases N(0, 0.02) -- the initialisation the benchmark configurations name.
* ``"unit"``: matrices N(0, 1/fan_in) so that activations keep unit scale through any
  depth, embeddings N(0, 1), conv taps N(0, 0.5), norm weights 1 + N(0, 0.1) -- close
  to flyweight's own test fixture (tests/lfm2_gguf_fixture.py:120-167); every part
  of the model then contributes visibly to the logits, which is what tests want.
"""
from __future__ import annotations

import json
import math
import zlib
from pathlib import Path
from typing import Dict, Mapping

import torch

from .loader import TensorDecl
from .safetensors_io import save_file

_MASK = (1 << 64) - 1


def _generator(seed: int, name: str, device) -> torch.Generator:
    # splitmix64 of (seed, name): every bit of the result depends on both, because some
    # generators use only the low 32 bits of the value they are seeded with
    value = ((int(seed) & _MASK) * 0x9E3779B97F4A7C15 + zlib.crc32(name.encode())) & _MASK
    value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK
    value ^= value >> 31
    gen = torch.Generator(device=device)
    gen.manual_seed(value & 0x7FFFFFFFFFFFFFFF)
    return gen


def random_tensor(name: str, decl: TensorDecl, seed: int, preset: str = "baseline",
                  dtype: torch.dtype = torch.bfloat16, device="cpu") -> torch.Tensor:
    gen = _generator(seed, name, device)
    shape = tuple(decl.shape)
    normal = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
    if decl.role == "norm":
        value = 1.0 + 0.1 * normal
    elif decl.role == "table":
        return torch.zeros(shape, dtype=torch.int32, device=device)
    elif preset == "baseline":
        value = 0.02 * normal
    elif preset == "unit":
        if decl.role == "embedding":
            value = normal
        elif decl.role == "taps":
            value = 0.5 * normal
        elif decl.role == "bias":
            value = 0.1 * normal
        else:
            fan_in = shape[-1] if len(shape) > 1 else 1
            value = normal / math.sqrt(fan_in)
    else:
        raise ValueError(f"unknown initialisation preset {preset!r}")
    return value.to(dtype)


def random_tensors(declared: Mapping[str, TensorDecl], seed: int, preset: str = "baseline",
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Dict[str, torch.Tensor]:
    return {name: random_tensor(name, decl, seed, preset, dtype, device)
            for name, decl in declared.items()}


def write_model_dir(out_dir, config_dict: Mapping, tensors: Mapping[str, torch.Tensor],
                    seed: int | None = None) -> Path:
    """A model folder: ``config.json`` and ``model.safetensors``."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "config.json").write_text(json.dumps(dict(config_dict), indent=2) + "\n")
    metadata = {"format": "pt"}
    if seed is not None:
        metadata["seed"] = str(seed)
    save_file(tensors, out_dir / "model.safetensors", metadata)
    return out_dir
