"""Binding checkpoint tensors to the tensors a model declares, by name.

The model (through its parts) declares every tensor it needs with its shape; the
loader compares that list with what the checkpoint holds and reports ALL problems in
one error: missing tensors, unexpected tensors, wrong shapes.  (flyweight stops at
the first: "required Qwen tensor is missing", native/src/v2_runtime.cpp:3356;
"unmapped HF tensor", native/include/flyweight_v2_hf.hpp:1455-1456.)

Tensors keep the dtype they were stored in: bfloat16 stays bfloat16, a tensor stored
in 32-bit stays 32-bit, integer tables become int32.  Nothing is widened here; the
float32 mode of the engine widens (exactly) when it binds.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Tuple

import torch

from .safetensors_io import load_model_tensors


class WeightError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and
    ``wrong_shape`` list the tensor names."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): "
                         + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{name}: stored {list(got)}, model needs {list(want)}"
                for name, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unusable dtypes ({len(self.wrong_dtype)}): " + "; ".join(
                f"{name}: {dtype}" for name, dtype in self.wrong_dtype))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part needs.  ``role`` picks the random initialisation
    (matrix / embedding / norm / taps / bias / table); ``also`` lists other stored
    shapes with the same bytes that are accepted and reshaped (a Conv1d weight
    stored as [H][1][L] for a declared [H][L])."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    also: Tuple[Tuple[int, ...], ...] = ()


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int32, torch.int64, torch.int8, torch.uint8)


def bind(declared: Mapping[str, TensorDecl],
         stored: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    missing = [name for name in declared if name not in stored]
    unexpected = [name for name in stored if name not in declared]
    wrong_shape, wrong_dtype = [], []
    out: Dict[str, torch.Tensor] = {}
    for name, decl in declared.items():
        if name not in stored:
            continue
        tensor = stored[name]
        shape = tuple(tensor.shape)
        if shape != tuple(decl.shape):
            if shape in decl.also:
                tensor = tensor.reshape(decl.shape)
            else:
                wrong_shape.append((name, shape, tuple(decl.shape)))
                continue
        if decl.role == "table":
            if tensor.dtype not in _INTS:
                wrong_dtype.append((name, str(tensor.dtype)))
                continue
            tensor = tensor.to(torch.int32)
        elif tensor.dtype == torch.float16 or tensor.dtype == torch.float64:
            # neither is a dtype the kernels read; widen/narrow to 32-bit once
            tensor = tensor.to(torch.float32)
        elif tensor.dtype not in _FLOATS:
            wrong_dtype.append((name, str(tensor.dtype)))
            continue
        out[name] = tensor
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype)
    return out


def load_checkpoint(model_dir, declared: Mapping[str, TensorDecl]) -> Dict[str, torch.Tensor]:
    return bind(declared, load_model_tensors(model_dir))
