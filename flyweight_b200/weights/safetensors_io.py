"""Reading and writing safetensors files, without any library for the format.

Container (the same checks flyweight makes, native/include/flyweight_v2_safetensors.hpp:50-135):
an unsigned 64-bit little-endian header length, a JSON object mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (plus an optional ``__metadata__``), then
one flat payload.  Every range is checked against the file size and against shape x dtype.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Mapping, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U8": (torch.uint8, 1),
    "I8": (torch.int8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int            # absolute byte offsets in the file
    end: int


def read_header(path) -> Dict[str, TensorEntry]:
    path = Path(path)
    size = path.stat().st_size
    with open(path, "rb") as handle:
        prefix = handle.read(8)
        if len(prefix) != 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (header_len,) = struct.unpack("<Q", prefix)
        if header_len <= 0 or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(handle.read(header_len))
        except ValueError as error:
            raise SafetensorsError(f"{path}: header is not JSON: {error}") from None
    base = 8 + header_len
    entries: Dict[str, TensorEntry] = {}
    for name, raw in header.items():
        if name == "__metadata__":
            continue
        kind = raw.get("dtype")
        if kind not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {kind}")
        dtype, width = _DTYPES[kind]
        shape = tuple(int(d) for d in raw.get("shape", ()))
        begin, end = (int(v) for v in raw["data_offsets"])
        count = 1
        for dim in shape:
            count *= dim
        if begin < 0 or end < begin or base + end > size:
            raise SafetensorsError(f"{path}: tensor {name} lies outside the file")
        if end - begin != count * width:
            raise SafetensorsError(f"{path}: tensor {name} has {end - begin} bytes, "
                                   f"but shape {list(shape)} of {kind} needs {count * width}")
        entries[name] = TensorEntry(name, dtype, shape, base + begin, base + end)
    return entries


def load_file(path) -> Dict[str, torch.Tensor]:
    """All tensors of one file, in the dtype they were stored in (host memory)."""
    path = Path(path)
    entries = read_header(path)
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as handle:
        mapped = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_READ)
        try:
            view = memoryview(mapped)
            for name, entry in entries.items():
                count = 1
                for dim in entry.shape:
                    count *= dim
                if count == 0:
                    out[name] = torch.empty(entry.shape, dtype=entry.dtype)
                    continue
                flat = torch.frombuffer(bytearray(view[entry.begin:entry.end]), dtype=entry.dtype)
                out[name] = flat.reshape(entry.shape)
            view.release()
        finally:
            mapped.close()
    return out


def load_model_tensors(model_dir) -> Dict[str, torch.Tensor]:
    """``model.safetensors``, or the shards that ``model.safetensors.index.json`` lists
    (flyweight merges shards the same way, native/include/flyweight_v2_hf.hpp:1290-1306)."""
    model_dir = Path(model_dir)
    single = model_dir / "model.safetensors"
    index = model_dir / "model.safetensors.index.json"
    if single.is_file():
        return load_file(single)
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        out: Dict[str, torch.Tensor] = {}
        for shard in sorted(set(weight_map.values())):
            out.update(load_file(model_dir / shard))
        return out
    raise FileNotFoundError(f"{model_dir} holds neither model.safetensors nor "
                            "model.safetensors.index.json")


def stored_shapes(model_dir) -> Dict[str, tuple]:
    """Tensor name -> stored shape for a model folder, from the headers alone (no payload read)."""
    model_dir = Path(model_dir)
    single = model_dir / "model.safetensors"
    index = model_dir / "model.safetensors.index.json"
    if single.is_file():
        files = [single]
    elif index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        files = [model_dir / shard for shard in sorted(set(weight_map.values()))]
    else:
        return {}
    shapes: Dict[str, tuple] = {}
    for path in files:
        shapes.update({name: tuple(entry.shape) for name, entry in read_header(path).items()})
    return shapes


def save_file(tensors: Mapping[str, torch.Tensor], path, metadata: Mapping[str, str] | None = None):
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    ordered = sorted(tensors.items())
    for name, tensor in ordered:
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {tensor.dtype} ({name})")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((-len(blob)) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for _, tensor in ordered:
            data = tensor.detach().to("cpu").contiguous()
            handle.write(data.reshape(-1).view(torch.uint8).numpy().tobytes() if data.numel() else b"")
