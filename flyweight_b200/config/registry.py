"""One registry from an architecture's name to its configuration class and model class.

The name is ``config.json``'s ``architectures[0]`` (flyweight dispatches the same way on
the HF side, native/include/flyweight_v2_hf.hpp:562-586, and refuses unknown names with
a message that says so, native/src/v2_runtime.cpp:19903-19915).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, Mapping


class UnknownArchitecture(ValueError):
    pass


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any            # has from_dict(mapping) and model_spec()
    model_class: Any             # built as model_class(config, ...) by the engine


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, model_class: Any) -> None:
    _REGISTRY[name] = Architecture(name, config_class, model_class)


def architectures() -> tuple:
    return tuple(sorted(_REGISTRY))


def lookup(name: str) -> Architecture:
    try:
        return _REGISTRY[name]
    except KeyError:
        raise UnknownArchitecture(
            f"unsupported architecture {name!r}; this engine runs: "
            + (", ".join(architectures()) or "(none registered)")) from None


def architecture_name(raw: Mapping[str, Any]) -> str:
    names = raw.get("architectures")
    if names:
        return str(names[0])
    raise UnknownArchitecture("config.json has no 'architectures' entry; this engine runs: "
                              + ", ".join(architectures()))


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} not found: a model folder holds config.json and "
                                "model.safetensors")
    return json.loads(path.read_text())


def load_config(model_dir):
    """(Architecture, typed config) for a model folder."""
    raw = read_config_json(model_dir)
    arch = lookup(architecture_name(raw))
    return arch, arch.config_class.from_dict(raw)
