"""Architecture-neutral description of a decoder model.

An architecture's typed configuration (for instance ``Lfm2Config``) turns itself
into a ``ModelSpec``: a list of layers, each put together from named parts with
their sizes and constants as parameters, and a schedule that says in which order
the layers run.  Everything below the configuration (parts, cache manager, step
function) reads only this description, never the architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the registry key of its implementation, and its parameters.

    ``params`` carries every size and constant the part needs (head counts, eps,
    theta, tap count, ...) and ``tensors`` maps the part's own role names (for an
    attention mixer: ``q``, ``k``, ``v``, ``o``, ...) to full tensor names in the
    checkpoint.
    """
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    tensors: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True, init=False)
class LayerSpec:
    """One layer: an arrangement (how its parts are wired around the residual stream) and the
    parts it wires, by role.  Which roles there are is the arrangement's business: the pre-norm
    residual block has ``mixer_norm``, ``mixer``, ``ffn_norm`` and ``feed_forward``; another
    arrangement may ask for more (post-norms), fewer (no feed-forward) or others.

        LayerSpec("prenorm_residual", mixer_norm, mixer, ffn_norm, feed_forward)     # the four, in order
        LayerSpec("my_arrangement", parts={"norm": ..., "feed_forward": ...})        # any roles
    """
    arrangement: str
    parts: Mapping[str, PartSpec]

    def __init__(self, arrangement: str, mixer_norm: Optional[PartSpec] = None,
                 mixer: Optional[PartSpec] = None, ffn_norm: Optional[PartSpec] = None,
                 feed_forward: Optional[PartSpec] = None, *,
                 parts: Optional[Mapping[str, PartSpec]] = None):
        named = dict(parts or {})
        for role, spec in (("mixer_norm", mixer_norm), ("mixer", mixer), ("ffn_norm", ffn_norm),
                           ("feed_forward", feed_forward)):
            if spec is not None:
                if role in named:
                    raise ValueError(f"layer part {role!r} is given twice")
                named[role] = spec
        object.__setattr__(self, "arrangement", arrangement)
        object.__setattr__(self, "parts", named)

    def __getattr__(self, role: str) -> PartSpec:
        parts = self.__dict__.get("parts", {})
        if role in parts:
            return parts[role]
        raise AttributeError(f"this layer ({self.__dict__.get('arrangement')!r}) has no part {role!r}")


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers``; a layer may appear in several entries
    (its weights are then shared, each execution keeping a cache of its own).
    ``cache_of`` names an earlier schedule position whose cache this execution
    reads instead of keeping one.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_tensor: str
    final_norm: PartSpec
    head_tensor: Optional[str]          # None: the head is the embedding table (tied)
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    embedding_scale: float = 1.0        # embedding rows are multiplied by this (LFM2: 1)
    logit_softcap: float = 0.0          # > 0: logits = cap * tanh(logits / cap) (LFM2: off)

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if self.logit_softcap < 0 or not self.embedding_scale == self.embedding_scale:
            raise ValueError("logit_softcap must not be negative")
        for position, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule position {position} names layer {entry.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < position:
                    raise ValueError(f"schedule position {position} reads the cache of position "
                                     f"{entry.cache_of}, which does not run before it")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(f"schedule position {position} reads a cache through position "
                                     f"{entry.cache_of}, which has none of its own")
