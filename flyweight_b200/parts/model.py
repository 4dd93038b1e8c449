"""A decoder model put together from a ``ModelSpec``: embedding, the layers in the
order its schedule names them, a final norm and the head.

LFM2 takes embedding rows without scaling (native/src/v2_runtime.cpp:27951-27956) and has
no soft-cap on its logits; ``ModelSpec.embedding_scale`` and ``logit_softcap`` are there for
architectures that have them.  The
head is the embedding table when the spec names none (native/src/v2_runtime.cpp:4190-4191);
the final norm and the head run only on the rows whose logits were asked for.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Mapping, Optional

import torch

from ..config.spec import ModelSpec
from ..kernels import ops
from ..weights.loader import TensorDecl, bind as bind_tensors
from .base import Arrangement, Precision, build_arrangement, build_norm


class DecoderModel:
    def __init__(self, spec: ModelSpec, precision: Precision, device):
        spec.validate()
        self.spec = spec
        self.precision = precision
        self.device = device
        self.layers: List[Arrangement] = [build_arrangement(layer) for layer in spec.layers]
        self.final_norm = build_norm(spec.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        for position, entry in enumerate(spec.schedule):
            layer = self.layers[entry.layer]
            if entry.cache_of is not None and layer.state_spec() is not None:
                raise ValueError(
                    f"schedule position {position} reads the cache of position {entry.cache_of}, "
                    f"but its mixer ({layer.stateful_part().kind}) keeps a cache of its own")

    # ------------------------------------------------------------------ weights
    def declare(self) -> Dict[str, TensorDecl]:
        spec = self.spec
        out = {spec.embedding_tensor: TensorDecl((spec.vocab_size, spec.hidden_size), "embedding")}
        if spec.head_tensor is not None:
            out[spec.head_tensor] = TensorDecl((spec.vocab_size, spec.hidden_size))
        out.update(self.final_norm.declare())
        for layer in self.layers:
            for part in layer.parts():
                out.update(part.declare())
        return out

    def load(self, stored: Mapping[str, torch.Tensor]) -> None:
        """Bind checkpoint tensors by name; one error lists everything that does not fit."""
        tensors = bind_tensors(self.declare(), stored)
        get: Callable[[str], torch.Tensor] = tensors.__getitem__
        spec, precision, device = self.spec, self.precision, self.device
        self.embedding = precision.matrix(get(spec.embedding_tensor), device)
        self.head = (self.embedding if spec.head_tensor is None
                     else precision.matrix(get(spec.head_tensor), device))
        self.final_norm.bind(get, precision, device)
        for layer in self.layers:
            for part in layer.parts():
                part.bind(get, precision, device)

    @property
    def graph_safe(self) -> bool:
        """Every part only launches kernels over the step's device buffers."""
        return all(part.graph_safe for layer in self.layers for part in layer.parts()) \
            and self.final_norm.graph_safe

    def prepare(self, max_positions: int) -> None:
        for layer in self.layers:
            layer.prepare(max_positions, self.device)

    def state_specs(self) -> list:
        """What each schedule position keeps in the cache manager."""
        return [None if entry.cache_of is not None else self.layers[entry.layer].state_spec()
                for entry in self.spec.schedule]

    def weight_bytes(self, with_embedding_rows: int = 0) -> int:
        """Bytes of weights one step reads: every scheduled layer once, the final norm, the
        head, and ``with_embedding_rows`` rows of the embedding table."""
        total = self.final_norm.weight_bytes()
        total += self.head.numel() * self.head.element_size()
        total += with_embedding_rows * self.spec.hidden_size * self.embedding.element_size()
        for entry in self.spec.schedule:
            total += sum(part.weight_bytes() for part in self.layers[entry.layer].parts())
        return total

    def flops_per_token(self, with_head: bool = False) -> float:
        """Operations of the matrix products one token passes through (every scheduled layer
        once; the head only if asked: it runs on the wanted rows alone)."""
        total = sum(part.flops_per_token() for entry in self.spec.schedule
                    for part in self.layers[entry.layer].parts())
        if with_head:
            total += 2.0 * self.spec.vocab_size * self.spec.hidden_size
        return total

    def context_flops(self, n_tokens: int) -> float:
        """Operations that grow with the context, for one causal prompt of ``n_tokens``."""
        return sum(part.context_flops(n_tokens) for entry in self.spec.schedule
                   for part in self.layers[entry.layer].parts())

    def parameter_count(self) -> int:
        return sum(int(torch.tensor(decl.shape).prod()) for decl in self.declare().values())

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, caches) -> torch.Tensor:
        """Logits [R][V] fp32 at ``ctx.batch.logit_rows`` (an empty tensor if R == 0).
        ``caches[i]`` is the ``LayerCache`` of schedule position i."""
        batch = ctx.batch
        x = ops.embed(self.embedding, batch.token_ids, ctx.bad_token_flag, self.spec.embedding_scale)
        pending = None
        for position, entry in enumerate(self.spec.schedule):
            source = position if entry.cache_of is None else entry.cache_of
            x, pending = self.layers[entry.layer].forward(ctx, x, pending, caches[source])
        if batch.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        n = self.final_norm.defer(ctx, x, rows=batch.logit_rows) if pending is None else None
        if n is None:
            n = self.final_norm.forward(ctx, x, delta=pending, rows=batch.logit_rows)
        logits = ops.linear(n, self.head, torch.float32)
        if self.spec.logit_softcap > 0:
            ops.softcap_(logits, self.spec.logit_softcap)
        return logits
