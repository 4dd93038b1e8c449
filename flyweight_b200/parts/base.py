"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from a ``PartSpec`` alone: its sizes and constants are parameters,
its tensors are named by the spec, and it never learns which model it is in.  There
is one registry per kind of part; an architecture (or a test) adds an implementation
with the matching ``register_*`` decorator and names it in its ``PartSpec.kind``.

Interfaces
----------
``Norm.forward(ctx, x, delta=None, rows=None)``
    x: fp32 residual [T][H].  Adds ``delta`` into x first when given (the residual
    sum, fp32), returns the normalised rows in ``ctx.precision.act_dtype``.
``Norm.defer(ctx, x, rows=None)`` -> ``DeferredNorm`` | ``None``  (optional)
    the same rows as a recipe instead of a tensor, for a consumer with ``takes_deferred_norm``:
    its first matrix product may then apply the norm itself (``ops.linear`` takes either).
``Mixer.state_spec()`` -> ``PagedKV`` | ``FixedState`` | ``None``
    what the cache manager must keep for one execution of this mixer.
``Mixer.forward(ctx, h, cache)`` -> fp32 [T][H]
    h: normalised input; cache: the ``LayerCache`` the manager made for this
    execution (or for the execution it shares with).  Returns the residual delta.
``FeedForward.forward(ctx, h)`` -> fp32 [T][H]
    A mixer or feed-forward with ``adds_residual`` is called with ``residual=x`` as well and
    may add its delta into x itself (its last product's epilogue); it then returns None.
``PositionEncoding.encode(ctx, qkv, ...)`` -> q; keys and values are in the cache afterwards.
    The default is the fused norm + rotation + page-write kernel fed by ``table(n_positions,
    device)``, ``rotary_dim`` and ``pairing``.
``Arrangement.forward(ctx, x, pending, cache)`` -> (x, pending)
    wires norms, mixer and feed-forward around the residual stream; ``pending`` is
    a delta not yet added to x, handed to the next norm so that the sum and the
    norm are one kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from ..config.spec import LayerSpec, PartSpec
from ..weights.loader import TensorDecl


# ------------------------------------------------------------------ precision
@dataclass(frozen=True)
class Precision:
    """``float32``: everything in true 32-bit.  ``bfloat16``: the serving precision --
    bfloat16 matrices, activations and cache, with the residual stream, norms,
    softmax, rotation and conv state in fp32."""
    name: str

    def __post_init__(self):
        if self.name not in ("float32", "bfloat16"):
            raise ValueError(f"dtype must be float32 or bfloat16, got {self.name!r}")

    @property
    def act_dtype(self) -> torch.dtype:
        return torch.float32 if self.name == "float32" else torch.bfloat16

    @property
    def cache_dtype(self) -> torch.dtype:
        return self.act_dtype

    def matrix(self, tensor: torch.Tensor, device) -> torch.Tensor:
        """A weight matrix on the device.  float32 mode widens (exactly); bfloat16 mode
        keeps the stored dtype (a matrix stored in 32-bit stays so and runs the 32-bit
        product)."""
        tensor = tensor.to(device)
        if self.name == "float32" and tensor.dtype != torch.float32:
            tensor = tensor.to(torch.float32)
        return tensor.contiguous()

    @staticmethod
    def vector(tensor: torch.Tensor, device) -> torch.Tensor:
        """Norm weights, conv taps, biases: kernels read them as fp32 (exact widening)."""
        return tensor.to(device=device, dtype=torch.float32).contiguous()


# ------------------------------------------------------------------ cache needs
@dataclass(frozen=True)
class PagedKV:
    """Keys and values that grow with the sequence.  ``window`` > 0: only the last
    ``window`` positions are ever read again, older pages may be given back."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size, zero when a request starts.  ``dtype``: fp32 unless the
    part says otherwise (a recurrent state kept in bfloat16, a counter in int32)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------------ a norm not yet applied
@dataclass
class DeferredNorm:
    """Rows of the fp32 residual together with the norm that is still to be applied to them.
    ``materialize`` runs the norm's kernel; ``ops.linear`` and the fused feed-forward product
    fold an RMS norm into their own kernel instead when the shape allows it."""
    x: torch.Tensor                      # fp32 residual [T][H]
    weight: torch.Tensor                 # fp32 [H]
    eps: float
    rows: Optional[torch.Tensor] = None  # int32 row indices (None: every row)
    kind: str = "rmsnorm"

    @property
    def n_rows(self) -> int:
        return self.rows.numel() if self.rows is not None else self.x.numel() // self.x.shape[-1]

    def materialize(self, dtype: torch.dtype) -> torch.Tensor:
        from ..kernels import ops
        return ops.rmsnorm(self.x, self.weight, self.eps, dtype, rows=self.rows)


# ------------------------------------------------------------------ part interfaces
class Part:
    kind: str = ""
    # True when forward() only launches kernels whose arguments are device buffers of the
    # step's batch (nothing read on the host), so a decode step may be captured in a CUDA
    # graph and replayed with new batch contents.  Parts defined elsewhere default to False.
    graph_safe: bool = False
    # True when forward() accepts a ``DeferredNorm`` in place of the normalised input.
    takes_deferred_norm: bool = False
    # True when forward() takes ``residual=`` and may add its delta into it (returning None).
    adds_residual: bool = False

    def __init__(self, spec: PartSpec):
        self.spec = spec
        self.params = dict(spec.params)
        self.names = dict(spec.tensors)

    def declare(self) -> Dict[str, TensorDecl]:
        """Full tensor name -> declaration, for every tensor this part binds."""
        return {}

    def bind(self, get: Callable[[str], torch.Tensor], precision: Precision, device) -> None:
        """Fetch the declared tensors (``get(full_name)`` returns the stored tensor)."""

    def weight_bytes(self) -> int:
        """Bytes of device weights a step reads (for roofline accounting)."""
        return 0

    def flops_per_token(self) -> float:
        """Floating-point operations of this part's matrix products for one token (2 per weight)."""
        return 0.0

    def context_flops(self, n_tokens: int) -> float:
        """Operations that grow with the context, for one causal prompt of ``n_tokens``
        (attention: scores and weighted values over the visible keys); 0 for most parts."""
        return 0.0


class Norm(Part):
    def forward(self, ctx, x, delta=None, rows=None):
        raise NotImplementedError

    def defer(self, ctx, x, rows=None):
        """The norm of ``x`` (no pending delta) as a ``DeferredNorm``, or None if this norm
        has no such form."""
        return None


class PositionEncoding(Part):
    """How positions enter an attention mixer.  The mixer hands its fused q|k|v rows to
    ``encode`` and gets the queries back; keys and values are in the cache afterwards.  The
    default ``encode`` is the fused kernel (per-head q/k norm, rotation from ``table``, page
    write) with this part's ``rotary_dim`` and ``pairing``, so a rotary encoding only has to
    supply its table; an encoding that is no rotation overrides ``encode``."""
    rotary_dim: int = 0                 # channels of a head that turn (0: none)
    pairing: str = "half_split"         # "half_split" (i, i + rotary_dim/2) | "interleaved" (2i, 2i+1)

    def table(self, n_positions: int, device):
        """[n_positions][rotary_dim/2][2] fp32 (cos, sin); pair i of a head turns by entry i."""
        raise NotImplementedError

    def prepare(self, max_positions: int, device) -> None:
        self._table = (self.table(max_positions, device) if self.rotary_dim > 0
                       else torch.zeros((1, 1, 2), dtype=torch.float32, device=device))

    def encode(self, ctx, qkv, *, n_heads: int, n_kv_in: int, head_dim: int, q_norm, k_norm,
               eps: float, cache, block_table):
        """qkv: [T][(n_heads + 2 n_kv_in) head_dim] in the activation dtype (``n_kv_in`` 0: queries
        only, for a mixer that reads another execution's cache).  Returns q [T][n_heads head_dim]."""
        from ..kernels import ops
        batch = ctx.batch
        return ops.qk_norm_rope(
            qkv, q_norm, k_norm, self._table, batch.positions, batch.tok_seg,
            block_table if n_kv_in else None, cache.k_pool if n_kv_in else None,
            cache.v_pool if n_kv_in else None, n_heads, n_kv_in, head_dim, self.rotary_dim,
            float(eps or 0.0), ctx.precision.act_dtype, pairing=self.pairing)

    def rotation(self):
        """(table, rotary_dim, pairing) for a mixer that can do the default ``encode`` inside a kernel
        of its own (the decode attention does, for steps of single tokens); None from an encoding that
        encodes in its own way, which is then always asked to ``encode``."""
        if type(self).encode is not PositionEncoding.encode:
            return None
        return self._table, self.rotary_dim, self.pairing

    def plan(self, builder, qkv, q_out, *, n_heads: int, n_kv_in: int, head_dim: int, q_norm, k_norm,
             eps, cache) -> None:
        """``encode`` for the native step plan.  Only an encoding that keeps the default ``encode``
        has this form; one that overrides ``encode`` leaves its model on the Python path unless it
        overrides ``plan`` as well."""
        from ..engine.plan import NotPlannable
        if type(self).encode is not PositionEncoding.encode:
            raise NotPlannable(f"position encoding {self.kind!r} encodes in its own way")
        builder.qk_rope(qkv, q_norm, k_norm, self._table, q_out, cache, n_heads, n_kv_in, head_dim,
                        self.rotary_dim, self.pairing, eps)


class Mixer(Part):
    def state_spec(self):
        return None

    def prepare(self, max_positions: int, device) -> None:
        """Build position tables and the like once the engine's limits are known."""

    def forward(self, ctx, h, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h):
        raise NotImplementedError


class Arrangement:
    """How a layer's parts are wired around the residual stream.  ``ROLES`` maps each role name
    the arrangement knows to the family its part is built from (``norm``, ``mixer``,
    ``feed_forward``) and says whether the layer must have it; the built parts become attributes
    named after their roles (absent optional ones are None)."""
    ROLES: Dict[str, Tuple[str, bool]] = {          # role -> (family, required)
        "mixer_norm": ("norm", True), "mixer": ("mixer", True),
        "ffn_norm": ("norm", True), "feed_forward": ("feed_forward", True)}

    def __init__(self, layer: LayerSpec):
        self.layer = layer
        unknown = sorted(set(layer.parts) - set(self.ROLES))
        missing = sorted(role for role, (_, required) in self.ROLES.items()
                         if required and role not in layer.parts)
        if unknown or missing:
            raise ValueError(f"arrangement {layer.arrangement!r}: "
                             + (f"unknown parts {unknown}; " if unknown else "")
                             + (f"missing parts {missing}; " if missing else "")
                             + "it wires " + ", ".join(self.ROLES))
        builders = {"norm": build_norm, "mixer": build_mixer, "feed_forward": build_feed_forward}
        self._built = []
        for role, (family, _) in self.ROLES.items():
            part = builders[family](layer.parts[role]) if role in layer.parts else None
            setattr(self, role, part)
            if part is not None:
                self._built.append(part)

    def parts(self):
        return tuple(self._built)

    def stateful_part(self):
        """The part whose ``state_spec()`` says what one execution of this layer keeps in the
        cache manager (None: nothing)."""
        return getattr(self, "mixer", None)

    def state_spec(self):
        part = self.stateful_part()
        return part.state_spec() if part is not None else None

    def prepare(self, max_positions: int, device) -> None:
        for part in self._built:
            prepare = getattr(part, "prepare", None)
            if prepare is not None:
                prepare(max_positions, device)

    def forward(self, ctx, x, pending, cache):
        raise NotImplementedError


# ------------------------------------------------------------------ registries
_NORMS: Dict[str, type] = {}
_MIXERS: Dict[str, type] = {}
_FEED_FORWARDS: Dict[str, type] = {}
_POSITIONS: Dict[str, type] = {}
_ARRANGEMENTS: Dict[str, type] = {}


def _register(table: Dict[str, type], what: str):
    def decorator_for(kind: str):
        def decorator(cls):
            cls.kind = kind
            table[kind] = cls
            return cls
        return decorator
    return decorator_for


register_norm = _register(_NORMS, "norm")
register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_position = _register(_POSITIONS, "position encoding")
register_arrangement = _register(_ARRANGEMENTS, "arrangement")


def _build(table: Dict[str, type], what: str, spec: PartSpec):
    try:
        cls = table[spec.kind]
    except KeyError:
        raise KeyError(f"no {what} registered under {spec.kind!r}; known: "
                       + ", ".join(sorted(table))) from None
    return cls(spec)


def build_norm(spec: PartSpec) -> Norm:
    return _build(_NORMS, "norm", spec)


def build_mixer(spec: PartSpec) -> Mixer:
    return _build(_MIXERS, "mixer", spec)


def build_feed_forward(spec: PartSpec) -> FeedForward:
    return _build(_FEED_FORWARDS, "feed-forward", spec)


def build_position(spec: PartSpec) -> PositionEncoding:
    return _build(_POSITIONS, "position encoding", spec)


def build_arrangement(layer: LayerSpec) -> Arrangement:
    try:
        cls = _ARRANGEMENTS[layer.arrangement]
    except KeyError:
        raise KeyError(f"no arrangement registered under {layer.arrangement!r}; known: "
                       + ", ".join(sorted(_ARRANGEMENTS))) from None
    return cls(layer)
