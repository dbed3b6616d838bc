"""Interfaces of the parts a model is assembled from, and their registries.

A *part* is a mixer, a feed-forward, a norm or a position encoding.  It is built
from a ``PartSpec`` (a registered kind plus sizes and constants), declares the
tensors it needs as ``ParamSpec`` entries, and runs on a ``StepContext``.  A part
never sees a model configuration and does not know which model it is in; the
configuration class of an architecture only names part kinds and parameters.

Adding a part: subclass ``Mixer`` / ``FeedForward`` / ``Norm`` /
``PositionEncoding`` and call the matching ``register_*`` with a new kind name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

from ..config.model_config import PartSpec


@dataclass(frozen=True)
class Source:
    """A checkpoint tensor that fills rows [row_start, row_end) of a parameter."""

    name: str            # tensor name relative to the part's checkpoint path
    row_start: int
    row_end: int


@dataclass(frozen=True)
class ParamSpec:
    """One tensor of a part.

    role "matrix": operand of a matrix product, kept in the engine's dtype.
    role "vector": small per-channel tensor; kept in the engine's dtype, but a
    tensor that the checkpoint stores in 32-bit stays 32-bit.
    role "int_table": integer table, kept as int32.
    init: "normal" (N(0, 0.02)), "norm_weight" (1 + U(-0.1, 0.1)) or "zeros", used by
    the random-weights mode.  ``sources`` lists the checkpoint tensors that fill it
    (default: one tensor of the same name and shape).  ``interleave_halves`` = b > 0: after the
    sources are placed, the rows of the first and the second half alternate in blocks of b rows
    (first-half rows [0, b), second-half rows [0, b), first-half rows [b, 2b), ...).
    """

    shape: tuple
    role: str = "matrix"
    init: str = "normal"
    sources: tuple = ()
    interleave_halves: int = 0


def interleave_halves(tensor, block: int):
    """Rows of the two halves of ``tensor`` alternating in blocks of ``block`` rows."""
    rows = tensor.shape[0]
    if block <= 0:
        return tensor
    if rows % (2 * block):
        raise ValueError(f"{rows} rows do not split into two halves of blocks of {block}")
    return tensor.view(2, rows // (2 * block), block, *tensor.shape[1:]).transpose(0, 1).reshape(tensor.shape)


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token: ``kind`` "full" keeps every key, "window"
    only the last ``window``.  Calls whose specs are equal share a page pool."""

    kind: str
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer: one tensor of ``shape`` per slot."""

    shape: tuple
    dtype: str = "float32"


class Part:
    """Base of all parts: a checkpoint path, parameter specs, bound tensors."""

    #: name of the part inside its block in checkpoint tensor names
    tree_name = ""

    def __init__(self):
        self.path = ""
        self.w: dict = {}

    def param_specs(self) -> dict:
        return {}

    def children(self) -> dict:
        return {}

    def set_path(self, path: str) -> None:
        self.path = path
        for name, child in self.children().items():
            child.set_path(f"{path}.{name}" if path else name)

    def named_parts(self):
        yield self
        for child in self.children().values():
            yield from child.named_parts()

    def bind(self, tensors: dict) -> None:
        """Receive this part's tensors (local names) after loading."""
        self.w = tensors

    def prepare(self, runtime) -> None:
        """Build device-side constants (tables) once weights are bound."""


class Norm(Part):
    def forward(self, x, out=None):
        raise NotImplementedError

    #: add_forward takes ``scaled_ok`` (see there); a norm without it is never asked for it
    supports_scaled_rows = False

    def add_forward(self, x, residual, rows=None):
        """residual += x (x may be None), return norm(residual) in the compute dtype.  x is what
        a mixer or feed-forward returned: a tensor, or a ``kernels.ops.SplitPartials`` or
        ``PendingProduct`` (pass it to ops.add_rmsnorm as it is, or turn it into a tensor with
        ops.materialize).  A norm with ``supports_scaled_rows`` also takes ``scaled_ok``: when the
        block sets it, the part that reads the result hands it to ops.linear only, and the norm may
        return a ``kernels.ops.ScaledRows`` in place of a tensor."""
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    tree_name = "mixer"
    #: forward hands h to ops.linear only (never reads it itself), so h may be a ScaledRows
    accepts_scaled_rows = False

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, h, ctx, call):
        """h [T, hidden] in the compute dtype -> [T, hidden] (a tensor, or what ops.linear
        returned with allow_partials=True).  ``call`` is the
        ``BoundCall`` of the run order: its cache entry, state entry and
        ``writes_cache``."""
        raise NotImplementedError


class FeedForward(Part):
    tree_name = "mlp"
    accepts_scaled_rows = False       # as for a Mixer

    def forward(self, h, ctx):
        raise NotImplementedError


MIXERS: dict[str, Callable] = {}
FEED_FORWARDS: dict[str, Callable] = {}
NORMS: dict[str, Callable] = {}
POSITION_ENCODINGS: dict[str, Callable] = {}


def _register(table, what):
    def register(kind: str, factory: Callable) -> None:
        table[kind] = factory
    register.__doc__ = f"Register a {what} kind: factory(PartSpec-params..., dim) -> part."
    return register


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")


def _build(table, what, spec: PartSpec, **extra):
    if spec.kind not in table:
        raise KeyError(f"{what} kind {spec.kind!r} is not registered; known: {sorted(table)}")
    return table[spec.kind](**spec.params, **extra)


def build_mixer(spec: PartSpec):
    return _build(MIXERS, "mixer", spec)


def build_feed_forward(spec: PartSpec):
    return _build(FEED_FORWARDS, "feed-forward", spec)


def build_norm(spec: PartSpec, dim: int):
    return _build(NORMS, "norm", spec, dim=dim)


def build_position_encoding(spec: PartSpec):
    return _build(POSITION_ENCODINGS, "position encoding", spec)
