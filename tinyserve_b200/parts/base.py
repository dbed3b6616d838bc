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
class CacheTensor:
    """One tensor that a mixer keeps per token: ``heads`` vectors of ``width`` elements."""

    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token, in pages: ``kind`` "full" keeps every token, "window" only
    the last ``window``; ``tensors`` lists what is kept (attention: keys and values of
    ``num_kv_heads`` heads of ``head_dim``, which is the default; a mixer that caches one latent
    vector per token lists that alone).  Calls whose specs are equal share a page pool."""

    kind: str
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    tensors: tuple = ()

    def __post_init__(self):
        if not self.tensors:
            object.__setattr__(self, "tensors", (CacheTensor("k", self.num_kv_heads, self.head_dim),
                                                 CacheTensor("v", self.num_kv_heads, self.head_dim)))
        names = [t.name for t in self.tensors]
        if len(set(names)) != len(names) or any(t.heads <= 0 or t.width <= 0 for t in self.tensors):
            raise ValueError(f"cache tensors need distinct names and positive sizes: {self.tensors}")

    def elements_per_token(self) -> int:
        return sum(t.heads * t.width for t in self.tensors)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer: one tensor of ``shape`` per slot."""

    shape: tuple
    dtype: str = "float32"


class Part:
    """Base of all parts: a checkpoint path, parameter specs, bound tensors."""

    #: name of the part inside its block in checkpoint tensor names (a LayerSpec may override it)
    tree_name = ""
    #: True if ``forward`` reads nothing on the host that changes from step to step (everything
    #: it needs of the batch comes from the device tensors of the StepContext), so that a captured
    #: CUDA graph of it can be replayed.  A part that reads ``ctx.host`` leaves it False; a model
    #: with such a part is never captured.
    capturable = False

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
    """y = norm(x) over the last dimension.  ``forward`` and ``add_forward`` get and return plain
    tensors; which kernels fuse a norm with the products around it is decided below this
    interface (a norm that is exactly x * rsqrt(mean(x^2) + eps) * weight says so with
    ``rms_parameters`` and the block then uses the fused kernels)."""

    def forward(self, x, out=None):
        raise NotImplementedError

    def add_forward(self, x, residual, rows=None):
        """residual (float32, in place) += x (a tensor of the compute dtype, or None); returns
        norm(residual) in the compute dtype.  With ``rows`` (int32) only those rows are normalised
        and returned, and the residual is left as it is."""
        raise NotImplementedError

    def rms_parameters(self):
        """(weight, eps) if this norm is a plain RMSNorm, else None."""
        return None


class PositionEncoding(Part):
    """Where positions enter.  Inside a mixer: the attention part hands its position encoding to
    the fused q/k kernel, which reads ``rotary_dim``, ``interleaved``, ``cos`` and ``sin`` off it.
    At the embeddings (``ModelSpec.embedding_position``): ``add_to_embeddings`` is called once per
    step, after the lookup and before the first block."""

    def add_to_embeddings(self, residual, ctx) -> None:
        """residual float32 [T, hidden] (in place) += this encoding of ``ctx.positions``."""


class Mixer(Part):
    tree_name = "mixer"
    #: forward hands h to ops.linear only (never reads it itself), so h may be a ScaledRows
    accepts_scaled_rows = False

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def work_tile_queries(self, dtype, page_size: int) -> int:
        """Queries per block of the attention work lists this mixer will ask for
        (``kernels.ops.attention_work``) in steps that bring prompt portions, or 0.  The step
        function then packs those lists with the step's other inputs."""
        return 0

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
