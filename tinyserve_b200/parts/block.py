"""A block arranges a mixer, a feed-forward and their norms.

"pre_norm" is tinyserve's decoder layer (serve.py:1177-1181): the stream travels as
(x, residual); each norm first adds x to the residual, then normalises it; the
sub-layer's output becomes the next x, so that r1 = r0 + mixer(norm1(r0)),
r2 = r1 + ffn(norm2(r1)).  Another arrangement is another class in ARRANGEMENTS.

The block also owns what lies below the parts' interfaces: a product may hand its result on
unfinished (split-K partial tiles, a product that has not run yet, rows without their norm
factor: ``kernels.ops``), and the kernel of the next norm or product finishes it.  That is
decided here, between built-in parts that say they can take part in it; every other part gets
and returns plain tensors."""
from __future__ import annotations

from ..config.model_config import LayerSpec
from ..kernels import ops
from .base import Part, build_feed_forward, build_mixer, build_norm


def add_and_norm(norm, x, residual, reader=None, rows=None, compute_dtype=None):
    """residual += x; returns norm(residual) for ``reader`` (a part, or None).  ``x`` is what a
    mixer or feed-forward returned: a tensor or one of ops' unfinished products.  A plain RMSNorm
    goes to the fused kernels, and a reader that only multiplies its input by a matrix
    (``accepts_scaled_rows``) may get rows without their norm factor; any other norm gets a
    finished tensor."""
    rms = norm.rms_parameters()
    if rms is None:
        return norm.add_forward(ops.materialize(x), residual, rows=rows)
    weight, eps = rms
    scaled_ok = rows is None and reader is not None and getattr(reader, "accepts_scaled_rows", False)
    return ops.add_rmsnorm(x, residual, weight, eps, compute_dtype or residual_compute_dtype(norm, x),
                           rows=rows, scaled_ok=scaled_ok)


def residual_compute_dtype(norm, x):
    dtype = getattr(norm, "compute_dtype", None)
    if dtype is None and x is not None:
        dtype = x.dtype
    return dtype


class PreNormBlock(Part):
    capturable = True

    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__()
        self.mixer = build_mixer(spec.mixer)
        self.ffn = build_feed_forward(spec.ffn)
        self.input_norm = build_norm(spec.norm, hidden_size)
        self.post_mixer_norm = build_norm(spec.norm, hidden_size)
        self._names = {
            "mixer": spec.name_of("mixer", self.mixer.tree_name),
            "ffn": spec.name_of("ffn", self.ffn.tree_name),
            "input_norm": spec.name_of("input_norm"),
            "post_mixer_norm": spec.name_of("post_mixer_norm"),
        }

    def children(self):
        n = self._names
        return {n["mixer"]: self.mixer, n["ffn"]: self.ffn, n["input_norm"]: self.input_norm,
                n["post_mixer_norm"]: self.post_mixer_norm}

    def forward(self, x, residual, ctx, call):
        """(x, residual) -> x of the next block; ``residual`` (32-bit) is updated in place.
        x is None for the first block: the residual then already holds the embeddings."""
        h = add_and_norm(self.input_norm, x, residual, self.mixer, compute_dtype=ctx.dtype)
        if not getattr(self.mixer, "accepts_scaled_rows", False):
            h = ops.materialize(h)
        x = self.mixer.forward(h, ctx, call)
        h = add_and_norm(self.post_mixer_norm, x, residual, self.ffn, compute_dtype=ctx.dtype)
        if not getattr(self.ffn, "accepts_scaled_rows", False):
            h = ops.materialize(h)
        return self.ffn.forward(h, ctx)


ARRANGEMENTS = {"pre_norm": PreNormBlock}


def build_block(spec: LayerSpec, hidden_size: int):
    if spec.arrangement not in ARRANGEMENTS:
        raise KeyError(f"block arrangement {spec.arrangement!r} is not registered")
    return ARRANGEMENTS[spec.arrangement](spec, hidden_size)
