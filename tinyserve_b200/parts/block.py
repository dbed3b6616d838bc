"""A block arranges a mixer, a feed-forward and their norms.

"pre_norm" is tinyserve's decoder layer (serve.py:1177-1181): the stream travels as
(x, residual); each norm first adds x to the residual, then normalises it; the
sub-layer's output becomes the next x, so that r1 = r0 + mixer(norm1(r0)),
r2 = r1 + ffn(norm2(r1)).  Another arrangement is another class in ARRANGEMENTS."""
from __future__ import annotations

from ..config.model_config import LayerSpec
from .base import Part, build_feed_forward, build_mixer, build_norm


class PreNormBlock(Part):
    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__()
        self.mixer = build_mixer(spec.mixer)
        self.ffn = build_feed_forward(spec.ffn)
        self.input_norm = build_norm(spec.norm, hidden_size)
        self.post_mixer_norm = build_norm(spec.norm, hidden_size)

    def children(self):
        return {self.mixer.tree_name: self.mixer, self.ffn.tree_name: self.ffn,
                "input_layernorm": self.input_norm,
                "post_attention_layernorm": self.post_mixer_norm}

    def forward(self, x, residual, ctx, call):
        """(x, residual) -> x of the next block; ``residual`` (32-bit) is updated in place.
        x is None for the first block: the residual then already holds the embeddings."""
        h = self._norm(self.input_norm, x, residual, self.mixer)
        h = self._norm(self.post_mixer_norm, self.mixer.forward(h, ctx, call), residual, self.ffn)
        return self.ffn.forward(h, ctx)

    @staticmethod
    def _norm(norm, x, residual, reader):
        # a reader that only multiplies h by a matrix may get rows without their norm factor
        if norm.supports_scaled_rows and reader.accepts_scaled_rows:
            return norm.add_forward(x, residual, scaled_ok=True)
        return norm.add_forward(x, residual)


ARRANGEMENTS = {"pre_norm": PreNormBlock}


def build_block(spec: LayerSpec, hidden_size: int):
    if spec.arrangement not in ARRANGEMENTS:
        raise KeyError(f"block arrangement {spec.arrangement!r} is not registered")
    return ARRANGEMENTS[spec.arrangement](spec, hidden_size)
