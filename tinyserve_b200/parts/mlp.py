"""Gated feed-forward (serve.py:908-919): down(act(gate(x)) * up(x)) with gate and up
as one fused projection (serve.py:911-912, 916).  Its rows alternate in blocks of 64, gate rows
then the matching up rows (when the width allows), so that a 128-row tile of the tcgen05 product
holds both and can apply the activation in its epilogue; the activation kernel reads the same
layout where the product is someone else's."""
from __future__ import annotations

from ..kernels import ops
from .base import FeedForward, ParamSpec, Source, register_feed_forward


DEFAULT_NAMES = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}


class GatedMLP(FeedForward):
    tree_name = "mlp"
    capturable = True

    def __init__(self, hidden_size, intermediate_size, activation="silu", names=None):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.ACTIVATIONS)}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.activation = activation
        self.block = ops.GATED_BLOCK if intermediate_size % ops.GATED_BLOCK == 0 else 0

    def param_specs(self):
        i, nm = self.intermediate_size, self.names
        return {
            "gate_up_proj.weight": ParamSpec((2 * i, self.hidden_size), sources=(
                Source(f"{nm['gate']}.weight", 0, i), Source(f"{nm['up']}.weight", i, 2 * i)),
                interleave_halves=self.block),
            "down_proj.weight": ParamSpec((self.hidden_size, i), sources=(
                Source(f"{nm['down']}.weight", 0, self.hidden_size),)),
        }

    accepts_scaled_rows = True

    def forward(self, h, ctx):
        act = ops.gated_linear(h, self.w["gate_up_proj.weight"], self.activation, self.block)
        return ops.linear(act, self.w["down_proj.weight"], allow_pending=True)


register_feed_forward("gated_mlp", GatedMLP)
