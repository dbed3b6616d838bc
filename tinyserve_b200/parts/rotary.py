"""Rotary position encoding.  Tables as tinyserve builds them (serve.py:1225-1228):
inv_freq and angles in float64, cos and sin stored in float32, one row per absolute
position up to the engine's max_model_len (serve.py:1621).  ``pairing`` "half"
rotates (i, i + rotary_dim/2) as serve.py:811-814 does; "interleaved" rotates
(2i, 2i+1).  ``rotary_dim`` may be smaller than the head size (partial rotary); the
other dimensions pass through."""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding

class Rotary(PositionEncoding):
    capturable = True

    def __init__(self, rotary_dim: int, theta: float, pairing: str = "half"):
        super().__init__()
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.rotary_dim = rotary_dim
        self.theta = float(theta)
        self.interleaved = pairing == "interleaved"
        self.cos = self.sin = None

    @staticmethod
    def tables(rotary_dim, theta, num_positions):
        inv_freq = 1.0 / theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)
        freqs = torch.outer(torch.arange(num_positions, dtype=torch.float64), inv_freq)
        return freqs.cos().float(), freqs.sin().float()

    def prepare(self, runtime):
        # one table per (sizes, base) and engine: the layers of a model share it
        key = ("rotary", self.rotary_dim, self.theta)
        if key not in runtime.shared:
            cos, sin = self.tables(self.rotary_dim, self.theta, runtime.max_positions)
            runtime.shared[key] = (cos.to(runtime.device).contiguous(), sin.to(runtime.device).contiguous())
        self.cos, self.sin = runtime.shared[key]


register_position_encoding("rotary", Rotary)
