"""Grouped-query attention over a paged cache (serve.py:816-906).

One fused projection for q, k and v (rows q heads, k heads, v heads: serve.py:827-828),
optional per-head norm of q and k before the position encoding (serve.py:873-876),
keys and values written to the cache pages of this step's tokens (serve.py:897-904),
attention of every query over its request's cached keys with j <= position and,
with ``window`` > 0, j > position - window (serve.py:668-680), output projection
(serve.py:883).  All sizes are parameters."""
from __future__ import annotations

from ..kernels import ops
from .base import (CacheSpec, Mixer, ParamSpec, Source, build_norm, build_position_encoding,
                   register_mixer)


class Attention(Mixer):
    tree_name = "self_attn"

    def __init__(self, hidden_size, num_heads, num_kv_heads, head_dim, bias=False, qk_norm=None,
                 position=None, window=0, scale=None):
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.bias, self.window = head_dim, bool(bias), int(window or 0)
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.q_norm = build_norm(qk_norm, head_dim) if qk_norm is not None else None
        self.k_norm = build_norm(qk_norm, head_dim) if qk_norm is not None else None
        self.position = build_position_encoding(position) if position is not None else None
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim

    def children(self):
        out = {}
        if self.q_norm is not None:
            out["q_norm"], out["k_norm"] = self.q_norm, self.k_norm
        if self.position is not None:
            out["position"] = self.position
        return out

    def param_specs(self):
        q, kv = self.q_size, self.kv_size
        rows = (("q_proj", 0, q), ("k_proj", q, q + kv), ("v_proj", q + kv, q + 2 * kv))
        specs = {
            "qkv_proj.weight": ParamSpec((q + 2 * kv, self.hidden_size), sources=tuple(
                Source(f"{n}.weight", a, b) for n, a, b in rows)),
            "o_proj.weight": ParamSpec((self.hidden_size, q)),
        }
        if self.bias:
            specs["qkv_proj.bias"] = ParamSpec((q + 2 * kv,), role="matrix", init="zeros", sources=tuple(
                Source(f"{n}.bias", a, b) for n, a, b in rows))
        return specs

    def cache_spec(self):
        kind = "window" if self.window > 0 else "full"
        return CacheSpec(kind, self.num_kv_heads, self.head_dim, self.window)

    accepts_scaled_rows = True

    def forward(self, h, ctx, call):
        qkv = ops.linear(h, self.w["qkv_proj.weight"], self.w.get("qkv_proj.bias"), allow_partials=True)
        cache = ctx.cache(call.cache)
        view = ctx.group(cache.group)
        out = ops.attention_from_qkv(
            qkv, ctx.positions, self.num_heads, self.num_kv_heads, self.head_dim, self.position,
            self.q_norm.w["weight"] if self.q_norm is not None else None,
            self.k_norm.w["weight"] if self.k_norm is not None else None,
            self.q_norm.eps if self.q_norm is not None else 0.0,
            cache.k, cache.v, view, ctx, self.scale, self.window, write_cache=call.writes_cache)
        return ops.linear(out.view(out.shape[0], self.q_size), self.w["o_proj.weight"], allow_pending=True)


register_mixer("attention", Attention)
