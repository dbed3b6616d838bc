"""Grouped-query attention over a paged cache (serve.py:816-906).

One fused projection for q, k and v (rows q heads, k heads, v heads: serve.py:827-828),
optional per-head norm of q and k before the position encoding (serve.py:873-876),
keys and values written to the cache pages of this step's tokens (serve.py:897-904),
attention of every query over its request's cached keys with j <= position and,
with ``window`` > 0, j > position - window (serve.py:668-680), output projection
(serve.py:883).  All sizes are parameters, and so are the checkpoint's names of the four
projections and the two norms (``names``)."""
from __future__ import annotations

from ..kernels import ops
from .base import (CacheSpec, Mixer, ParamSpec, Source, build_norm, build_position_encoding,
                   register_mixer)


DEFAULT_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "q_norm": "q_norm", "k_norm": "k_norm"}


class Attention(Mixer):
    tree_name = "self_attn"
    capturable = True

    def __init__(self, hidden_size, num_heads, num_kv_heads, head_dim, bias=False, qk_norm=None,
                 position=None, window=0, scale=None, names=None):
        super().__init__()
        self.names = dict(DEFAULT_NAMES, **(names or {}))
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
            out[self.names["q_norm"]], out[self.names["k_norm"]] = self.q_norm, self.k_norm
        if self.position is not None:
            out["position"] = self.position
        return out

    def param_specs(self):
        q, kv = self.q_size, self.kv_size
        nm = self.names
        rows = ((nm["q"], 0, q), (nm["k"], q, q + kv), (nm["v"], q + kv, q + 2 * kv))
        specs = {
            "qkv_proj.weight": ParamSpec((q + 2 * kv, self.hidden_size), sources=tuple(
                Source(f"{n}.weight", a, b) for n, a, b in rows)),
            "o_proj.weight": ParamSpec((self.hidden_size, q), sources=(Source(f"{nm['o']}.weight", 0, self.hidden_size),)),
        }
        if self.bias:
            # drawn like a matrix in the random-weights mode: a bias of zeros would hide a fault
            specs["qkv_proj.bias"] = ParamSpec((q + 2 * kv,), role="matrix", init="normal", sources=tuple(
                Source(f"{n}.bias", a, b) for n, a, b in rows))
        return specs

    def cache_spec(self):
        kind = "window" if self.window > 0 else "full"
        return CacheSpec(kind, self.num_kv_heads, self.head_dim, self.window)

    accepts_scaled_rows = True

    def work_tile_queries(self, dtype, page_size):
        return ops.prefill_tile_queries(dtype, self.num_heads, self.num_kv_heads, self.head_dim, page_size)

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
