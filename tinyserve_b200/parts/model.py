"""The decoder stack: embedding, blocks in a run order that is data, final norm, logits.

tinyserve's ``Model`` (serve.py:1195-1263): x = embed_tokens[ids]; the layers; the last
residual add with the final norm; logits = hidden @ W.T with W the embedding table when
``tie_word_embeddings`` else ``lm_head``.  Here only the rows whose logits are wanted go
through the final norm and the vocabulary projection, and logits are returned in 32-bit."""
from __future__ import annotations

from dataclasses import dataclass

from ..config.model_config import ModelSpec
from ..kernels import ops
from .base import CacheSpec, ParamSpec, Part, StateSpec, build_norm
from .block import build_block


class Embedding(Part):
    def __init__(self, vocab_size, hidden_size):
        super().__init__()
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}


class LMHead(Part):
    def __init__(self, vocab_size, hidden_size):
        super().__init__()
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}


@dataclass(frozen=True)
class BoundCall:
    """A run-order entry resolved against the model: which block runs, which cache
    entry and which state entry (-1: none) its mixer uses."""

    layer: int
    cache: int
    state: int
    writes_cache: bool


@dataclass(frozen=True)
class CacheEntryInfo:
    spec: CacheSpec
    group: int           # index into DecoderModel.cache_groups
    index_in_group: int


class DecoderModel(Part):
    def __init__(self, spec: ModelSpec):
        super().__init__()
        self.spec = spec
        self.vocab_size, self.hidden_size = spec.vocab_size, spec.hidden_size
        self.embed_tokens = Embedding(spec.vocab_size, spec.hidden_size)
        self.blocks = [build_block(layer, spec.hidden_size) for layer in spec.layers]
        self.norm = build_norm(spec.final_norm, spec.hidden_size)
        self.lm_head = None if spec.tie_word_embeddings else LMHead(spec.vocab_size, spec.hidden_size)
        prefix = spec.weight_prefix
        self.embed_tokens.set_path(prefix + "embed_tokens")
        for i, block in enumerate(self.blocks):
            block.set_path(f"{prefix}layers.{i}")
        self.norm.set_path(prefix + "norm")
        if self.lm_head is not None:
            self.lm_head.set_path("lm_head")
        self._resolve_order()

    # ------------------------------------------------------------------ structure
    def _resolve_order(self):
        spec = self.spec
        cache_ids, self.cache_entries, self.cache_groups = {}, [], []
        self.state_entries, self.calls = [], []
        group_sizes = []
        # first pass: a cache entry takes its geometry from the call that writes it
        writers = {}
        for call in spec.order:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"run order names layer {call.layer}, model has {len(self.blocks)}")
            if call.writes_cache:
                if call.cache in writers:
                    raise ValueError(f"cache entry {call.cache} is written by two calls")
                writers[call.cache] = call
        for call in spec.order:
            mixer = self.blocks[call.layer].mixer
            cspec = mixer.cache_spec()
            cache_index = -1
            if cspec is not None:
                if call.cache not in writers:
                    raise ValueError(f"cache entry {call.cache} is read but never written")
                wspec = self.blocks[writers[call.cache].layer].mixer.cache_spec()
                if (wspec.num_kv_heads, wspec.head_dim) != (cspec.num_kv_heads, cspec.head_dim):
                    raise ValueError(f"cache entry {call.cache}: reader and writer differ in geometry")
                if call.cache not in cache_ids:
                    if wspec not in self.cache_groups:
                        self.cache_groups.append(wspec)
                        group_sizes.append(0)
                    g = self.cache_groups.index(wspec)
                    cache_ids[call.cache] = len(self.cache_entries)
                    self.cache_entries.append(CacheEntryInfo(wspec, g, group_sizes[g]))
                    group_sizes[g] += 1
                cache_index = cache_ids[call.cache]
            sspec = mixer.state_spec()
            state_index = -1
            if sspec is not None:
                state_index = len(self.state_entries)
                self.state_entries.append(sspec)
            self.calls.append(BoundCall(call.layer, cache_index, state_index, call.writes_cache))
        self.group_sizes = group_sizes

    def children(self):
        out = {"embed_tokens": self.embed_tokens, "norm": self.norm}
        for i, block in enumerate(self.blocks):
            out[f"layers.{i}"] = block
        if self.lm_head is not None:
            out["lm_head"] = self.lm_head
        return out

    def named_parts(self):
        yield self.embed_tokens
        for block in self.blocks:
            yield from block.named_parts()
        yield self.norm
        if self.lm_head is not None:
            yield self.lm_head

    def prepare(self, runtime):
        for part in self.named_parts():
            part.prepare(runtime)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx):
        """Run this step's tokens; returns 32-bit logits [len(ctx.logit_rows), vocab]."""
        residual = ops.embed_lookup(self.embed_tokens.w["weight"], ctx.token_ids, ctx.slot_tokens)
        x = None
        for call in self.calls:
            x = self.blocks[call.layer].forward(x, residual, ctx, call)
        if ctx.num_logit_rows == 0:
            return None
        hidden = self.norm.add_forward(x, residual, rows=ctx.logit_rows)
        head = self.lm_head.w["weight"] if self.lm_head is not None else self.embed_tokens.w["weight"]
        return ops.linear(hidden, head, out_float32=True)
