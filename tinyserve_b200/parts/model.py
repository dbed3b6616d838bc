"""The decoder stack: embedding, blocks in a run order that is data, final norm, logits.

tinyserve's ``Model`` (serve.py:1195-1263): x = embed_tokens[ids]; the layers; the last
residual add with the final norm; logits = hidden @ W.T with W the embedding table when
``tie_word_embeddings`` else ``lm_head``.  Here only the rows whose logits are wanted go
through the final norm and the vocabulary projection, and logits are returned in 32-bit."""
from __future__ import annotations

from dataclasses import dataclass

from ..config.model_config import ModelConfig, ModelSpec
from ..kernels import ops
from .base import CacheSpec, ParamSpec, Part, StateSpec, build_norm, build_position_encoding
from .block import add_and_norm, build_block


class Embedding(Part):
    capturable = True

    def __init__(self, vocab_size, hidden_size):
        super().__init__()
        self.vocab_size, self.hidden_size = vocab_size, hidden_size

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}


class LMHead(Part):
    capturable = True

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
        self.embed_position = (build_position_encoding(spec.embedding_position)
                               if spec.embedding_position is not None else None)
        # checkpoint names are data of the specification
        self.embed_tokens.set_path(spec.name_of("embed"))
        for i, block in enumerate(self.blocks):
            block.set_path(spec.name_of("layers", i=i))
        self.norm.set_path(spec.name_of("final_norm"))
        if self.lm_head is not None:
            self.lm_head.set_path(spec.name_of("lm_head"))
        if self.embed_position is not None:
            self.embed_position.set_path(spec.name_of("embed_position"))
        self._resolve_order()
        #: every part allows a captured graph of its forward pass to be replayed
        self.capturable = all(part.capturable for part in self.named_parts())

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
                if wspec.tensors != cspec.tensors:
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

    def named_parts(self):
        yield self.embed_tokens
        if self.embed_position is not None:
            yield from self.embed_position.named_parts()
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
        if self.embed_position is not None:
            self.embed_position.add_to_embeddings(residual, ctx)
        x = None
        for call in self.calls:
            x = self.blocks[call.layer].forward(x, residual, ctx, call)
        if ctx.num_logit_rows == 0:
            return None
        hidden = add_and_norm(self.norm, x, residual, rows=ctx.logit_rows, compute_dtype=ctx.dtype)
        head = self.lm_head.w["weight"] if self.lm_head is not None else self.embed_tokens.w["weight"]
        return ops.linear(hidden, head, out_float32=True)


def build_model(config: ModelConfig) -> DecoderModel:
    """From an architecture's configuration to a model made of parts: the configuration names
    the parts, layer by layer, and the run order; nothing else of it reaches the parts."""
    return DecoderModel(config.model_spec())
