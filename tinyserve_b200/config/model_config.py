"""Typed model configurations read from an architecture's own ``config.json`` keys.

A configuration class owns every size and constant of its architecture; no model
size stands anywhere else in the package.  ``LayerSpec``/``ModelSpec`` are the
architecture-neutral description that a configuration is turned into: which mixer,
feed-forward, norm and position encoding each layer has, and in which order layers
run.  Parts are built from specs, never from a configuration, so a part does not
know which model it is in.

Reference behaviour: tinyserve reads these keys through ``transformers.AutoConfig``
with ``getattr`` defaults scattered over its module constructors
(serve.py:819-831, 1205-1223, 1305).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that is missing a key, or holds a value the engine refuses."""


@dataclass(frozen=True)
class PartSpec:
    """Name of a registered part kind plus its constructor parameters."""

    kind: str
    params: dict = field(default_factory=dict)

    def get(self, key, default=None):
        return self.params.get(key, default)


#: names of a block's parts inside checkpoint tensor names; "mixer" and "ffn" default to the
#: part's own ``tree_name``
LAYER_NAMES = {"input_norm": "input_layernorm", "post_mixer_norm": "post_attention_layernorm"}
#: names of the model's own tensors and of its layers ("{i}" is the layer's index)
MODEL_NAMES = {"embed": "{prefix}embed_tokens", "layers": "{prefix}layers.{i}", "final_norm": "{prefix}norm",
               "lm_head": "lm_head", "embed_position": "{prefix}embed_positions"}


@dataclass(frozen=True)
class LayerSpec:
    """One block: its mixer, its feed-forward, the norm kind and the arrangement.  ``names``
    overrides entries of LAYER_NAMES (and "mixer" / "ffn"): how the block's parts are called in
    the checkpoint's tensor names."""

    mixer: PartSpec
    ffn: PartSpec
    norm: PartSpec
    arrangement: str = "pre_norm"
    names: dict = field(default_factory=dict)

    def name_of(self, key: str, default: str = "") -> str:
        return self.names.get(key, LAYER_NAMES.get(key, default))


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named twice: it then
    runs twice with the same weights).  ``cache`` names the cache entry that this
    call's mixer uses; two calls that name the same entry share it, and only the
    call with ``writes_cache`` stores keys and values there, so that a later call
    can read another layer's cache.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden_size: int
    layers: tuple
    order: tuple
    final_norm: PartSpec
    tie_word_embeddings: bool
    # prefix of every tensor name of the decoder stack in a checkpoint
    weight_prefix: str = "model."
    # overrides of MODEL_NAMES: the checkpoint's names of the embedding table, the layers
    # ("{i}" = index), the final norm and the output projection
    names: dict = field(default_factory=dict)
    # a position encoding that adds to the embeddings before the first block (learned or
    # absolute positions); None: positions enter inside the mixers only
    embedding_position: PartSpec = None

    def name_of(self, key: str, **fmt) -> str:
        return self.names.get(key, MODEL_NAMES[key]).format(prefix=self.weight_prefix, **fmt)


@dataclass(frozen=True)
class ModelConfig:
    """Base class: subclasses list their config.json keys as dataclass fields."""

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        raise NotImplementedError

    @classmethod
    def from_json(cls, path: str) -> "ModelConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as fh:
            return cls.from_dict(json.load(fh))

    def to_dict(self) -> dict:
        """config.json content that reads back to an equal configuration."""
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError


def _require(raw: dict, key: str, kind=None):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json has no '{key}'")
    value = raw[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json '{key}' must be an integer, got {value!r}")
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json '{key}' must be a number, got {value!r}")
        value = float(value)
    return value


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder (``Qwen3ForCausalLM``, ``model_type: qwen3``).

    Keys and defaults follow what tinyserve reads for this model type:
    head_dim defaults to hidden_size // num_attention_heads (serve.py:821),
    attention_bias to False (serve.py:824), tie_word_embeddings to False
    (serve.py:1209), rope_theta comes flat or from rope_parameters / rope_scaling
    with default 10000.0 and only rope_type "default" is accepted
    (serve.py:1218-1223); rms_norm_eps has no default (serve.py:1106).

    tinyserve ignores the sliding-window keys of this architecture and always
    attends to all keys.  Here they select, layer by layer, attention over a window
    of keys: with ``use_sliding_window`` set, layers with index >=
    ``max_window_layers`` (or those that ``layer_types`` marks
    "sliding_attention") see the last ``sliding_window`` keys only.  With
    ``use_sliding_window`` false (every published checkpoint) the model is the one
    tinyserve runs.
    """

    architecture: ClassVar[str] = "Qwen3ForCausalLM"

    vocab_size: int = 0
    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    max_position_embeddings: int = 0
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    layer_types: tuple = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        model_type = raw.get("model_type", "qwen3")
        if model_type != "qwen3":
            raise ConfigError(f"Qwen3Config reads model_type 'qwen3', got {model_type!r}")
        hidden = _require(raw, "hidden_size", int)
        heads = _require(raw, "num_attention_heads", int)
        kv_heads = raw.get("num_key_value_heads")
        if kv_heads is None:
            kv_heads = heads
        head_dim = raw.get("head_dim") or hidden // heads
        rope = raw.get("rope_parameters") or raw.get("rope_scaling") or {}
        rope_type = rope.get("rope_type", rope.get("type", "default"))
        if rope_type != "default":
            raise ConfigError(f"rope_type {rope_type!r} is not supported (only 'default')")
        theta = raw.get("rope_theta") or rope.get("rope_theta") or 10000.0
        layers = _require(raw, "num_hidden_layers", int)
        use_window = bool(raw.get("use_sliding_window", False))
        window = raw.get("sliding_window") or 0
        layer_types = tuple(raw.get("layer_types") or ())
        max_window_layers = raw.get("max_window_layers")
        if max_window_layers is None:
            max_window_layers = layers
        cfg = cls(
            vocab_size=_require(raw, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=int(kv_heads),
            head_dim=int(head_dim),
            intermediate_size=_require(raw, "intermediate_size", int),
            rms_norm_eps=_require(raw, "rms_norm_eps", float),
            rope_theta=float(theta),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            max_position_embeddings=int(raw.get("max_position_embeddings") or 0),
            use_sliding_window=use_window,
            sliding_window=int(window) if use_window else 0,
            max_window_layers=int(max_window_layers),
            layer_types=layer_types if use_window else (),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for f in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "intermediate_size"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"'{f}' must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError("'rms_norm_eps' must be positive")
        if self.use_sliding_window:
            if self.sliding_window <= 0:
                raise ConfigError("use_sliding_window is set but sliding_window is not positive")
            if self.layer_types and len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError("layer_types must name every layer")
            for t in self.layer_types:
                if t not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"unknown layer type {t!r}")

    def layer_window(self, i: int) -> int:
        """Window of layer ``i`` in keys; 0 = all keys."""
        if not self.use_sliding_window:
            return 0
        if self.layer_types:
            return self.sliding_window if self.layer_types[i] == "sliding_attention" else 0
        return self.sliding_window if i >= self.max_window_layers else 0

    def to_dict(self) -> dict:
        out: dict[str, Any] = {"architectures": [self.architecture], "model_type": "qwen3"}
        for f in fields(self):
            value = getattr(self, f.name)
            if f.name == "layer_types":
                if value:
                    out[f.name] = list(value)
                continue
            if f.name in ("sliding_window", "max_window_layers") and not self.use_sliding_window:
                continue
            out[f.name] = value
        return out

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"eps": self.rms_norm_eps})
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "bias": self.attention_bias,
                "qk_norm": PartSpec("rmsnorm", {"eps": self.rms_norm_eps}),
                "position": PartSpec("rotary", {"rotary_dim": self.head_dim,
                                                "theta": self.rope_theta,
                                                "pairing": "half"}),
                "window": self.layer_window(i),
                "scale": self.head_dim ** -0.5,
            })
            ffn = PartSpec("gated_mlp", {"hidden_size": self.hidden_size,
                                         "intermediate_size": self.intermediate_size,
                                         "activation": "silu"})
            layers.append(LayerSpec(mixer, ffn, norm))
        order = tuple(LayerCall(i, i) for i in range(self.num_hidden_layers))
        return ModelSpec(self.vocab_size, self.hidden_size, tuple(layers), order, norm,
                         self.tie_word_embeddings)
