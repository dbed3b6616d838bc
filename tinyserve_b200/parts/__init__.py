from .base import (CacheSpec, CacheTensor, FeedForward, Mixer, Norm, ParamSpec, Part, PositionEncoding, Source,
                   StateSpec, build_feed_forward, build_mixer, build_norm,
                   build_position_encoding, register_feed_forward, register_mixer, register_norm,
                   register_position_encoding)
from .norm import RMSNorm
from .rotary import Rotary
from .attention import Attention
from .mlp import GatedMLP
from .block import ARRANGEMENTS, PreNormBlock, build_block
from .model import BoundCall, DecoderModel, Embedding, LMHead, build_model
