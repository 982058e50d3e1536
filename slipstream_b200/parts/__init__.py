"""Parts a model is put together from; importing this package registers the built-in ones."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec,
                   Embedding, FeedForward, Head, IntoNorm, LayerBinding, Mixer, Norm, Part, PositionEncoding, Registry, Runtime,
                   StateSpec, WeightSpec)
from .attention import PagedAttention
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .mlp import SwiGLUFeedForward
from .norm import RMSNorm
from .rotary import NoPositionEncoding, RotaryEncoding

__all__ = ["BLOCKS", "EMBEDDINGS", "HEADS", "Embedding", "Head", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheSpec",
           "FeedForward", "IntoNorm", "LayerBinding", "Mixer", "Norm", "Part", "PositionEncoding", "Registry",
           "Runtime", "StateSpec", "WeightSpec", "PagedAttention", "PreNormBlock", "LMHead",
           "TokenEmbedding", "SwiGLUFeedForward", "RMSNorm", "NoPositionEncoding", "RotaryEncoding"]
