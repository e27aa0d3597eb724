"""Layer parts: norm, position encoding, mixer, feed-forward, their arrangement in a block, and the
embedding and head at a model's two ends."""

from paged_kv_serving_b200.parts.attention import PagedAttention
from paged_kv_serving_b200.parts.base import (
    Block, CacheBinding, GroupView, IntArena, Normed, PagedKVRequest, ParamSpec, Part, StateRequest, StepContext,
)
from paged_kv_serving_b200.parts.block import PreNormBlock
from paged_kv_serving_b200.parts.feed_forward import SwiGLU
from paged_kv_serving_b200.parts.io import LinearHead, TokenEmbedding
from paged_kv_serving_b200.parts.norms import RMSNorm
from paged_kv_serving_b200.parts.position import NoPositionEncoding, PositionEncoding, RotaryEncoding

__all__ = [
    "Block", "CacheBinding", "GroupView", "IntArena", "LinearHead", "NoPositionEncoding", "Normed", "PagedAttention",
    "PagedKVRequest", "ParamSpec", "Part", "PositionEncoding", "PreNormBlock", "RMSNorm", "RotaryEncoding",
    "StateRequest", "StepContext", "SwiGLU", "TokenEmbedding",
]
