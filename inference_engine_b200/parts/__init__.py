from . import (  # noqa: F401 (register)
    attention, block, delta_rule, embedding, feedforward, latent_attention, norm, position, routed,
)
from .base import (
    Block,
    BuildEnv,
    CacheBinding,
    FeedForward,
    Mixer,
    Norm,
    PagedKVRequest,
    Part,
    PositionEncoding,
    StateRequest,
    WeightDecl,
)
from .registry import build_part, register_part, registered_kinds

__all__ = [
    "Block", "BuildEnv", "CacheBinding", "FeedForward", "Mixer", "Norm", "PagedKVRequest",
    "Part", "PositionEncoding", "StateRequest", "WeightDecl", "build_part", "register_part",
    "registered_kinds",
]
