from .base import (Arrangement, Embedding, FeedForward, FixedState, Mixer, Norm, PagedKV, Part,
                   PositionEncoding, Precision, StreamShift, build_arrangement, build_embedding,
                   build_feed_forward, build_shift,
                   build_mixer, build_norm, build_position, register_arrangement,
                   register_embedding, register_feed_forward, register_mixer, register_norm,
                   register_position, register_shift)
from . import (attention, block, delta_rule, embedding, latent_attention, moe, norm, outnorm_block, rope,  # noqa: F401
               sandwich_block, shortconv, swiglu, token_shift)  # noqa: F401  (register the parts)

__all__ = [
    "Arrangement", "Embedding", "FeedForward", "FixedState", "Mixer", "Norm", "PagedKV", "Part",
    "PositionEncoding", "Precision", "StreamShift", "build_arrangement", "build_embedding", "build_shift", "build_feed_forward", "build_mixer",
    "build_norm", "build_position", "register_arrangement", "register_feed_forward",
    "register_mixer", "register_norm", "register_position", "register_embedding", "register_shift",
]
