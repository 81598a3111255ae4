from . import attention, block, ends, mlp, norm, rope    # register the built-in kinds
from .base import (CacheRequest, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Rotation, lookup,
                   register_block, register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                   register_position)
from .linear import Linear
from .runtime import Runtime
