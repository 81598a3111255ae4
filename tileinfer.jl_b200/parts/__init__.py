from . import attention, block, mlp, norm, rope          # register the built-in kinds
from .base import (CacheRequest, FeedForward, Mixer, Norm, Part, PositionEncoding, lookup, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)
from .linear import Linear
from .runtime import Runtime
