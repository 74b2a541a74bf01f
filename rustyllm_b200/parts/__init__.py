"""Parts a layer is put together from; importing the package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime  # noqa: F401
from .registry import (build_part, known, register, register_block, register_feed_forward,  # noqa: F401
                       register_mixer, register_norm, register_position)
