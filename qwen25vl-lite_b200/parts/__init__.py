"""Parts a layer is put together from.  Importing this package registers the built-in kinds."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward,
                   KVCacheNeed, Mixer, Norm, Part, PositionEncoding, StateNeed, TensorSpec, build_part,
                   register_block, register_embedding, register_feed_forward, register_head, register_mixer,
                   register_norm, register_position_encoding)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registration)
from .position import prompt_positions  # noqa: F401
