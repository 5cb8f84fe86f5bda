from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, FeedForward,
                   FixedState, LayerSpec, Mixer, ModelSpec, Norm, PagedKV, Part, PartSpec, PositionEncoding,
                   ScheduleItem, TensorSpec, build_part, register_block, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm, register_position)
from . import attention, block, embedding, mlp, norms, rope  # noqa: F401  (register the built-in parts)
