from .base import (BLOCKS, CONNECTIONS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, Connection, FeedForward,
                   FixedState, LayerSpec, Mixer, ModelSpec, Norm, PagedKV, Part, PartSpec, PositionEncoding,
                   ScheduleItem, TensorSpec, build_part, register_block, register_connection, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm, register_position)
from . import (attention, block, connections, delta_rule, embedding, mlp, moe, norms, rope,  # noqa: F401
               talking_attention)                                                  # (register the built-in parts)
