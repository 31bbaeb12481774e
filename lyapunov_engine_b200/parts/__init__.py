from . import attention, base, block, embedding, feedforward, norm, rope  # noqa: F401  (registers the kinds)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward,
                   KVNeed, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, ResidualStream,
                   RunSpec, StateNeed, TensorDecl, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position_encoding)
