from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheRequest, EMBED_ADDS, EmbedAdd, FeedForward, LayerCache,
                   Mixer, Norm, Part, PositionEncoding, PostNormed, Runtime, ScaledSum, make_part, register_block, register_feed_forward,
                   register_embed_add, register_mixer, register_norm, register_position_encoding, to_f32, to_operand)
from . import norm, position, embedding, attention, latent_attention, ssm, delta, retention, ffn, side, block   # noqa: F401  (register the built-in parts)
