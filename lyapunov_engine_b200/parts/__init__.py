from . import (attention, base, block, differential_attention, embedding, feedforward, hyper,  # noqa: F401  (registers the kinds)
               latent_attention, moe, norm, rope, short_conv)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, INPUT_FILTERS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward,
                   InputFilter, register_input_filter,
                   KVNeed, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec, PositionEncoding, ResidualStream,
                   RunSpec, StateNeed, TensorDecl, register_block, register_embedding, register_feed_forward,
                   register_head, register_mixer, register_norm, register_position_encoding)
