"""Parts a model is put together from; importing this package registers the built-in ones."""
from . import (adapters, attention, block, embedding, experts, feed_forward, gated_attention, head,  # noqa: F401
               latent_attention, linear_attention, mixer_pair, norm, recurrent, rotary, window_attention)
from .registry import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                       POSITION_ENCODINGS, STREAM_ADAPTERS, register_stream_adapter, BuildContext, WeightAccess, lookup, register_block,
                       register_embedding, register_feed_forward, register_head, register_mixer,
                       register_norm, register_position_encoding)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "STREAM_ADAPTERS", "register_stream_adapter",
           "BuildContext", "WeightAccess", "lookup", "register_block", "register_embedding",
           "register_feed_forward", "register_head", "register_mixer", "register_norm",
           "register_position_encoding"]
