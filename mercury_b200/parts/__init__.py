"""The parts a model is put together from; importing this package registers the built-in
kinds."""

from .base import (  # noqa: F401
    CacheNeed,
    Embedding,
    FeedForward,
    Head,
    LayerCache,
    Mixer,
    Norm,
    Part,
    PartSetup,
    PartSpec,
    PositionEncoding,
    StateNeed,
    TensorSpec,
    build_part,
    register_arrangement,
    register_embedding,
    register_head,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_position_encoding,
)
from . import attention, block, embedding, feedforward, norm, rotary  # noqa: F401,E402
