"""Parts of a decoder and their registries; importing this package registers the built-in kinds."""

from .base import (BLOCKS, DeferredNorm, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block,
                   CacheBinding, Embedding, FeedForward, FollowNorm, GroupView, Head, Mixer, Norm, PagedKVNeed, PagedNeed, Part, PreparedNorm,
                   PositionEncoding, Registry, ResidualStream, Runtime, StateNeed, StepContext)
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401  (registration)
from .linear import Linear
