"""Parts a layer is put together from; importing this package registers the built-in kinds."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, Embedding,
                   FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Segment, StepState, Workspace)
from . import (attention, block, embedding, gla, latent_attention, mlp, mlstm, moe, norm, rope, sparse_attention,  # noqa: F401
               tied_attention)  # (registration)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv",
           "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "Segment", "StepState",
           "Workspace"]
