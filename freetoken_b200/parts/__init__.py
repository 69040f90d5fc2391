"""Parts a layer is put together from; importing this package registers the built-in kinds."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, Embedding,
                   FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Segment, StepState, Workspace)
from . import (attention, block, delta, embedding, gla, latent_attention, mamba2, mlp, mlstm, moe, norm, rope,  # noqa: F401
               side_by_side, sparse_attention, tied_attention)  # (registration)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv",
           "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "Segment", "StepState",
           "Workspace"]
