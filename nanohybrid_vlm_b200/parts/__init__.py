from . import (attention, block, delta_rule, embedding, feed_forward, mlstm, moe, norm, parallel_mixer, position,  # noqa: F401
               sink_attention, state_space)    # (importing registers the built-in parts)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, CacheView, CompositeNeed,
                   Embedding,
                   FeedForward, FixedStateNeed, Head, Mixer, Norm, PagedKVNeed, Part, Pending, PositionEncoding)
from .spec import LayerRun, LayerSpec, ModelSpec, ParamDecl, PartSpec, PartUse, Source, part

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv", "CacheView", "CompositeNeed",
           "Embedding", "FeedForward", "FixedStateNeed", "Head", "Mixer", "Norm", "PagedKVNeed", "Part", "Pending", "PositionEncoding",
           "LayerRun", "LayerSpec", "ModelSpec", "ParamDecl", "PartSpec", "PartUse", "Source", "part"]
