"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""

from . import (attention, bigram, block, channel_delta, feed_forward, latent_attention, norms, rope,  # noqa: F401
               routed_experts)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildContext,  # noqa: F401
                   CacheNeeds, FeedForward, KVNeeds, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, ScheduleEntry, Stage, StateNeeds, TensorSpec)
