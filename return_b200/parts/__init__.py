"""Parts a decoder is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, mlp, norm, rope  # noqa: F401  (registration)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildEnv, FeedForward,
                   KVCacheNeed, KVView, LayerContext, Mixer, Norm, ParamSpec, Part, PositionEncoding, StateNeed)
from .spec import (AttentionSpec, BlockSpec, DecoderSpec, NormSpec, RopeSpec, ScheduleEntry, SwiGLUSpec)
