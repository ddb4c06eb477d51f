from .base import (Block, BuildEnv, CacheNeed, FeedForward, LayerCache, Mixer, Norm, Part,
                   PositionEncoding, ResidualStream, StateNeed, StepContext)
from .registry import build_part, part, part_class, register_part
from .spec import (AttentionSpec, BlockSpec, ModelSpec, PartSpec, RMSNormSpec, RopeSpec, ScheduleEntry,
                   SwiGLUSpec)
from . import norm, rope, attention, mlp, block  # noqa: F401  (register the built-in parts)
