"""Parts that layers are put together from: norms, position encodings, mixers,
feed-forwards, and their arrangement in a block."""
from .base import (KVRequest, KVView, LayerCache, LayerRun, LayerSpec, Part, PartSpec, StateRequest, ChunkRequest, Position,  # noqa: F401
                   StepInfo, WeightSpec, register_feed_forward, register_mixer, register_norm, register_position)
from . import norm, position, feed_forward, mixers  # noqa: F401  (registers the built-in parts)
from .block import Block  # noqa: F401
