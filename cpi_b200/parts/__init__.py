from .base import (Part, Norm, Position, RotaryEncoding, ScoreBias, Mixer, FeedForward, Block, CacheView, build_part, registered,
                   register_norm, register_position, register_mixer, register_feed_forward, register_block)
from .workspace import Workspace
from . import norms, positions, attention, feedforward, block  # noqa: F401  (register the built-in kinds)
