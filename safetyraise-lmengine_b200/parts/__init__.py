"""The parts a model is assembled from.  Importing the package registers the built-in kinds."""
from . import attention, block, feedforward, norm, position  # noqa: F401
from .base import (BLOCKS, Block, EMBEDDING, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, ROTATION,  # noqa: F401
                   CacheNeed, ModelContext, Rotation, Part, StepContext, Workspace, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position_encoding)
