"""Parts a model is put together from.  Importing this package registers the built-in kinds."""
from . import registry
from .base import Linear, Runtime, StepContext, Workspace
from . import norm, position, attention, feedforward, block, embedding  # noqa: F401  (registration)
from .registry import (register_arrangement, register_embedding, register_feed_forward, register_head,
                       register_mixer, register_norm, register_position)
