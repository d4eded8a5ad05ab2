"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, connector, embedding, feed_forward, linear_attention, mixer_pair, norm, position, recurrent  # noqa: F401
from .base import (Block, Connector, DeferredUpdate, UpdateSum, WeightedRows, FeedForward, Mixer, Norm, Part, Position, as_tensor, build_block, build_part,
                   build_position, register_part, registered)

__all__ = ["Block", "Connector", "DeferredUpdate", "UpdateSum", "WeightedRows", "as_tensor", "FeedForward", "Mixer", "Norm", "Part", "Position", "build_block", "build_part",
           "build_position", "register_part", "registered"]
