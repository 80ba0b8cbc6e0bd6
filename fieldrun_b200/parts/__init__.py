"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""
from . import addition, attention, block, connector, embedding, feed_forward, latent_attention, linear_attention, mixer_pair, norm, position, recurrent  # noqa: F401
from .base import (Addition, Block, Connector, DeferredUpdate, UpdateSum, WeightedRows, FeedForward, Mixer, Norm, Part, Position, as_tensor, build_block, build_part,
                   build_position, register_part, registered)

__all__ = ["Addition", "Block", "Connector", "DeferredUpdate", "UpdateSum", "WeightedRows", "as_tensor", "FeedForward", "Mixer", "Norm", "Part", "Position", "build_block", "build_part",
           "build_position", "register_part", "registered"]
