"""Parts a layer is put together from: norms, position encodings, mixers,
feed-forwards and their arrangement in a block."""
from .base import (Block, FeedForward, KVRequest, Mixer, Norm, ParamSpec, Part, PositionEncoding,
                   StateRequest, build_block, build_feed_forward, build_mixer, build_norm,
                   build_position, register_block, register_feed_forward, register_mixer,
                   register_norm, register_position)
from . import norms, position, attention, feedforward, block  # register the built-in kinds
from .block import AssembledBlock
