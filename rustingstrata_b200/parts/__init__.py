from .spec import PartSpec, TensorNeed, LayerSpec, LayerCall, ModelSpec, CacheNeed, StateNeed
from .registry import register_part, unregister_part, part_class, registered_parts, CATEGORIES
from .base import (Runtime, HostBatch, CallInfo, LayerCallInfo, StepContext, Part, Mixer, FeedForward, Norm, PositionEncoding, Block)
# importing the modules registers the built-in parts
from . import (norm, position, attention, feed_forward, block, embedding, short_conv, recurrent, latent_attention,  # noqa: E402,F401
               experts, streams, conv_attention, talking_attention, state_mixers)
