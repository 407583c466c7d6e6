from .base import CacheNeed, Part, StateNeed, WeightSpec
from .context import LaneView, StepContext, Workspace
from .registry import build_block, build_part, register_part, registered_parts
from . import attention, block, embedding, experts, feed_forward, hyper, latent, norm, position, recurrent, side  # registers the built-in parts
from .model import DecoderModel

__all__ = [
    "CacheNeed", "DecoderModel", "LaneView", "Part", "StateNeed", "StepContext", "WeightSpec", "Workspace",
    "build_block", "build_part", "register_part", "registered_parts",
]
