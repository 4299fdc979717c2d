"""Parts of a layer: norm, position encoding, mixer, feed-forward and their arrangement."""
from .base import (FeedForward, Mixer, Norm, Part, PositionEncoding, Runtime, StepContext, part_class,
                   register_arrangement, register_feed_forward, register_mixer, register_norm, register_position)
from .linear import Linear
from .norm import RMSNorm
from .position import RotaryPosition, rotary_inverse_frequencies
from .attention import AttentionMixer
from .swiglu import SwiGLUFeedForward
from .block import PreNormBlock

__all__ = ["FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "StepContext", "part_class",
           "register_arrangement", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "Linear", "RMSNorm", "RotaryPosition", "rotary_inverse_frequencies",
           "AttentionMixer", "SwiGLUFeedForward", "PreNormBlock"]
