from . import spec
from .base import (Block, FeedForward, Mixer, Norm, Part, PositionEncoding, StepContext,
                   build_block, build_feed_forward, build_mixer, build_norm, build_position,
                   register_block, register_feed_forward, register_mixer, register_norm,
                   register_position)
from .attention import AttentionMixer
from .block import PreNormBlock
from .feedforward import GatedMlp
from .norm import RmsNorm
from .position import Rope, inverse_frequencies

__all__ = ["spec", "Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
           "StepContext", "build_block", "build_feed_forward", "build_mixer", "build_norm",
           "build_position", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position", "AttentionMixer", "PreNormBlock", "GatedMlp",
           "RmsNorm", "Rope", "inverse_frequencies"]
