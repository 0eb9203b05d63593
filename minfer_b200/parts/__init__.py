"""The parts that ship with the library, registered under their kinds."""
from ..registry import register_part
from .attention import Attention
from .base import (Block, CacheRequest, CacheView, CallBinding, FeedForward, Mixer, Norm, Part,
                   PositionEncoding, StateRequest, StepContext)
from .block import PreNormBlock
from .linear import Linear
from .mlp import DenseMlp, GatedMlp
from .norm import RmsNorm
from .positions import LearnedPositions
from .rotary import NoPosition, Rotary
from .shift import TokenShift
from .sink_attention import SinkAttention

register_part("norm", "rms_norm", RmsNorm, replace=True)
register_part("position", "rotary", Rotary, replace=True)
register_part("position", "none", NoPosition, replace=True)
register_part("mixer", "attention", Attention, replace=True)
register_part("mixer", "sink_attention", SinkAttention, replace=True)
register_part("feed_forward", "gated_mlp", GatedMlp, replace=True)
register_part("feed_forward", "dense_mlp", DenseMlp, replace=True)
register_part("model", "learned_positions", LearnedPositions, replace=True)
register_part("block", "pre_norm", lambda layer, **options: PreNormBlock(layer, **options),
              replace=True)
