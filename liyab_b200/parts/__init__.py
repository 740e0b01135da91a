"""The parts a model is put together from, and their registries."""
from .registry import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, PartRegistry
from .base import CacheUnit, GroupView, Runtime, StepContext, Workspace
from .linear import Linear
from .norm import LayerNorm
from .position import LearnedAbsolutePosition, NoPosition
from .attention import CausalSelfAttention
from .feed_forward import DenseFeedForward
from .block import LayerParts, PreNormBlock

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "PartRegistry", "CacheUnit", "GroupView",
           "Runtime", "StepContext", "Workspace", "Linear", "LayerNorm", "LearnedAbsolutePosition", "NoPosition",
           "CausalSelfAttention", "DenseFeedForward", "LayerParts", "PreNormBlock"]
