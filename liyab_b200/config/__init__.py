"""Typed configurations and the architecture registry."""
from .spec import (AttentionSpec, CheckpointTensor, DenseFeedForwardSpec, EmbeddingSpec, GenericSpec, HeadSpec,
                   LayerSpec, ModelSpec, NormSpec, PartSpec, PositionSpec, RunEntry)
from .registry import (Architecture, find_architecture, parse_config, read_config, register_architecture,
                       supported_architectures)
from .gpt2 import GPT2Config

__all__ = [
    "AttentionSpec", "CheckpointTensor", "DenseFeedForwardSpec", "EmbeddingSpec", "GenericSpec", "HeadSpec",
    "LayerSpec", "ModelSpec", "NormSpec", "PartSpec", "PositionSpec", "RunEntry", "Architecture",
    "find_architecture", "parse_config", "read_config", "register_architecture", "supported_architectures",
    "GPT2Config",
]
