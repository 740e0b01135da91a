"""Typed descriptions of a model, part by part.

A model is data before it is code: an architecture's configuration is turned
into a `ModelSpec`, a list of `LayerSpec`s (each naming its mixer, feed-forward
and norms by `kind` with their own sizes and constants) and a `run_order` that
says which layer runs when and whose cache it reads.  The parts registry
(`liyab_b200.parts.registry`) maps each `kind` to the class that implements it,
so a layer's parts are chosen layer by layer and no part knows the model it is in.

The reference keeps the same split: `ModelConfig` holds the global facts and a
`BlockPlan` per block holds n_head, n_head_kv, n_ff, head_dim, attn_scale, the
mixer and the feed-forward kind (src/compat/architecture.h:282-380, 452-630).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


@dataclass(frozen=True)
class PartSpec:
    """Base of every part description: `kind` selects the implementation."""
    kind: str


@dataclass(frozen=True)
class NormSpec(PartSpec):
    size: int = 0
    eps: float = 1e-5
    bias: bool = True


@dataclass(frozen=True)
class PositionSpec(PartSpec):
    """`learned_absolute`: a table of `max_positions` rows added to the embedding."""
    size: int = 0
    max_positions: int = 0


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    """Causal self-attention with one fused query/key/value projection.

    `scale` multiplies every query-key product (it already contains the
    1/sqrt(head_dim) factor and any per-layer factor).  `window` = 0 means a
    query sees every earlier key; w > 0 means the w latest keys (itself included).
    """
    hidden: int = 0
    n_head: int = 0
    n_kv_head: int = 0
    head_dim: int = 0
    scale: float = 1.0
    window: int = 0
    bias: bool = True


@dataclass(frozen=True)
class DenseFeedForwardSpec(PartSpec):
    """down(act(up(x))) without a gate; `activation` is gelu_tanh or gelu_erf."""
    hidden: int = 0
    inner: int = 0
    activation: str = "gelu_tanh"
    bias: bool = True


@dataclass(frozen=True)
class GenericSpec(PartSpec):
    """A part that is not built in (tests register toy parts with it)."""
    hidden: int = 0
    options: Mapping[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:  # options may hold unhashable values
        return hash((self.kind, self.hidden))


@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts, and how they are arranged around the residual."""
    arrangement: str                  # e.g. "pre_norm"
    mixer_norm: PartSpec
    mixer: PartSpec
    ff_norm: PartSpec
    feed_forward: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order.

    `layer` indexes `ModelSpec.layers` (a layer may be named twice: its weights
    are then used twice).  `cache` names the cache unit this run of the layer
    reads; when it equals the entry's own index in the run order the entry also
    writes that unit, otherwise it reads the keys and values that the entry
    numbered `cache` wrote (and writes none of its own).
    """
    layer: int
    cache: int


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    size: int
    scale: float = 1.0


@dataclass(frozen=True)
class HeadSpec:
    """The projection to the vocabulary; `tied` reuses the embedding table."""
    vocab_size: int
    size: int
    tied: bool = True
    bias: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    embedding: EmbeddingSpec
    position: PartSpec
    layers: Sequence[LayerSpec]
    run_order: Sequence[RunEntry]
    final_norm: PartSpec
    head: HeadSpec
    max_positions: int
    eos_token_id: Optional[int] = None

    @property
    def vocab_size(self) -> int:
        return self.embedding.vocab_size

    @property
    def hidden(self) -> int:
        return self.embedding.size


@dataclass(frozen=True)
class CheckpointTensor:
    """Where a parameter lives in the model file.

    `name` is the tensor's name in the file; `transform` is applied after
    reading: "none", or "transpose" for matrices stored [in, out].  `init` is
    (mean, std) for the random-weights mode.  `kind` decides the storage type
    in reduced precision: "matrix" and "table" are kept in the compute type,
    "vector" (norm gains, biases) always in 32-bit.
    """
    name: str
    shape: tuple            # shape in the file
    transform: str = "none"
    kind: str = "matrix"
    init: tuple = (0.0, 0.02)
