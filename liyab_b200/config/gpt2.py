"""GPT-2: a dense pre-LayerNorm decoder with learned absolute positions, fused
query/key/value attention, an ungated GELU feed-forward and a tied output head.

The reference's row for it fixes LayerNorm, the tanh GELU and "no rotary"
(src/compat/architecture.cpp:81-88); sizes come from the file's metadata
(architecture.cpp:588-600, 699-708, 799-805, 975-985, 994-998, 1012-1022).  Here
the same facts are read from the keys of GPT-2's own config.json.  Two options
of that file have no counterpart in the reference and are wired onto the
per-layer attention scale: `scale_attn_weights` and
`scale_attn_by_inverse_layer_idx`; and `activation_function` may name the exact
(erf) GELU, which the reference implements beside the tanh form
(src/core/transformer.cpp:125-142).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Any, Dict, List, Mapping, Optional, Sequence

from ..status import invalid_model, unsupported
from .registry import Architecture, register_architecture
from .spec import (AttentionSpec, CheckpointTensor, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec,
                   ModelSpec, NormSpec, PositionSpec, RunEntry)

_ACTIVATIONS = {
    "gelu_new": "gelu_tanh",
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_fast": "gelu_tanh",
    "gelu": "gelu_erf",
}


def _int_key(raw: Mapping[str, Any], key: str, *, lo: int = 1, hi: int = 1 << 24, default: Any = None,
             aliases: Sequence[str] = ()) -> int:
    value = raw.get(key)
    for alias in aliases:
        if value is None:
            value = raw.get(alias)
    if value is None:
        value = default
    if isinstance(value, bool) or not isinstance(value, int) or not (lo <= value <= hi):
        raise invalid_model(f"missing or invalid {key} in config.json (got {value!r}, need an integer in [{lo}, {hi}])")
    return value


def _bool_key(raw: Mapping[str, Any], key: str, default: bool) -> bool:
    value = raw.get(key, default)
    if value is None:
        value = default
    if not isinstance(value, bool):
        raise invalid_model(f"invalid {key} in config.json (got {value!r}, need true or false)")
    return value


@dataclass(frozen=True)
class GPT2Config:
    n_layer: int
    n_embd: int
    n_head: int
    n_inner: int
    n_positions: int
    vocab_size: int
    layer_norm_epsilon: float
    activation_function: str
    scale_attn_weights: bool
    scale_attn_by_inverse_layer_idx: bool
    tie_word_embeddings: bool
    eos_token_id: Optional[int]
    bos_token_id: Optional[int]

    @staticmethod
    def parse(raw: Mapping[str, Any]) -> "GPT2Config":
        n_layer = _int_key(raw, "n_layer", aliases=("num_hidden_layers",))
        n_embd = _int_key(raw, "n_embd", aliases=("hidden_size",))
        n_head = _int_key(raw, "n_head", aliases=("num_attention_heads",))
        if n_embd % n_head != 0:
            raise invalid_model(f"invalid head dimensions: n_embd {n_embd} is not a multiple of n_head {n_head}")
        n_inner = _int_key(raw, "n_inner", default=4 * n_embd)
        n_positions = _int_key(raw, "n_positions", aliases=("n_ctx", "max_position_embeddings"))
        vocab_size = _int_key(raw, "vocab_size")
        eps = raw.get("layer_norm_epsilon", 1e-5)
        if isinstance(eps, bool) or not isinstance(eps, (int, float)) or not math.isfinite(eps) or eps < 0:
            raise invalid_model(f"invalid layer_norm_epsilon in config.json (got {eps!r}, need a finite number >= 0)")
        act = raw.get("activation_function", "gelu_new")
        if act not in _ACTIVATIONS:
            raise unsupported(f"activation_function {act!r} is not supported; supported: {', '.join(sorted(_ACTIVATIONS))}")
        if _bool_key(raw, "reorder_and_upcast_attn", False):
            # Only changes where the layer factor is applied in half precision;
            # scores are computed in 32-bit here either way.
            pass
        if raw.get("add_cross_attention"):
            raise unsupported("add_cross_attention is not supported")
        ids: List[Optional[int]] = []
        for key in ("eos_token_id", "bos_token_id"):
            v = raw.get(key)
            if v is not None and (isinstance(v, bool) or not isinstance(v, int) or not (0 <= v < vocab_size)):
                raise invalid_model(f"invalid {key} in config.json (got {v!r}, need an id below vocab_size {vocab_size})")
            ids.append(v)
        return GPT2Config(
            n_layer=n_layer, n_embd=n_embd, n_head=n_head, n_inner=n_inner, n_positions=n_positions,
            vocab_size=vocab_size, layer_norm_epsilon=float(eps), activation_function=act,
            scale_attn_weights=_bool_key(raw, "scale_attn_weights", True),
            scale_attn_by_inverse_layer_idx=_bool_key(raw, "scale_attn_by_inverse_layer_idx", False),
            tie_word_embeddings=_bool_key(raw, "tie_word_embeddings", True),
            eos_token_id=ids[0], bos_token_id=ids[1])

    # ---- what the framework asks of a configuration -------------------------

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["model_type"] = "gpt2"
        d["architectures"] = ["GPT2LMHeadModel"]
        return d

    def attention_scale(self, layer: int) -> float:
        """1/sqrt(head_dim) computed in float as the reference does
        (architecture.cpp:975-985), divided by (layer + 1) when the
        configuration asks for it."""
        scale = 1.0 / math.sqrt(self.head_dim) if self.scale_attn_weights else 1.0
        if self.scale_attn_by_inverse_layer_idx:
            scale /= float(layer + 1)
        return scale

    def model_spec(self) -> ModelSpec:
        d = self.n_embd
        layers = []
        for i in range(self.n_layer):
            norm = NormSpec(kind="layernorm", size=d, eps=self.layer_norm_epsilon, bias=True)
            layers.append(LayerSpec(
                arrangement="pre_norm",
                mixer_norm=norm,
                mixer=AttentionSpec(kind="attention", hidden=d, n_head=self.n_head, n_kv_head=self.n_head,
                                    head_dim=self.head_dim, scale=self.attention_scale(i), window=0, bias=True),
                ff_norm=norm,
                feed_forward=DenseFeedForwardSpec(kind="dense", hidden=d, inner=self.n_inner,
                                                  activation=_ACTIVATIONS[self.activation_function], bias=True)))
        return ModelSpec(
            architecture="gpt2",
            embedding=EmbeddingSpec(vocab_size=self.vocab_size, size=d),
            position=PositionSpec(kind="learned_absolute", size=d, max_positions=self.n_positions),
            layers=tuple(layers),
            run_order=tuple(RunEntry(layer=i, cache=i) for i in range(self.n_layer)),
            final_norm=NormSpec(kind="layernorm", size=d, eps=self.layer_norm_epsilon, bias=True),
            head=HeadSpec(vocab_size=self.vocab_size, size=d, tied=self.tie_word_embeddings, bias=False),
            max_positions=self.n_positions,
            eos_token_id=self.eos_token_id)

    def checkpoint_map(self) -> Mapping[str, CheckpointTensor]:
        """Parameter path -> tensor of the model file.  GPT-2's projections are
        stored [in, out] (the converter the reference relies on transposes them:
        docs/validation/models-stage1/converter-classic.patch:11-22); the engine
        keeps every matrix [out, in]."""
        d, ff, L = self.n_embd, self.n_inner, self.n_layer
        proj_std = 0.02 / math.sqrt(2.0 * L)
        m: Dict[str, CheckpointTensor] = {
            "embedding.weight": CheckpointTensor("wte.weight", (self.vocab_size, d), kind="table"),
            "position.weight": CheckpointTensor("wpe.weight", (self.n_positions, d), kind="table"),
            "final_norm.weight": CheckpointTensor("ln_f.weight", (d,), kind="vector", init=(1.0, 0.1)),
            "final_norm.bias": CheckpointTensor("ln_f.bias", (d,), kind="vector"),
        }
        if not self.tie_word_embeddings:
            m["head.weight"] = CheckpointTensor("lm_head.weight", (self.vocab_size, d))
        for i in range(L):
            p, h = f"layers.{i}.", f"h.{i}."
            m[p + "mixer_norm.weight"] = CheckpointTensor(h + "ln_1.weight", (d,), kind="vector", init=(1.0, 0.1))
            m[p + "mixer_norm.bias"] = CheckpointTensor(h + "ln_1.bias", (d,), kind="vector")
            m[p + "mixer.qkv.weight"] = CheckpointTensor(h + "attn.c_attn.weight", (d, 3 * d), transform="transpose")
            m[p + "mixer.qkv.bias"] = CheckpointTensor(h + "attn.c_attn.bias", (3 * d,), kind="vector")
            m[p + "mixer.out.weight"] = CheckpointTensor(h + "attn.c_proj.weight", (d, d), transform="transpose",
                                                         init=(0.0, proj_std))
            m[p + "mixer.out.bias"] = CheckpointTensor(h + "attn.c_proj.bias", (d,), kind="vector")
            m[p + "ff_norm.weight"] = CheckpointTensor(h + "ln_2.weight", (d,), kind="vector", init=(1.0, 0.1))
            m[p + "ff_norm.bias"] = CheckpointTensor(h + "ln_2.bias", (d,), kind="vector")
            m[p + "feed_forward.up.weight"] = CheckpointTensor(h + "mlp.c_fc.weight", (d, ff), transform="transpose")
            m[p + "feed_forward.up.bias"] = CheckpointTensor(h + "mlp.c_fc.bias", (ff,), kind="vector")
            m[p + "feed_forward.down.weight"] = CheckpointTensor(h + "mlp.c_proj.weight", (ff, d),
                                                                 transform="transpose", init=(0.0, proj_std))
            m[p + "feed_forward.down.bias"] = CheckpointTensor(h + "mlp.c_proj.bias", (d,), kind="vector")
        return m

    def ignored_tensors(self) -> Sequence[str]:
        """Tensors a GPT-2 file may hold that carry no weights: the causal-mask
        buffers (dropped by the converter, converter-classic.patch:14-19) and a
        stored copy of the tied head."""
        pats = [r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias"]
        if self.tie_word_embeddings:
            pats.append(r"lm_head\.weight")
        return pats

    def name_prefixes(self) -> Sequence[str]:
        """Prefixes a file may put before every tensor name."""
        return ("", "transformer.")


register_architecture(Architecture(name="gpt2", class_names=("GPT2LMHeadModel", "GPT2Model"), parse=GPT2Config.parse))
