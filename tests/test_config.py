"""Typed configuration and the architecture registry."""
import json

import pytest

from liyab_b200 import ErrorCode, LiyabError
from liyab_b200.config import GPT2Config, parse_config, read_config, supported_architectures
from tiny_models import CONFIG_A, CONFIG_B


def test_gpt2_is_registered_and_parsed_from_its_own_keys():
    assert "gpt2" in supported_architectures()
    cfg = parse_config(CONFIG_B)
    assert isinstance(cfg, GPT2Config)
    assert (cfg.n_layer, cfg.n_embd, cfg.n_head, cfg.n_inner, cfg.vocab_size, cfg.n_positions) == (3, 96, 3, 320, 1000, 256)
    assert cfg.head_dim == 32 and cfg.layer_norm_epsilon == 1e-6
    spec = cfg.model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    assert spec.layers[0].feed_forward.activation == "gelu_erf"
    assert spec.layers[0].mixer_norm.eps == 1e-6
    # per-layer attention factor: 1/sqrt(hd) / (layer + 1)
    scales = [l.mixer.scale for l in spec.layers]
    assert scales == pytest.approx([32 ** -0.5, 32 ** -0.5 / 2, 32 ** -0.5 / 3])
    assert spec.head.tied and spec.max_positions == 256


def test_class_name_selects_the_architecture_and_defaults_apply():
    cfg = parse_config({"architectures": ["GPT2LMHeadModel"], "n_layer": 1, "n_embd": 32, "n_head": 2,
                        "n_positions": 8, "vocab_size": 11, "n_inner": None})
    assert cfg.n_inner == 128 and cfg.layer_norm_epsilon == 1e-5 and cfg.activation_function == "gelu_new"
    assert cfg.model_spec().layers[0].mixer.scale == pytest.approx(0.25)
    no_scale = parse_config({"model_type": "gpt2", "n_layer": 1, "n_embd": 32, "n_head": 2, "n_positions": 8,
                             "vocab_size": 11, "scale_attn_weights": False})
    assert no_scale.model_spec().layers[0].mixer.scale == 1.0


def test_unknown_architecture_lists_the_supported_ones():
    with pytest.raises(LiyabError) as e:
        parse_config({"model_type": "llama"})
    assert e.value.code == ErrorCode.UNSUPPORTED and "gpt2" in e.value.message


@pytest.mark.parametrize("patch,needle", [
    ({"n_layer": 0}, "n_layer"), ({"n_embd": None}, "n_embd"), ({"n_head": 5}, "n_head"),
    ({"layer_norm_epsilon": -1.0}, "layer_norm_epsilon"), ({"vocab_size": "many"}, "vocab_size"),
    ({"eos_token_id": 512}, "eos_token_id"), ({"scale_attn_weights": 1}, "scale_attn_weights")])
def test_errors_name_the_key(patch, needle):
    raw = dict(CONFIG_A)
    raw.update(patch)
    with pytest.raises(LiyabError) as e:
        parse_config(raw)
    assert e.value.code == ErrorCode.INVALID_MODEL and needle in e.value.message


def test_unsupported_activation():
    raw = dict(CONFIG_A, activation_function="relu")
    with pytest.raises(LiyabError) as e:
        parse_config(raw)
    assert e.value.code == ErrorCode.UNSUPPORTED


def test_read_config_from_a_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CONFIG_A))
    assert read_config(str(tmp_path)).n_embd == 64
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(LiyabError):
        read_config(str(tmp_path))
    with pytest.raises(LiyabError) as e:
        read_config(str(tmp_path / "absent"))
    assert e.value.code == ErrorCode.IO_ERROR
