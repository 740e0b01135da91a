"""Typed configuration and the architecture registry."""
import json

import pytest

from liyab_b200 import ErrorCode, LiyabError
from liyab_b200.config import describe_config, parse_config, read_config, slot, supported_architectures
from tiny_models import CONFIG_A, CONFIG_B


def test_gpt2_is_registered_and_parsed_from_its_own_keys():
    assert "gpt2" in supported_architectures()
    d = describe_config(CONFIG_B)
    cfg, spec = d["config"], d["spec"]
    assert d["architecture"] == "gpt2"
    assert (cfg["n_layer"], cfg["n_embd"], cfg["n_head"], cfg["n_inner"], cfg["vocab_size"], cfg["n_positions"]) == (3, 96, 3, 320, 1000, 256)
    assert cfg["layer_norm_epsilon"] == 1e-6
    assert len(spec["layers"]) == 3 and [e["layer"] for e in spec["run_order"]] == [0, 1, 2]
    assert [s["name"] for s in spec["layers"][0]["slots"]] == ["mixer_norm", "mixer", "ff_norm", "feed_forward"]
    assert slot(spec["layers"][0], "feed_forward")["activation"] == "gelu_erf"
    assert slot(spec["layers"][0], "mixer_norm")["eps"] == 1e-6 and slot(spec["layers"][0], "mixer")["head_dim"] == 32
    # per-layer attention factor: 1/sqrt(hd) / (layer + 1)
    scales = [slot(l, "mixer")["scale"] for l in spec["layers"]]
    assert scales == pytest.approx([32 ** -0.5, 32 ** -0.5 / 2, 32 ** -0.5 / 3])
    assert spec["head"]["tied"] and spec["max_positions"] == 256
    # the file's layout: GPT-2's matrices are stored [in, out] and transposed at load
    ck = d["checkpoint"]["layers.0.mixer.qkv.weight"]
    assert ck["sources"] == [{"name": "h.0.attn.c_attn.weight", "shape": [96, 288]}] and ck["transform"] == "transpose"


def test_class_name_selects_the_architecture_and_defaults_apply():
    d = describe_config({"architectures": ["GPT2LMHeadModel"], "n_layer": 1, "n_embd": 32, "n_head": 2,
                         "n_positions": 8, "vocab_size": 11, "n_inner": None})
    cfg = d["config"]
    assert cfg["n_inner"] == 128 and cfg["layer_norm_epsilon"] == 1e-5 and cfg["activation_function"] == "gelu_new"
    assert slot(d["spec"]["layers"][0], "mixer")["scale"] == pytest.approx(0.25)
    no_scale = describe_config({"model_type": "gpt2", "n_layer": 1, "n_embd": 32, "n_head": 2, "n_positions": 8,
                                "vocab_size": 11, "scale_attn_weights": False})
    assert slot(no_scale["spec"]["layers"][0], "mixer")["scale"] == 1.0


def test_unknown_architecture_lists_the_supported_ones():
    with pytest.raises(LiyabError) as e:
        parse_config({"model_type": "llama"})
    assert e.value.code == ErrorCode.UNSUPPORTED and "gpt2" in e.value.message and "llama" in e.value.message


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
    assert read_config(str(tmp_path))["config"]["n_embd"] == 64
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(LiyabError) as e:
        read_config(str(tmp_path))
    assert e.value.code == ErrorCode.INVALID_MODEL
    with pytest.raises(LiyabError) as e:
        read_config(str(tmp_path / "absent"))
    assert e.value.code == ErrorCode.IO_ERROR


def test_a_model_given_wholly_as_data_round_trips():
    """The description of a model (layers of named slots, run order, head) is data: what describe_config returns for
    GPT-2 can be handed back as a `liyab_spec` configuration and comes out unchanged."""
    spec = describe_config(CONFIG_A)["spec"]
    again = describe_config({"model_type": "liyab_spec", "spec": spec})
    assert again["spec"] == dict(spec, architecture="gpt2")
    assert "layers.1.feed_forward.down.weight" in again["checkpoint"]
    bad = json.loads(json.dumps(spec))
    bad["layers"][0]["slots"][1]["role"] = "mixing"
    with pytest.raises(LiyabError) as e:
        describe_config({"model_type": "liyab_spec", "spec": bad})
    assert e.value.code == ErrorCode.INVALID_MODEL and "mixing" in e.value.message
